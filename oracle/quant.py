"""FP8 KV-cache records (656 bytes per token, and the 584-byte "MODEL1" form) : CPU restatement of the
reference's quantiser / de-quantiser.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Record layout (flash_mla/flash_mla_interface.py:92-98, tests/quant.py:35-53):
  bytes   0..511  512 x float8_e4m3fn   "NoPE" part, quantised per 128-value group
  bytes 512..527  4 x float32           one scale per group (x = fp8 * scale)
  bytes 528..655  64 x bfloat16         "RoPE" part, stored unquantised
"""
import torch

D_QK, D_NOPE, D_ROPE, GROUP, NUM_GROUPS = 576, 512, 64, 128, 4
BYTES_PER_TOKEN = D_NOPE + 4 * NUM_GROUPS + 2 * D_ROPE     # 656


def quantize_v32(blocked_k: torch.Tensor, pow2_scale: bool, pad_rows: int = 1) -> torch.Tensor:
    """Restates quantize_k_cache, V32 branch (tests/quant.py:20-53).
    blocked_k [num_blocks, block_size, 1, 576] bf16 -> [num_blocks, block_size, 1, 656] float8_e4m3fn
    view of a buffer with `pad_rows` spare rows per block (the reference allocates block_size+1 rows,
    :37, so stride(0) != block_size*656).
    pow2_scale=True reproduces the reference's rounding of the scale up to a power of two
    (_cast_scale_inv_to_ue8m0, :17-18); False keeps scale = amax/448 as an fp32 number."""
    nb, bs, h_k, d = blocked_k.shape
    assert h_k == 1 and d == D_QK
    x = blocked_k.squeeze(2)
    res = torch.empty((nb, bs + pad_rows, BYTES_PER_TOKEN), dtype=torch.float8_e4m3fn)[:, :bs, :]
    nope = res[..., :D_NOPE]
    scales = res[..., D_NOPE:D_NOPE + 4 * NUM_GROUPS].view(torch.float32)
    rope = res[..., D_NOPE + 4 * NUM_GROUPS:].view(blocked_k.dtype)
    rope[:] = x[..., D_NOPE:]
    for g in range(NUM_GROUPS):
        grp = x[..., g * GROUP:(g + 1) * GROUP]
        s = grp.abs().max(dim=-1).values.float() / 448.0
        if pow2_scale:
            s = torch.pow(2, torch.clamp_min(s, 1e-4).log2().ceil()).float()
        else:
            s = torch.clamp_min(s, 1e-30)
        scales[:, :, g] = s
        nope[..., g * GROUP:(g + 1) * GROUP] = (grp.float() / s.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return res.view(nb, bs, 1, BYTES_PER_TOKEN)


def dequantize_v32(quant: torch.Tensor) -> torch.Tensor:
    """Restates dequantize_k_cache, V32 branch (tests/quant.py:81-104):
    bf16( fp32(e4m3) * fp32(scale) ), RoPE copied.  Returns [num_blocks, block_size, 1, 576] bf16."""
    nb, bs, h_k, nbytes = quant.shape
    assert h_k == 1 and nbytes == BYTES_PER_TOKEN
    qv = quant.view(torch.float8_e4m3fn) if quant.dtype != torch.float8_e4m3fn else quant
    qv = qv.reshape(nb, bs, nbytes) if qv.is_contiguous() else qv.squeeze(2)
    out = torch.empty((nb, bs, D_QK), dtype=torch.bfloat16)
    nope = qv[..., :D_NOPE]
    scales = qv[..., D_NOPE:D_NOPE + 4 * NUM_GROUPS].view(torch.float32)
    out[..., D_NOPE:] = qv[..., D_NOPE + 4 * NUM_GROUPS:].view(torch.bfloat16)
    for g in range(NUM_GROUPS):
        out[..., g * GROUP:(g + 1) * GROUP] = nope[..., g * GROUP:(g + 1) * GROUP].float() * scales[..., g].unsqueeze(-1)
    return out.view(nb, bs, 1, D_QK)


# ---- "MODEL1" records (d_qk = 512): tests/quant.py:55-75 (quantiser), :106-117 (de-quantiser) -------------------------
# A block of block_size tokens is stored as
#   block_size x [448 x float8_e4m3fn "NoPE" | 64 x bfloat16 "RoPE"]      (576 bytes per token)
#   block_size x [7 x float8_e8m0fnu scales (one per 64 NoPE values) | 1 pad byte]
# padded up to a multiple of 576 bytes; the tensor handed to the kernels is the [num_blocks, block_size, 1, 584] view of it.
M1_D, M1_NOPE, M1_ROPE, M1_GROUP, M1_NUM_GROUPS = 512, 448, 64, 64, 7
M1_BYTES_PER_TOKEN = M1_NOPE + 2 * M1_ROPE + M1_NUM_GROUPS + 1      # 584


def model1_block_bytes(block_size: int) -> int:
    """Bytes from one block to the next (tests/quant.py:57)."""
    return (block_size * M1_BYTES_PER_TOKEN + 575) // 576 * 576


def quantize_model1(blocked_k: torch.Tensor) -> torch.Tensor:
    """Restates quantize_k_cache, MODEL1 branch (tests/quant.py:55-75): scale = 2^ceil(log2(max(amax/448, 1e-4))) stored as
    e8m0; value = e4m3(x / scale).  blocked_k [num_blocks, block_size, 1, 512] bf16 -> [num_blocks, block_size, 1, 584]
    float8_e4m3fn view (block stride model1_block_bytes(block_size))."""
    nb, bs, h_k, d = blocked_k.shape
    assert h_k == 1 and d == M1_D
    x = blocked_k.squeeze(2)
    res = torch.zeros((nb, model1_block_bytes(bs)), dtype=torch.uint8).view(torch.float8_e4m3fn)[:, :bs * M1_BYTES_PER_TOKEN]   # pad bytes 0
    data = res[:, :bs * 576].view(nb, bs, 576)
    nope = data[:, :, :M1_NOPE]
    rope = data[:, :, M1_NOPE:].view(blocked_k.dtype)
    scales = res[:, bs * 576:].view(nb, bs, 8)[:, :, :M1_NUM_GROUPS].view(torch.float8_e8m0fnu)
    rope[:] = x[..., M1_NOPE:]
    for g in range(M1_NUM_GROUPS):
        grp = x[..., g * M1_GROUP:(g + 1) * M1_GROUP]
        s = grp.abs().max(dim=-1).values.float() / 448.0
        s = torch.pow(2, torch.clamp_min(s, 1e-4).log2().ceil())
        scales[:, :, g] = s.to(torch.float8_e8m0fnu)
        nope[:, :, g * M1_GROUP:(g + 1) * M1_GROUP] = (grp.float() / s.unsqueeze(-1).float()).to(torch.float8_e4m3fn)
    return res.view(nb, bs, 1, M1_BYTES_PER_TOKEN)


def dequantize_model1(quant: torch.Tensor) -> torch.Tensor:
    """Restates dequantize_k_cache, MODEL1 branch (tests/quant.py:106-117): bf16(e4m3) * bf16(e8m0 scale) in bf16, RoPE
    copied.  Returns [num_blocks, block_size, 1, 512] bf16."""
    nb, bs, h_k, nbytes = quant.shape
    assert h_k == 1 and nbytes == M1_BYTES_PER_TOKEN
    qv = quant if quant.dtype == torch.float8_e4m3fn else quant.view(torch.float8_e4m3fn)
    flat = qv.reshape(nb, -1) if qv.is_contiguous() else qv.view(nb, -1)
    data = flat[:, :bs * 576].view(nb, bs, 576)
    nope = data[:, :, :M1_NOPE]
    rope = data[:, :, M1_NOPE:].view(torch.bfloat16)
    scales = flat[:, bs * 576:].view(nb, bs, 8)[:, :, :M1_NUM_GROUPS].view(torch.float8_e8m0fnu)
    out = torch.empty((nb, bs, M1_D), dtype=torch.bfloat16)
    out[..., M1_NOPE:] = rope
    for g in range(M1_NUM_GROUPS):
        out[..., g * M1_GROUP:(g + 1) * M1_GROUP] = nope[..., g * M1_GROUP:(g + 1) * M1_GROUP].to(torch.bfloat16) * \
            scales[:, :, g].to(torch.bfloat16).unsqueeze(-1)
    return out.view(nb, bs, 1, M1_D)


def abs_to_physical_indices(abs_indices: torch.Tensor, block_table: torch.Tensor, block_size: int) -> torch.Tensor:
    """Restates abs_indices2indices_in_kvcache (tests/quant.py:126-158): logical token position ->
    page * block_size + offset through the request's block-table row; -1 stays -1."""
    b, s_q, topk = abs_indices.shape
    a = abs_indices.clone().long()
    invalid = a == -1
    a[invalid] = 0
    out = torch.empty_like(a)
    for i in range(b):
        out[i] = block_table[i].long().index_select(0, (a[i] // block_size).reshape(-1)).view(s_q, topk) * block_size + a[i] % block_size
    out[invalid] = -1
    return out.to(torch.int32)
