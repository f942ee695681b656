"""FP8 KV-cache records for the sparse decode path (the cache-write side of the path).

Per token 656 bytes: 512 float8_e4m3fn "NoPE" values quantised per group of 128 with one fp32
scale per group (x ~= fp8 * scale), the 4 scales, then 64 bf16 "RoPE" values stored as they are
(layout: flash_mla/flash_mla_interface.py:92-98 of the reference).  The 512-wide "MODEL1" form keeps 448 values in
groups of 64 with power-of-two scales (e8m0 bytes) and stores a block as block_size x 576 value bytes followed by
block_size x 8 scale bytes (flash_mla/flash_mla_interface.py:99-103).  The records are written by the library's
kernel (mla_quantize_fp8_kvcache); there is no CPU path.
"""
import torch

from . import _capi

D_QK, D_NOPE, D_ROPE, GROUP, NUM_GROUPS = 576, 512, 64, 128, 4
BYTES_PER_TOKEN = D_NOPE + 4 * NUM_GROUPS + 2 * D_ROPE


def quantize_fp8_kvcache(blocked_k: torch.Tensor, pow2_scale: bool = False, pad_rows: int = 0) -> torch.Tensor:
    """blocked_k [num_blocks, block_size, 1, 576] bf16 -> [num_blocks, block_size, 1, 656] float8_e4m3fn.

    scale = amax/448 of each 128-value group; with pow2_scale it is rounded up to a power of two
    (the convention of the reference's test quantiser).  pad_rows > 0 leaves spare rows at the end of
    every block, which makes the block stride differ from block_size * 656."""
    nb, bs, h_k, d = blocked_k.shape
    assert h_k == 1 and d == D_QK
    assert blocked_k.dtype == torch.bfloat16
    if not blocked_k.is_cuda:
        raise RuntimeError("blocked_k must be a CUDA tensor (this library has no CPU path)")
    x = blocked_k.squeeze(2)
    buf = torch.empty((nb, bs + pad_rows, BYTES_PER_TOKEN), dtype=torch.float8_e4m3fn, device=blocked_k.device)
    res = buf[:, :bs, :]
    assert x.stride(-1) == 1, "the last dimension of blocked_k must be contiguous"
    with torch.cuda.device(blocked_k.device):
        args = _capi.QuantizeArgs(
            x=_capi.ptr(x), x_stride_block=x.stride(0), x_stride_row=x.stride(1), num_blocks=nb, block_size=bs,
            out=_capi.ptr(buf), out_stride_block_bytes=buf.stride(0), pow2_scale=1 if pow2_scale else 0,
            stream=torch.cuda.current_stream().cuda_stream)
        _capi.check(_capi.lib().mla_quantize_fp8_kvcache(args), "mla_quantize_fp8_kvcache")
    return res.view(nb, bs, 1, BYTES_PER_TOKEN)


M1_D, M1_BYTES_PER_TOKEN = 512, 584


def model1_block_bytes(block_size: int) -> int:
    """Bytes from one block to the next in the 512-wide form: the reference pads a block to a multiple of 576 bytes
    (tests/quant.py:57)."""
    return (block_size * M1_BYTES_PER_TOKEN + 575) // 576 * 576


def quantize_fp8_kvcache_model1(blocked_k: torch.Tensor) -> torch.Tensor:
    """blocked_k [num_blocks, block_size, 1, 512] bf16 -> the [num_blocks, block_size, 1, 584] float8_e4m3fn view the
    sparse decode path takes for 512-wide queries (block stride model1_block_bytes(block_size))."""
    nb, bs, h_k, d = blocked_k.shape
    assert h_k == 1 and d == M1_D
    assert blocked_k.dtype == torch.bfloat16
    if not blocked_k.is_cuda:
        raise RuntimeError("blocked_k must be a CUDA tensor (this library has no CPU path)")
    x = blocked_k.squeeze(2)
    assert x.stride(-1) == 1, "the last dimension of blocked_k must be contiguous"
    buf = torch.zeros((nb, model1_block_bytes(bs)), dtype=torch.uint8, device=blocked_k.device).view(torch.float8_e4m3fn)
    with torch.cuda.device(blocked_k.device):
        args = _capi.QuantizeArgs(
            x=_capi.ptr(x), x_stride_block=x.stride(0), x_stride_row=x.stride(1), num_blocks=nb, block_size=bs,
            out=_capi.ptr(buf), out_stride_block_bytes=buf.stride(0), pow2_scale=1, layout=1,
            stream=torch.cuda.current_stream().cuda_stream)
        _capi.check(_capi.lib().mla_quantize_fp8_kvcache(args), "mla_quantize_fp8_kvcache")
    return buf[:, :bs * M1_BYTES_PER_TOKEN].view(nb, bs, 1, M1_BYTES_PER_TOKEN)
