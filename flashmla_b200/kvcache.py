"""FP8 KV-cache records for the sparse decode path (the cache-write side of the path).

Per token 656 bytes: 512 float8_e4m3fn "NoPE" values quantised per group of 128 with one fp32
scale per group (x ~= fp8 * scale), the 4 scales, then 64 bf16 "RoPE" values stored as they are
(layout: flash_mla/flash_mla_interface.py:92-98 of the reference).  The records are written by the library's
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
