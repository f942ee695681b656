"""KV-sharded ("context-parallel") dense decode: every rank holds a part of each request's KV cache, computes
attention over its part with the ordinary decode path, and the partial results are merged with the same split-KV
combine kernel that merges the partials of SM partitions inside one GPU.

The one exchange step is an all_gather of (partial output, partial log-sum-exp) over the process group
(NCCL over NVLink for CUDA tensors).  A rank's partial is a softmax-normalised output o_r and its natural-log
normaliser lse_r; the merged result is sum_r exp(lse_r - lse) * o_r with lse = log sum_r exp(lse_r), which is what
mla_combine computes from base-2 LSEs (csrc/smxx/decode/combine/combine.cu:18-162 of the reference is the
in-GPU counterpart).  Decode only: one query token per request, or several without a causal mask.
"""
import math
from typing import Optional, Tuple

import torch

from . import _capi
from .flash_mla_interface import flash_mla_with_kvcache, get_mla_metadata

_LOG2E = 1.4426950408889634


def partials_to_split_layout(outs: torch.Tensor, lses: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Arranges gathered per-rank partials as the combine kernel's split-KV scratch.

    outs [world, b, s_q, h_q, d_v] (any float dtype), lses [world, b, h_q, s_q] natural log (+inf or -inf where a
    rank's part of a request is empty).  Returns (o_accum [b*world, s_q, h_q, d_v] fp32, lse_accum [b*world, s_q,
    h_q] fp32 base 2 with -inf for empty parts, num_splits [b+1] int32): request i owns rows i*world .. (i+1)*world."""
    world, b, s_q, h_q, d_v = outs.shape
    o_accum = outs.permute(1, 0, 2, 3, 4).reshape(b * world, s_q, h_q, d_v).float().contiguous()
    lse = lses.permute(1, 0, 3, 2).reshape(b * world, s_q, h_q).float()
    lse_accum = torch.where(torch.isinf(lse), torch.full_like(lse, -math.inf), lse * _LOG2E).contiguous()
    num_splits = (torch.arange(b + 1, dtype=torch.int32, device=outs.device) * world).contiguous()
    return o_accum, lse_accum, num_splits


def merge_kv_shard_partials(outs: torch.Tensor, lses: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merges the partial results of `world` KV shards with the library's combine kernel (mla_combine).

    outs [world, b, s_q, h_q, d_v], lses [world, b, h_q, s_q] (natural log; +/-inf where a shard holds nothing of a
    request), both CUDA tensors on one device - the all-gathered results of the ranks, or partials computed one after
    the other on a single GPU.  Returns (out [b, s_q, h_q, d_v] in out_dtype, lse [b, h_q, s_q] fp32)."""
    if not outs.is_cuda:
        raise RuntimeError("flashmla_b200 runs on CUDA devices only (there is no CPU path)")
    if out_dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError("out_dtype must be bfloat16 or float16")
    world, b, s_q, h_q, d_v = outs.shape
    o_accum, lse_accum, num_splits = partials_to_split_layout(outs, lses)
    out = torch.empty((b, s_q, h_q, d_v), dtype=out_dtype, device=outs.device)
    lse = torch.empty((b, h_q, s_q), dtype=torch.float32, device=outs.device)
    if world == 1:
        out.copy_(outs[0])
        lse.copy_(lses[0])
        return out, lse
    with torch.cuda.device(outs.device):
        c = _capi.CombineArgs(
            b=b, s_q=s_q, h_q=h_q, d_v=d_v,
            lse=_capi.ptr(lse), lse_stride_b=lse.stride(0), lse_stride_s=lse.stride(2), lse_stride_h=lse.stride(1),
            out=_capi.ptr(out), o_stride_b=out.stride(0), o_stride_s=out.stride(1), o_stride_h=out.stride(2),
            lse_accum=_capi.ptr(lse_accum), o_accum=_capi.ptr(o_accum), num_splits=_capi.ptr(num_splits), attn_sink=None,
            dtype=_capi.MLA_DTYPE_FP16 if out_dtype == torch.float16 else _capi.MLA_DTYPE_BF16,
            stream=torch.cuda.current_stream(outs.device).cuda_stream)
        _capi.check(_capi.lib().mla_combine(c), "mla_combine")
    return out, lse


def flash_mla_decode_kv_sharded(q: torch.Tensor, k_cache: torch.Tensor, block_table: torch.Tensor,
                                cache_seqlens: torch.Tensor, head_dim_v: int, softmax_scale: Optional[float] = None,
                                group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense MLA decode over a KV cache that is sharded across the ranks of `group`.

    q [b, s_q, h_q, 576] is the same on every rank; k_cache / block_table / cache_seqlens describe THIS rank's part
    of every request (a length of 0 is allowed).  Returns (out [b, s_q, h_q, d_v], lse [b, h_q, s_q]) of the
    attention over the union of all parts, identical on every rank."""
    import torch.distributed as dist
    if not q.is_cuda:
        raise RuntimeError("flashmla_b200 runs on CUDA devices only (there is no CPU path)")
    world = dist.get_world_size(group)
    meta, _ = get_mla_metadata()
    out_r, lse_r = flash_mla_with_kvcache(q, k_cache, block_table, cache_seqlens, head_dim_v, meta, None, softmax_scale, False)
    if world == 1:
        return out_r, lse_r
    outs = torch.empty((world,) + tuple(out_r.shape), dtype=out_r.dtype, device=q.device)
    lses = torch.empty((world,) + tuple(lse_r.shape), dtype=lse_r.dtype, device=q.device)
    dist.all_gather_into_tensor(outs, out_r.contiguous(), group=group)
    dist.all_gather_into_tensor(lses, lse_r.contiguous(), group=group)
    return merge_kv_shard_partials(outs, lses, q.dtype)
