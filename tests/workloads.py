"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(dense decode at the DeepSeek-V3 serving shape, sparse FP8 decode, token-sparse prefill, the
long-context batch-sharded sweep).  Used by the tests, bench.py and the smoke run; data is random-normal, no
dataset is involved.  Test and benchmark infrastructure: not part of the shipped package.
"""
import math
from typing import Dict, Optional

import torch

BLOCK = 64


def quantize_fp8_kvcache(blocked_k: torch.Tensor, pow2_scale: bool = False, pad_rows: int = 0) -> torch.Tensor:
    """656-byte FP8 records of a bf16 cache: CUDA tensors through the library's cache-write kernel, CPU tensors
    (fixtures that a CPU checker must see bit for bit) through the oracle's quantiser."""
    if blocked_k.is_cuda:
        from flashmla_b200.kvcache import quantize_fp8_kvcache as gpu_quantize
        return gpu_quantize(blocked_k, pow2_scale, pad_rows)
    from oracle import quant
    return quant.quantize_v32(blocked_k, pow2_scale=pow2_scale, pad_rows=pad_rows)


def _gen(seed: int, device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def seqlens_normal(b: int, mean: float, std: float, lo: int, hi: int, force_max: bool, seed: int) -> torch.Tensor:
    """N(mean, std^2) rounded and clipped to [lo, hi]; element 0 forced to hi when force_max."""
    g = _gen(seed)
    s = torch.clamp(torch.round(torch.randn(b, generator=g) * std + mean), lo, hi).to(torch.int32)
    if force_max:
        s[0] = hi
    return s


def seqlens_lognormal(b: int, median: float, sigma: float, lo: int, hi: int, seed: int) -> torch.Tensor:
    g = _gen(seed)
    s = torch.exp(torch.randn(b, generator=g) * sigma + math.log(median))
    return torch.clamp(torch.round(s), lo, hi).to(torch.int32)


def dense_decode_inputs(cache_seqlens: torch.Tensor, s_q: int, h_q: int, h_kv: int = 1, d: int = 576,
                        seed: int = 0, device="cuda", poison_unused: bool = False,
                        data_on_device: bool = False) -> Dict[str, torch.Tensor]:
    """Paged bf16 cache with a random block-table permutation, q and KV ~ N(0,1).

    data_on_device=False draws everything on the CPU (bit-identical inputs for a CPU checker) and
    copies; True draws q / KV with the device generator (large benchmark caches).
    poison_unused fills every cache row no request owns with NaN and the unused block-table entries
    with an out-of-range page id."""
    b = cache_seqlens.numel()
    max_len = int(cache_seqlens.max())
    max_blocks = max((max_len + BLOCK - 1) // BLOCK, 1)
    max_blocks = (max_blocks + 3) // 4 * 4
    g = _gen(seed + 1)
    block_table = torch.randperm(b * max_blocks, generator=g).to(torch.int32).view(b, max_blocks)
    num_blocks = b * max_blocks
    if data_on_device:
        gd = _gen(seed + 2, device)
        q = torch.randn(b, s_q, h_q, d, generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
        blocked_k = torch.empty(num_blocks, BLOCK, h_kv, d, dtype=torch.bfloat16, device=device)
        step = max(1, (1 << 28) // (BLOCK * h_kv * d))
        for i in range(0, num_blocks, step):
            n = min(step, num_blocks - i)
            blocked_k[i:i + n] = torch.randn(n, BLOCK, h_kv, d, generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
    else:
        q = torch.randn(b, s_q, h_q, d, generator=g).to(torch.bfloat16)
        blocked_k = torch.randn(num_blocks, BLOCK, h_kv, d, generator=g).to(torch.bfloat16)
    if poison_unused:
        bt_long = block_table.long()
        used_rows = torch.zeros(num_blocks, BLOCK, dtype=torch.bool)
        for i in range(b):
            n = int(cache_seqlens[i])
            nb = (n + BLOCK - 1) // BLOCK
            if nb:
                used_rows[bt_long[i, :nb]] = True
                if n % BLOCK:
                    used_rows[bt_long[i, nb - 1], n % BLOCK:] = False
            block_table[i, nb:] = 2147480000
        blocked_k[(~used_rows).to(blocked_k.device)] = float("nan")
    return dict(q=q.to(device), blocked_k=blocked_k.to(device), block_table=block_table.to(device),
                cache_seqlens=cache_seqlens.to(device))


def sparse_decode_inputs(b: int, s_q: int, h_q: int, s_kv: int, topk: int, pad_frac: float = 0.05, seed: int = 0,
                         device="cuda", pow2_scale: bool = False, pad_rows: int = 0,
                         data_on_device: bool = False, page_size: int = BLOCK, model1: bool = False) -> Dict[str, torch.Tensor]:
    """FP8 cache of s_kv tokens per request (656-byte records, scale = amax/448) in pages of `page_size` tokens, random
    block table, indices = unique tokens drawn without replacement, the last pad_frac of each row set to -1,
    expressed as physical positions page * page_size + offset.  model1: 512-wide queries and the 584-byte record form
    (device data only)."""
    d = 512 if model1 else 576
    blocks_per_seq = (s_kv + page_size - 1) // page_size
    num_blocks = b * blocks_per_seq
    g = _gen(seed + 1)
    block_table = torch.randperm(num_blocks, generator=g).to(torch.int32).view(b, blocks_per_seq)
    if data_on_device:
        gd = _gen(seed + 2, device)
        q = torch.randn(b, s_q, h_q, d, generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
        if model1:
            from flashmla_b200.kvcache import model1_block_bytes, quantize_fp8_kvcache_model1
            kv_fp8 = torch.zeros(num_blocks, model1_block_bytes(page_size), dtype=torch.uint8, device=device) \
                .view(torch.float8_e4m3fn)[:, :page_size * 584].view(num_blocks, page_size, 1, 584)
        else:
            kv_fp8 = torch.empty(num_blocks, page_size + pad_rows, 656, dtype=torch.float8_e4m3fn, device=device)[:, :page_size].unsqueeze(2)
        step = max(1, 4096 * 64 // page_size)
        for i in range(0, num_blocks, step):
            n = min(step, num_blocks - i)
            chunk = torch.randn(n, page_size, 1, d, generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
            if model1:
                kv_fp8[i:i + n].view(torch.uint8).copy_(quantize_fp8_kvcache_model1(chunk).view(torch.uint8))
            else:
                kv_fp8[i:i + n] = quantize_fp8_kvcache(chunk, pow2_scale)
    else:
        assert not model1, "the 512-wide form is generated on the device only"
        q = torch.randn(b, s_q, h_q, d, generator=g).to(torch.bfloat16)
        blocked_k = torch.randn(num_blocks, page_size, 1, d, generator=g).to(torch.bfloat16)
        kv_fp8 = quantize_fp8_kvcache(blocked_k, pow2_scale, pad_rows)
    n_valid = min(topk - int(topk * pad_frac), s_kv)
    abs_idx = torch.full((b, s_q, topk), -1, dtype=torch.int64)
    for i in range(b):
        for t in range(s_q):
            abs_idx[i, t, :n_valid] = torch.randperm(s_kv, generator=g)[:n_valid]
    invalid = abs_idx < 0
    a = abs_idx.clamp_min(0)
    page = torch.gather(block_table.long().unsqueeze(1).expand(b, s_q, blocks_per_seq), 2, a // page_size)
    phys = (page * page_size + a % page_size)
    phys[invalid] = -1
    return dict(q=q.to(device), kv_fp8=kv_fp8.to(device) if not data_on_device else kv_fp8,
                indices=phys.to(torch.int32).to(device), block_table=block_table, n_valid=n_valid)


def sparse_prefill_inputs(s_q: int, h_q: int, s_kv: int, topk: int, causal_base: Optional[int] = None, seed: int = 0,
                          device="cuda", data_on_device: bool = False) -> Dict[str, torch.Tensor]:
    """bf16 q [s_q, h_q, 576], kv [s_kv, 1, 576] ~ N(0,1); indices[t] = topk unique draws from
    [0, causal_base + t] (causal-valid) or from [0, s_kv) when causal_base is None."""
    d = 576
    g = _gen(seed + 1)
    if data_on_device:
        gd = _gen(seed + 2, device)
        q = torch.randn(s_q, h_q, d, generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
        kv = torch.randn(s_kv, 1, d, generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
        # top-k of random keys = sampling without replacement, drawn on the device for speed
        limit = (torch.arange(s_q, device=device) + (causal_base if causal_base is not None else s_kv - 1) + 1).clamp_max(s_kv)
        indices = torch.empty(s_q, 1, topk, dtype=torch.int32, device=device)
        step = 256
        for r0 in range(0, s_q, step):
            r1 = min(s_q, r0 + step)
            keys = torch.rand(r1 - r0, s_kv, generator=gd, device=device)
            keys[torch.arange(s_kv, device=device).unsqueeze(0) >= limit[r0:r1].unsqueeze(1)] = -1.0
            indices[r0:r1, 0] = keys.topk(topk, dim=-1).indices.to(torch.int32)
        return dict(q=q, kv=kv, indices=indices)
    q = torch.randn(s_q, h_q, d, generator=g).to(torch.bfloat16)
    kv = torch.randn(s_kv, 1, d, generator=g).to(torch.bfloat16)
    indices = torch.empty(s_q, 1, topk, dtype=torch.int32)
    for t in range(s_q):
        lim = s_kv if causal_base is None else min(causal_base + t + 1, s_kv)
        perm = torch.randperm(lim, generator=g)[:topk].to(torch.int32)
        indices[t, 0, :perm.numel()] = perm
        indices[t, 0, perm.numel():] = -1
    return dict(q=q.to(device), kv=kv.to(device), indices=indices.to(device))
