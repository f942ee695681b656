"""Attention oracles: fp32 torch-on-CPU restatements of the reference's own
torch implementations.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

* dense_decode      <- tests/test_flash_mla_dense_decoding.py:73-141 (reference_torch)
* sparse_decode     <- tests/ref.py:55-103 (ref_sparse_attn_decode)
* sparse_prefill    <- tests/ref.py:19-52  (ref_sparse_attn_fwd)

All three are pinned against outputs of those reference functions (vectors in
tests/golden/, produced by tests/golden/make_golden.py).
"""
import math
from typing import Optional, Tuple

import torch


def _attend(q: torch.Tensor, kv: torch.Tensor, invalid: Optional[torch.Tensor], scale: float, d_v: int,
            scale_by_division: bool = False):
    """q [R, d] fp32, kv [T, d] fp32, invalid [R, T] or [T] bool or None.
    Returns out [R, d_v] fp32, lse [R] (natural log; -inf when no key is valid),
    max_logits [R]."""
    logits = q @ kv.transpose(0, 1)                        # [R, T]
    if scale_by_division:
        logits = logits / scale                             # dense oracle divides by sqrt(d) (:109)
    else:
        logits = logits * scale                             # sparse oracles multiply by sm_scale (ref.py:35,84)
    if invalid is not None:
        logits = logits.masked_fill(invalid if invalid.dim() == 2 else invalid.unsqueeze(0), float("-inf"))
    if logits.size(1) == 0:
        lse = torch.full((q.size(0),), float("-inf"))
        mx = torch.full((q.size(0),), float("-inf"))
    else:
        lse = torch.logsumexp(logits, dim=-1)
        mx = logits.max(dim=-1).values
    return logits, lse, mx


def dense_decode(
    q: torch.Tensor,              # [b, s_q, h_q, d]
    blocked_k: torch.Tensor,      # [num_blocks, block_size, h_kv, d]
    block_table: torch.Tensor,    # [b, max_blocks] int32
    cache_seqlens: torch.Tensor,  # [b] int32
    d_v: int,
    is_causal: bool,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Restates reference_torch (tests/test_flash_mla_dense_decoding.py:73-141).

    Per request: gather the first ceil(len/bs) pages through the block table and
    keep `len` tokens (:131-134); NaN in KV -> 0 (:100); scores = q k^T / sqrt(d)
    (:101,109); causal mask tril(diagonal = s_k - s_q) only when s_q > 1
    (:102-108); lse = logsumexp (:110); out = softmax @ kv[:, :d_v] (:111-112);
    rows with no key: out = 0, lse = +inf (:113-116).  The softmax scale is
    always 1/sqrt(d) in the reference oracle.
    Returns out [b, s_q, h_q, d_v] in q.dtype and lse [b, h_q, s_q] fp32.
    """
    b, s_q, h_q, d = q.shape
    bs, h_kv = blocked_k.size(1), blocked_k.size(2)
    g = h_q // h_kv
    out = torch.zeros(b, s_q, h_q, d_v, dtype=torch.float32)
    lse_out = torch.empty(b, h_q, s_q, dtype=torch.float32)
    for i in range(b):
        n = int(cache_seqlens[i])
        nb = (n + bs - 1) // bs
        pages = block_table[i, :nb].long()
        kv = blocked_k[pages].reshape(-1, h_kv, d)[:n].float()      # [n, h_kv, d]
        kv = torch.where(kv != kv, torch.zeros_like(kv), kv)        # :100
        invalid = None
        if is_causal and s_q > 1:
            # tril(diagonal = s_k - s_q): query t sees keys j <= t + n - s_q   (:102-108)
            invalid = torch.arange(n).view(1, n) > (torch.arange(s_q).view(s_q, 1) + n - s_q)     # [s_q, n]
            invalid = invalid.unsqueeze(1).expand(s_q, g, n).reshape(s_q * g, n)
        for hk in range(h_kv):
            qh = q[i, :, hk * g:(hk + 1) * g, :].float().reshape(s_q * g, d)
            logits, lse, _ = _attend(qh, kv[:, hk], invalid, math.sqrt(d), d_v, scale_by_division=True)
            lonely = lse == float("-inf")
            lse_safe = torch.where(lonely, torch.zeros_like(lse), lse)
            p = torch.exp(logits - lse_safe.unsqueeze(-1))
            o = p @ kv[:, hk, :d_v] if n else torch.zeros(s_q * g, d_v)
            o[lonely] = 0.0
            out[i, :, hk * g:(hk + 1) * g] = o.view(s_q, g, d_v)
            lse_fix = torch.where(lonely, torch.full_like(lse, float("inf")), lse)
            lse_out[i, hk * g:(hk + 1) * g, :] = lse_fix.view(s_q, g).transpose(0, 1)
    return out.to(q.dtype), lse_out


def _gather_scope(kv_flat: torch.Tensor, indices: torch.Tensor, topk_length: Optional[torch.Tensor]):
    """kv_flat [tokens, d]; indices [b, s_q, topk]; returns gathered [b, s_q, topk, d] fp32 and
    invalid [b, s_q, topk] (tests/ref.py:66-75: invalid iff index == -1 or position >= topk_length)."""
    b, s_q, topk = indices.shape
    fixed = indices.clamp_min(0).long()
    gathered = kv_flat.index_select(0, fixed.reshape(-1)).view(b, s_q, topk, -1).float()
    invalid = indices == -1
    if topk_length is not None:
        invalid = invalid | (torch.arange(topk).view(1, 1, topk) >= topk_length.view(b, 1, 1))
    return gathered, invalid


def sparse_decode(
    q: torch.Tensor,                       # [b, s_q, h_q, d_qk]
    blocked_k: torch.Tensor,               # [num_blocks, block_size, 1, d_qk]  (already de-quantised)
    indices_in_kvcache: torch.Tensor,      # [b, s_q, topk] int32, -1 = invalid
    sm_scale: float,
    d_v: int,
    attn_sink: Optional[torch.Tensor] = None,      # [h_q] fp32
    topk_length: Optional[torch.Tensor] = None,    # [b] int32
    extra_blocked_k: Optional[torch.Tensor] = None,
    extra_indices_in_kvcache: Optional[torch.Tensor] = None,
    extra_topk_length: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Restates ref_sparse_attn_decode (tests/ref.py:55-103).
    Returns out [b, s_q, h_q, d_v] bf16, lse [b, h_q, s_q] fp32 (+inf for rows
    without a valid key; attn_sink scales out by 1/(1+exp(sink-lse)) and leaves
    lse unchanged, :93-96)."""
    b, s_q, h_q, d_qk = q.shape
    gathered, invalid = _gather_scope(blocked_k.reshape(-1, d_qk), indices_in_kvcache, topk_length)
    if extra_blocked_k is not None:
        g1, i1 = _gather_scope(extra_blocked_k.reshape(-1, d_qk), extra_indices_in_kvcache, extra_topk_length)
        gathered = torch.cat([gathered, g1], dim=2)
        invalid = torch.cat([invalid, i1], dim=2)
    gathered = torch.where(gathered != gathered, torch.zeros_like(gathered), gathered)   # :81
    out = torch.zeros(b, s_q, h_q, d_v, dtype=torch.float32)
    lse_out = torch.empty(b, s_q, h_q, dtype=torch.float32)
    for i in range(b):
        for t in range(s_q):
            kv = gathered[i, t]
            logits, lse, _ = _attend(q[i, t].float(), kv, invalid[i, t], sm_scale, d_v)
            lonely = lse == float("-inf")
            lse_safe = torch.where(lonely, torch.zeros_like(lse), lse)
            o = torch.exp(logits - lse_safe.unsqueeze(-1)) @ kv[:, :d_v]
            if attn_sink is not None:
                o = o * (1.0 / (1.0 + torch.exp(attn_sink - lse))).unsqueeze(-1)
            o[lonely] = 0.0
            out[i, t] = o
            lse_out[i, t] = torch.where(lonely, torch.full_like(lse, float("inf")), lse)
    return out.to(torch.bfloat16), lse_out.transpose(1, 2)


def sparse_prefill(
    q: torch.Tensor,            # [s_q, h_q, d_qk] bf16
    kv: torch.Tensor,           # [s_kv, 1, d_qk] bf16
    indices: torch.Tensor,      # [s_q, 1, topk] int32
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,     # [h_q]
    topk_length: Optional[torch.Tensor] = None,   # [s_q]
    row_chunk: int = 64,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Restates ref_sparse_attn_fwd (tests/ref.py:19-52), processed in chunks of
    query rows (the semantics are per row, so chunking is exact).
    invalid iff idx < 0 or idx >= s_kv or position >= topk_length (:27-31);
    out is scaled by exp(lse)/(exp(lse)+exp(sink)) (:43-48); rows with no valid
    key: out 0, max_logits -inf, lse +inf (:50-52).
    Returns (out bf16 [s_q,h_q,d_v], max_logits fp32 [s_q,h_q], lse fp32 [s_q,h_q])."""
    s_q, h_q, d_qk = q.shape
    s_kv = kv.size(0)
    topk = indices.size(-1)
    kv2 = kv.reshape(s_kv, d_qk)
    out = torch.empty(s_q, h_q, d_v, dtype=torch.bfloat16)
    max_logits = torch.empty(s_q, h_q, dtype=torch.float32)
    lse_out = torch.empty(s_q, h_q, dtype=torch.float32)
    for r0 in range(0, s_q, row_chunk):
        r1 = min(s_q, r0 + row_chunk)
        idx = indices[r0:r1, 0, :].clone().long()
        invalid = (idx < 0) | (idx >= s_kv)
        if topk_length is not None:
            invalid |= torch.arange(topk).unsqueeze(0) >= topk_length[r0:r1].unsqueeze(1)
        idx[invalid] = 0
        g = kv2.index_select(0, idx.reshape(-1)).view(r1 - r0, topk, d_qk).float()
        P = torch.bmm(q[r0:r1].float(), g.transpose(1, 2)) * sm_scale          # [r, h_q, topk]
        P = P.masked_fill(invalid.unsqueeze(1), float("-inf"))
        lse = torch.logsumexp(P, dim=-1)
        mx = P.max(dim=-1).values
        lse_for_o = lse if attn_sink is None else torch.logsumexp(
            torch.stack([lse, attn_sink.view(1, h_q).expand_as(lse)], dim=0), dim=0)
        lse_for_o = torch.where(lse_for_o == float("-inf"), torch.full_like(lse_for_o, float("inf")), lse_for_o)
        o = torch.bmm(torch.exp(P - lse_for_o.unsqueeze(-1)), g[..., :d_v])
        out[r0:r1] = o.to(torch.bfloat16)
        max_logits[r0:r1] = mx
        lse_out[r0:r1] = torch.where(lse == float("-inf"), torch.full_like(lse, float("inf")), lse)
    return out, max_logits, lse_out
