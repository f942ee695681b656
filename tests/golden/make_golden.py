"""Generate the golden vectors in this directory by running the reference's OWN
torch code (imported unchanged from a FlashMLA checkout) on small seeded inputs.

Usage:  python tests/golden/make_golden.py <path-to-FlashMLA-checkout> [model1]

The reference test helpers import the compiled `flash_mla` extension at module
scope; it is replaced by an empty stub module because only the pure-torch
oracle functions are called:
  * tests/test_flash_mla_dense_decoding.py::reference_torch
  * tests/ref.py::ref_sparse_attn_decode, ref_sparse_attn_fwd
  * tests/quant.py::quantize_k_cache, dequantize_k_cache, abs_indices2indices_in_kvcache
Inputs and outputs are stored together so the parity tests never need the
checkout.
"""
import os
import sys
import types
import random

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(root):
    sys.modules.setdefault("flash_mla", types.ModuleType("flash_mla"))
    sys.path.insert(0, os.path.join(root, "tests"))
    import lib, ref, quant            # noqa: E401
    import test_flash_mla_dense_decoding as dense
    return lib, ref, quant, dense


def _seed(s):
    random.seed(s)
    torch.manual_seed(s)


def dense_cases(dense):
    cases = []
    specs = [
        # b, s_q, h_q, h_kv, seqlens, causal
        (3, 1, 8, 1, [130, 64, 1], False),
        (3, 2, 8, 1, [150, 77, 2], True),
        (2, 2, 8, 2, [100, 0], True),
        (2, 4, 6, 1, [3, 200], True),
        (2, 1, 16, 1, [0, 129], False),
    ]
    for ci, (b, s_q, h_q, h_kv, seqlens, causal) in enumerate(specs):
        _seed(100 + ci)
        d, dv, bs = 576, 512, 64
        max_blocks = 4
        q = torch.randn(b, s_q, h_q, d).to(torch.bfloat16)
        block_table = torch.randperm(b * max_blocks).to(torch.int32).view(b, max_blocks)
        blocked_k = torch.randn(b * max_blocks, bs, h_kv, d).to(torch.bfloat16)
        cache_seqlens = torch.tensor(seqlens, dtype=torch.int32)
        # the reference's habit: unused KV is NaN, unused block-table entries are out of range
        for i in range(b):
            n = seqlens[i]
            nb = (n + bs - 1) // bs
            blocked_k[block_table[i, nb:].long()] = float("nan")
            if n % bs:
                blocked_k[block_table[i, nb - 1].long(), n % bs:] = float("nan")
            block_table[i, nb:] = 2147480000
        out, lse = dense.reference_torch(cache_seqlens, block_table, q, blocked_k, dv, causal)
        cases.append(dict(q=q, blocked_k=blocked_k, block_table=block_table, cache_seqlens=cache_seqlens,
                          d_v=dv, causal=causal, out=out, lse=lse))
    return cases


def quant_cases(quant):
    _seed(200)
    x = torch.randn(3, 64, 1, 576).to(torch.bfloat16)
    x[0, 5, 0, :128] = 0.0      # an all-zero group: the scale clamp path
    qz = quant.quantize_k_cache(x, quant.FP8KVCacheLayout.V32_FP8Sparse)
    dq = quant.dequantize_k_cache(qz, quant.FP8KVCacheLayout.V32_FP8Sparse)
    abs_idx = torch.tensor([[[0, 63, 64, 130, -1]], [[191, 5, -1, 70, 64]]], dtype=torch.int32)
    bt = torch.tensor([[7, 2, 9], [4, 0, 1]], dtype=torch.int32)
    phys = quant.abs_indices2indices_in_kvcache(abs_idx, bt, 64)
    return dict(x=x, quant_bytes=qz.contiguous().view(torch.uint8), quant_stride0=qz.stride(0), dequant=dq,
                abs_indices=abs_idx, block_table=bt, phys_indices=phys)


def sparse_decode_cases(lib, ref, quant):
    cases = []
    specs = [
        # b, s_q, h_q, s_kv, topk, sink, topk_len, extra_topk, all_invalid_row
        (2, 1, 8, 256, 128, False, False, None, False),
        (2, 2, 8, 192, 128, True, True, None, False),
        (2, 1, 8, 256, 64, True, True, 64, True),
    ]
    for ci, (b, s_q, h_q, s_kv, topk, sink, tl, extra_topk, all_inv) in enumerate(specs):
        _seed(300 + ci)
        d_qk, d_v, bs = 576, 512, 64
        p = lib.TestParam(s_q, s_kv, topk, h_q, 1, d_qk, d_v, seed=300 + ci, have_attn_sink=sink,
                          have_topk_length=tl,
                          decode=lib.ExtraTestParamForDecode(b, False, False, extra_topk=extra_topk))
        q = torch.randn(b, s_q, h_q, d_qk).to(torch.bfloat16)
        attn_sink = None
        if sink:
            attn_sink = torch.randn(h_q)
            attn_sink[0] = float("inf")
            attn_sink[1] = float("-inf")

        def scope(topk_, s_kv_, with_len):
            nblk = b * (s_kv_ // bs)
            block_table = torch.randperm(nblk).to(torch.int32).view(b, -1)
            blocked_k = torch.randn(nblk, bs, 1, d_qk).to(torch.bfloat16)
            abs_idx = torch.stack([torch.stack([torch.randperm(s_kv_)[:topk_] for _ in range(s_q)]) for _ in range(b)]).to(torch.int32)
            abs_idx[:, :, -5:] = -1
            if all_inv:
                abs_idx[0] = -1
            phys = quant.abs_indices2indices_in_kvcache(abs_idx, block_table, bs)
            tlen = torch.randint(0, topk_ + 1, (b,), dtype=torch.int32) if with_len else None
            sc = lib.KVScope(p, torch.full((b,), s_kv_, dtype=torch.int32), block_table, blocked_k, abs_idx, phys, tlen)
            sc.quant_and_dequant_()
            return sc

        s0 = scope(topk, s_kv, tl)
        s1 = scope(extra_topk, 128, tl) if extra_topk else None
        t = lib.TestcaseForDecode(p, q, attn_sink, d_qk ** -0.55, s0, s1)
        out, lse = ref.ref_sparse_attn_decode(p, t)
        c = dict(q=q, attn_sink=attn_sink, sm_scale=t.sm_scale, d_v=d_v,
                 kv_bytes=s0.blocked_k_quantized.contiguous().view(torch.uint8),
                 indices=s0.indices_in_kvcache, topk_length=s0.topk_length, out=out, lse=lse.contiguous())
        if s1 is not None:
            c.update(extra_kv_bytes=s1.blocked_k_quantized.contiguous().view(torch.uint8),
                     extra_indices=s1.indices_in_kvcache, extra_topk_length=s1.topk_length)
        cases.append(c)
    return cases


def model1_cases(lib, ref, quant):
    """The d_qk = 512 ("MODEL1") forms: 584-byte FP8 records with e8m0 scales for decode, 512-wide rows for prefill."""
    L = quant.FP8KVCacheLayout.MODEL1_FP8Sparse
    _seed(500)
    x = (torch.randn(3, 64, 1, 512) * 2).to(torch.bfloat16)
    x[0, 0] = 0                                   # an all-zero token: scale clamps to 2^-13
    x[1, 3] *= 1000                               # a large token
    qz = quant.quantize_k_cache(x, L)
    qcase = dict(x=x, quant_bytes=qz.contiguous().view(torch.uint8), quant_stride0=qz.stride(0),
                 dequant=quant.dequantize_k_cache(qz, L))
    decode = []
    specs = [
        # b, s_q, h_q, s_kv, topk, sink, topk_len, extra_topk, block size
        (2, 1, 8, 256, 128, False, False, None, 64),
        (2, 2, 8, 192, 128, True, True, 64, 64),
        (2, 1, 8, 256, 64, True, False, None, 16),
    ]
    for ci, (b, s_q, h_q, s_kv, topk, sink, tl, extra_topk, bs) in enumerate(specs):
        _seed(510 + ci)
        d_qk, d_v = 512, 512
        p = lib.TestParam(s_q, s_kv, topk, h_q, 1, d_qk, d_v, seed=510 + ci, have_attn_sink=sink, have_topk_length=tl,
                          decode=lib.ExtraTestParamForDecode(b, False, False, extra_topk=extra_topk))
        q = torch.randn(b, s_q, h_q, d_qk).to(torch.bfloat16)
        attn_sink = None
        if sink:
            attn_sink = torch.randn(h_q)
            attn_sink[0] = float("inf")
            attn_sink[1] = float("-inf")

        def scope(topk_, s_kv_, with_len):
            nblk = b * (s_kv_ // bs)
            block_table = torch.randperm(nblk).to(torch.int32).view(b, -1)
            blocked_k = torch.randn(nblk, bs, 1, d_qk).to(torch.bfloat16)
            abs_idx = torch.stack([torch.stack([torch.randperm(s_kv_)[:topk_] for _ in range(s_q)]) for _ in range(b)]).to(torch.int32)
            abs_idx[:, :, -5:] = -1
            phys = quant.abs_indices2indices_in_kvcache(abs_idx, block_table, bs)
            tlen = torch.randint(0, topk_ + 1, (b,), dtype=torch.int32) if with_len else None
            sc = lib.KVScope(p, torch.full((b,), s_kv_, dtype=torch.int32), block_table, blocked_k, abs_idx, phys, tlen)
            sc.quant_and_dequant_()
            return sc

        s0 = scope(topk, s_kv, tl)
        s1 = scope(extra_topk, 128, tl) if extra_topk else None
        t = lib.TestcaseForDecode(p, q, attn_sink, d_qk ** -0.55, s0, s1)
        out, lse = ref.ref_sparse_attn_decode(p, t)
        c = dict(q=q, attn_sink=attn_sink, sm_scale=t.sm_scale, d_v=d_v, block_size=bs,
                 kv_bytes=s0.blocked_k_quantized.contiguous().view(torch.uint8),
                 kv_stride0=s0.blocked_k_quantized.stride(0),
                 indices=s0.indices_in_kvcache, topk_length=s0.topk_length, out=out, lse=lse.contiguous())
        if s1 is not None:
            c.update(extra_kv_bytes=s1.blocked_k_quantized.contiguous().view(torch.uint8),
                     extra_kv_stride0=s1.blocked_k_quantized.stride(0),
                     extra_indices=s1.indices_in_kvcache, extra_topk_length=s1.topk_length)
        decode.append(c)
    prefill = []
    for ci, (s_q, h_q, s_kv, topk, sink, tl) in enumerate([(5, 8, 200, 128, False, False), (4, 8, 300, 64, True, True)]):
        _seed(520 + ci)
        d_qk, d_v = 512, 512
        p = lib.TestParam(s_q, s_kv, topk, h_q, 1, d_qk, d_v, seed=520 + ci, have_attn_sink=sink, have_topk_length=tl)
        q = (torch.randn(s_q, h_q, d_qk) / 3).to(torch.bfloat16)
        kv = torch.randn(s_kv, 1, d_qk).to(torch.bfloat16)
        indices = torch.stack([torch.randperm(s_kv)[:topk] for _ in range(s_q)]).to(torch.int32).view(s_q, 1, topk)
        indices[:, :, -3:] = -1
        attn_sink = torch.randn(h_q) if sink else None
        topk_length = torch.randint(0, topk + 1, (s_q,), dtype=torch.int32) if tl else None
        t = lib.Testcase(p, None, q, kv, indices, d_qk ** -0.5, attn_sink, topk_length)
        out, _, max_logits, lse = ref.ref_sparse_attn_fwd(p, t)
        prefill.append(dict(q=q, kv=kv, indices=indices, sm_scale=t.sm_scale, d_v=d_v, attn_sink=attn_sink,
                            topk_length=topk_length, out=out, max_logits=max_logits, lse=lse))
    return dict(quant=qcase, decode=decode, prefill=prefill)


def sparse_prefill_cases(lib, ref):
    cases = []
    specs = [
        # s_q, h_q, s_kv, topk, sink, topk_len
        (5, 8, 200, 128, False, False),
        (6, 8, 100, 128, True, True),      # s_kv < topk: padded with the invalid-index zoo
    ]
    zoo = [-2147483648, -123456, -1, None, 114514, 1919810, 2147480000, 2147483647]
    for ci, (s_q, h_q, s_kv, topk, sink, tl) in enumerate(specs):
        _seed(400 + ci)
        d_qk, d_v = 576, 512
        p = lib.TestParam(s_q, s_kv, topk, h_q, 1, d_qk, d_v, seed=400 + ci, have_attn_sink=sink, have_topk_length=tl)
        q = (torch.randn(s_q, h_q, d_qk) / 3).to(torch.bfloat16)
        kv = torch.randn(s_kv, 1, d_qk).to(torch.bfloat16)
        indices = torch.empty(s_q, 1, topk, dtype=torch.int32)
        for r in range(s_q):
            perm = torch.randperm(s_kv)[:topk].to(torch.int32)
            row = torch.empty(topk, dtype=torch.int32)
            row[:perm.numel()] = perm
            for j in range(perm.numel(), topk):
                z = zoo[j % len(zoo)]
                row[j] = s_kv if z is None else z
            row[3] = zoo[r % len(zoo)] if zoo[r % len(zoo)] is not None else s_kv
            indices[r, 0] = row
        if ci == 1:
            indices[2] = 2147483647           # a query row without any valid key
        attn_sink = None
        if sink:
            attn_sink = torch.randn(h_q)
            attn_sink[0] = float("inf")
            attn_sink[1] = float("-inf")
        topk_length = torch.randint(0, topk + 1, (s_q,), dtype=torch.int32) if tl else None
        t = lib.Testcase(p, None, q, kv, indices, 0.5 if ci else d_qk ** -0.5, attn_sink, topk_length)
        out, _, max_logits, lse = ref.ref_sparse_attn_fwd(p, t)
        cases.append(dict(q=q, kv=kv, indices=indices, sm_scale=t.sm_scale, d_v=d_v, attn_sink=attn_sink,
                          topk_length=topk_length, out=out, max_logits=max_logits, lse=lse))
    return cases


def main():
    root = sys.argv[1]
    only = sys.argv[2] if len(sys.argv) > 2 else None          # e.g. "model1": write that file alone
    lib, ref, quant, dense = _import_reference(root)
    torch.set_num_threads(4)
    if only in (None, "model1"):
        torch.save(model1_cases(lib, ref, quant), os.path.join(HERE, "model1.pt"))
    if only is not None:
        return
    torch.save(dense_cases(dense), os.path.join(HERE, "dense_decode.pt"))
    torch.save(quant_cases(quant), os.path.join(HERE, "quant_v32.pt"))
    torch.save(sparse_decode_cases(lib, ref, quant), os.path.join(HERE, "sparse_decode.pt"))
    torch.save(sparse_prefill_cases(lib, ref), os.path.join(HERE, "sparse_prefill.pt"))
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
