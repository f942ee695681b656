"""GPU: tile-scheduler metadata (bit-exact vs the CPU restatement) and the split-KV combine kernel."""
import ctypes
import random

import numpy as np
import pytest
import torch

from oracle import sched_meta as osm
from tests.helpers import check_schedule_properties

pytestmark = pytest.mark.gpu


def _run_meta(b, P, bs, F, seqlens=None, topk=-1, extra_topk=0, topk_length=None, extra_topk_length=None):
    from flashmla_b200 import _capi
    dev = torch.device("cuda:0")
    t = lambda x: None if x is None else torch.tensor(x, dtype=torch.int32, device=dev)
    seq_t, tl_t, etl_t = t(seqlens), t(topk_length), t(extra_topk_length)
    meta = torch.full((P, 8), -7, dtype=torch.int32, device=dev)
    ns = torch.full((b + 1,), -7, dtype=torch.int32, device=dev)
    a = _capi.SchedMetaArgs(b=b, s_q=1, block_size_n=bs, fixed_overhead_num_blocks=F, topk=topk, extra_topk=extra_topk,
                            topk_length=_capi.ptr(tl_t), extra_topk_length=_capi.ptr(etl_t), seqlens_k=_capi.ptr(seq_t),
                            meta=_capi.ptr(meta), num_splits=_capi.ptr(ns), num_sm_parts=P,
                            stream=torch.cuda.current_stream().cuda_stream)
    _capi.check(_capi.lib().mla_get_sched_meta(a), "mla_get_sched_meta")
    torch.cuda.synchronize()
    return meta.cpu().numpy(), ns.cpu().numpy()


def test_sched_meta_known_answers_on_the_gpu(golden_dir):
    """The hand-derived vectors (dense, sparse with per-request lengths incl. 0, extra cache, zero-length requests,
    more partitions than work, fixed overhead 3) against the CUDA kernel itself."""
    import json
    import os
    for c in json.load(open(os.path.join(golden_dir, "sched_meta_known_answers.json")))["cases"]:
        if "seqlens" in c:
            meta, ns = _run_meta(len(c["seqlens"]), c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"], seqlens=c["seqlens"])
        else:
            b = c.get("b") or len(c["topk_length"])
            meta, ns = _run_meta(b, c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"], topk=c["topk"], extra_topk=c["extra_topk"],
                                 topk_length=c.get("topk_length"), extra_topk_length=c.get("extra_topk_length"))
        assert meta[:, :7].tolist() == c["meta"], c
        assert ns.tolist() == c["num_splits"], c


def test_sched_meta_bit_exact_dense():
    rng = random.Random(0)
    cases = [([200, 70], 4), ([1000], 4), ([0], 3), ([0, 0, 5], 2), ([64] * 7, 74), ([8192] + [4096] * 127, 74)]
    for _ in range(40):
        b = rng.randint(1, 300)
        P = rng.choice([1, 2, 5, 37, 74, 148])
        kind = rng.random()
        seq = [0 if rng.random() < 0.1 else (rng.randint(1, 200) if kind < 0.3 else rng.randint(1, 20000)) for _ in range(b)]
        cases.append((seq, P))
    for seq, P in cases:
        for F in (5, 3, 0):
            ref_meta, ref_ns = osm.get_sched_meta(len(seq), P, 64, F, seqlens_k=seq)
            meta, ns = _run_meta(len(seq), P, 64, F, seqlens=seq)
            assert np.array_equal(meta[:, :7], ref_meta[:, :7]), (seq[:8], P, F)
            assert np.array_equal(ns, ref_ns), (seq[:8], P, F)
            check_schedule_properties(meta, ns, seq, P, 64, F)        # the kernel's own output, not the oracle's


def test_sched_meta_bit_exact_sparse():
    rng = random.Random(1)
    for _ in range(30):
        b = rng.randint(1, 200)
        P = rng.choice([1, 3, 74, 148])
        topk = rng.choice([64, 128, 2048, 100])
        tl = [rng.randint(0, topk) for _ in range(b)] if rng.random() < 0.5 else None
        extra_topk = rng.choice([0, 64, 192])
        etl = [rng.randint(0, extra_topk) for _ in range(b)] if extra_topk and rng.random() < 0.5 else None
        ref_meta, ref_ns = osm.get_sched_meta(b, P, 64, 5, topk=topk, extra_topk=extra_topk, topk_length=tl, extra_topk_length=etl)
        meta, ns = _run_meta(b, P, 64, 5, topk=topk, extra_topk=extra_topk, topk_length=tl, extra_topk_length=etl)
        assert np.array_equal(meta[:, :7], ref_meta[:, :7])
        assert np.array_equal(ns, ref_ns)
        eff = osm.effective_seqlens(b, 64, None, topk, extra_topk, tl, etl)
        check_schedule_properties(meta, ns, eff, P, 64, 5)


def _combine_ref(lse_acc, o_acc, num_splits, b, s_q, h_q, sink, out_init, lse_init):
    """torch restatement of csrc/smxx/decode/combine/combine.cu:72-160."""
    LOG2E = 1.4426950408889634
    out, lse = out_init.clone().float(), lse_init.clone()
    for i in range(b):
        s0, s1 = int(num_splits[i]), int(num_splits[i + 1])
        if s1 - s0 <= 1:
            continue
        l = lse_acc[s0:s1]                                  # [n, s_q, h_q]
        mx = l.max(dim=0).values
        mx = torch.where(mx == float("-inf"), torch.zeros_like(mx), mx)
        sm = torch.exp2(l - mx).sum(dim=0)
        g = torch.where(sm == 0, torch.full_like(sm, float("inf")), torch.log2(sm) + mx)
        lse[i] = (g / LOG2E).transpose(0, 1)                # lse is [b, h_q, s_q]
        if sink is not None:
            sk = sink.view(1, h_q) * LOG2E
            g_fin = g + torch.log2(1 + torch.exp2(sk - g))
            g_inf = torch.where(sink.view(1, h_q) == float("-inf"), torch.full_like(g, float("inf")), sk.expand_as(g))
            g = torch.where(g != float("inf"), g_fin, g_inf)
        w = torch.exp2(l - g)                               # [n, s_q, h_q]
        out[i] = (w.unsqueeze(-1) * o_acc[s0:s1]).sum(dim=0)
    return out, lse


@pytest.mark.parametrize("with_sink", [False, True])
def test_combine_kernel(with_sink):
    from flashmla_b200 import _capi
    torch.manual_seed(3)
    dev = torch.device("cuda:0")
    b, s_q, h_q, d_v = 5, 2, 11, 512
    counts = [1, 3, 2, 40, 1]
    num_splits = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32)
    total = int(num_splits[-1])
    lse_acc = torch.randn(total, s_q, h_q) * 3
    lse_acc[1, 0, 0] = float("-inf")
    lse_acc[4:6, 1, 3] = float("-inf")                       # request 2 (2 splits), a row with no keys at all
    o_acc = torch.randn(total, s_q, h_q, d_v)
    o_acc[4:6, 1, 3] = 0
    sink = None
    if with_sink:
        sink = torch.randn(h_q)
        sink[0] = float("inf")
        sink[1] = float("-inf")
        sink[3] = float("inf")
    out_init = torch.randn(b, s_q, h_q, d_v).to(torch.bfloat16)
    lse_init = torch.randn(b, h_q, s_q)
    ref_out, ref_lse = _combine_ref(lse_acc, o_acc, num_splits, b, s_q, h_q, sink, out_init, lse_init)
    out, lse = out_init.to(dev), lse_init.to(dev)
    lse_acc_d, o_acc_d, ns_d = lse_acc.to(dev), o_acc.to(dev), num_splits.to(dev)
    sink_d = None if sink is None else sink.to(dev)
    c = _capi.CombineArgs(
        b=b, s_q=s_q, h_q=h_q, d_v=d_v,
        lse=_capi.ptr(lse), lse_stride_b=lse.stride(0), lse_stride_s=lse.stride(2), lse_stride_h=lse.stride(1),
        out=_capi.ptr(out), o_stride_b=out.stride(0), o_stride_s=out.stride(1), o_stride_h=out.stride(2),
        lse_accum=_capi.ptr(lse_acc_d), o_accum=_capi.ptr(o_acc_d), num_splits=_capi.ptr(ns_d), attn_sink=_capi.ptr(sink_d),
        stream=torch.cuda.current_stream().cuda_stream)
    _capi.check(_capi.lib().mla_combine(c), "mla_combine")
    torch.cuda.synchronize()
    out_c, lse_c = out.cpu().float(), lse.cpu()
    ref_bf16 = ref_out.to(torch.bfloat16).float()
    finite = torch.isfinite(ref_bf16)
    assert torch.equal(torch.isnan(out_c), torch.isnan(ref_bf16))
    assert (out_c[finite] - ref_bf16[finite]).abs().max() <= 2e-2
    assert torch.allclose(out_c[finite], ref_bf16[finite], rtol=2 ** -7, atol=1e-5)
    assert torch.equal(lse_c == float("inf"), ref_lse == float("inf"))
    fin = torch.isfinite(ref_lse)
    assert torch.allclose(lse_c[fin], ref_lse[fin], rtol=1e-5, atol=1e-5)


def test_uniform_partition_count_never_straddles_requests():
    """mla_num_sm_parts_uniform returns either the general count or exactly the batch size; with the batch size every
    partition holds exactly one whole request (the sparse decode path then skips the combine launch)."""
    from flashmla_b200 import _capi
    lib = _capi.lib()
    general = lib.mla_num_sm_parts(0, _capi.MLA_MODE_SPARSE_DECODE, 128, 1, 1)
    for b in (1, 7, 36, 37, 64, 73, 74, 75, 200):
        for blocks in (1, 2, 8, 32, 33, 48):
            P = lib.mla_num_sm_parts_uniform(0, _capi.MLA_MODE_SPARSE_DECODE, 128, 1, 1, b, blocks)
            assert P in (b, general), (b, blocks, P)
            if b > general:
                assert P == general
            if P == b:
                meta, ns = _run_meta(b, P, 64, 5, topk=blocks * 64)
                assert ns.tolist() == list(range(b + 1))
                assert meta[:, 0].tolist() == list(range(b)) and meta[:, 1].tolist() == list(range(b))
                assert not meta[:, 5].any() and not meta[:, 6].any()
