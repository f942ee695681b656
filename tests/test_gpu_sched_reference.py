"""GPU: the tile-scheduler metadata of this repository (CUDA kernel and CPU restatement) against the REFERENCE'S OWN kernel,
value for value.  The reference kernel (csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu, unmodified) is
compiled by oracle/build_ref.py into oracle/_ref/libref_sched_meta.so where a FlashMLA checkout is at hand; the built
library travels with the repository.  Without it these tests are skipped (the hand-derived vectors and the schedule
properties in tests/test_gpu_sched_combine.py remain).

Every case is first run through the CPU restatement, which asserts the reference's closing device assert
(get_decoding_sched_meta.cu:100) on the host, so that the reference kernel is only launched on inputs it accepts."""
import ctypes
import json
import os
import random

import numpy as np
import pytest
import torch

from oracle import sched_meta as osm

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_sched_meta.so")


@pytest.fixture(scope="module")
def ref_lib():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libref_sched_meta.so has not been built (python oracle/build_ref.py <FlashMLA checkout>)")
    lib = ctypes.CDLL(REF_LIB)
    lib.ref_get_decoding_sched_meta.restype = ctypes.c_int
    lib.ref_get_decoding_sched_meta.argtypes = [ctypes.c_int] * 6 + [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_void_p]
    return lib


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _three_ways(lib, b, P, bs, F, seqlens=None, topk=-1, extra_topk=0, topk_length=None, extra_topk_length=None):
    """(reference kernel, this repository's kernel, CPU restatement) on the same inputs."""
    from flashmla_b200 import _capi
    # the restatement first: it raises where the reference kernel's device assert would fire
    o_meta, o_ns = osm.get_sched_meta(b, P, bs, F, seqlens_k=seqlens, topk=topk, extra_topk=extra_topk,
                                      topk_length=topk_length, extra_topk_length=extra_topk_length)
    dev = torch.device("cuda:0")
    t = lambda x: None if x is None else torch.tensor(x, dtype=torch.int32, device=dev)
    seq_t, tl_t, etl_t = t(seqlens), t(topk_length), t(extra_topk_length)
    stream = torch.cuda.current_stream().cuda_stream
    r_meta = torch.full((P, 8), -7, dtype=torch.int32, device=dev)
    r_ns = torch.full((b + 1,), -7, dtype=torch.int32, device=dev)
    rc = lib.ref_get_decoding_sched_meta(b, 1, bs, F, topk, extra_topk, _ptr(tl_t), _ptr(etl_t), _ptr(seq_t), _ptr(r_meta), _ptr(r_ns),
                                         P, ctypes.c_void_p(stream))
    assert rc == 0
    m_meta = torch.full((P, 8), -7, dtype=torch.int32, device=dev)
    m_ns = torch.full((b + 1,), -7, dtype=torch.int32, device=dev)
    a = _capi.SchedMetaArgs(b=b, s_q=1, block_size_n=bs, fixed_overhead_num_blocks=F, topk=topk, extra_topk=extra_topk,
                            topk_length=_capi.ptr(tl_t), extra_topk_length=_capi.ptr(etl_t), seqlens_k=_capi.ptr(seq_t),
                            meta=_capi.ptr(m_meta), num_splits=_capi.ptr(m_ns), num_sm_parts=P, stream=stream)
    _capi.check(_capi.lib().mla_get_sched_meta(a), "mla_get_sched_meta")
    torch.cuda.synchronize()
    return (r_meta.cpu().numpy(), r_ns.cpu().numpy()), (m_meta.cpu().numpy(), m_ns.cpu().numpy()), (o_meta, o_ns)


def _same(three, what):
    (r_meta, r_ns), (m_meta, m_ns), (o_meta, o_ns) = three
    # seven meaningful words per record; the eighth is padding the reference leaves unwritten
    assert np.array_equal(m_meta[:, :7], r_meta[:, :7]), ("kernel vs reference", what)
    assert np.array_equal(m_ns, r_ns), ("kernel vs reference", what)
    assert np.array_equal(o_meta[:, :7], r_meta[:, :7]), ("restatement vs reference", what)
    assert np.array_equal(o_ns, r_ns), ("restatement vs reference", what)


def test_reference_kernel_agrees_on_the_known_answers(ref_lib, golden_dir):
    for c in json.load(open(os.path.join(golden_dir, "sched_meta_known_answers.json")))["cases"]:
        if "seqlens" in c:
            three = _three_ways(ref_lib, len(c["seqlens"]), c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"], seqlens=c["seqlens"])
        else:
            b = c.get("b") or len(c["topk_length"])
            three = _three_ways(ref_lib, b, c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"], topk=c["topk"], extra_topk=c["extra_topk"],
                                topk_length=c.get("topk_length"), extra_topk_length=c.get("extra_topk_length"))
        _same(three, c)
        assert three[0][0][:, :7].tolist() == c["meta"] and three[0][1].tolist() == c["num_splits"], c     # the hand derivation itself


def test_reference_kernel_dense_random(ref_lib):
    rng = random.Random(0)
    cases = [([200, 70], 4), ([1000], 4), ([0], 3), ([0, 0, 5], 2), ([64] * 7, 74), ([8192] + [4096] * 127, 74),
             ([4096] * 128, 74), ([1] * 500, 148), ([131072, 256, 300], 74)]
    for _ in range(60):
        b = rng.randint(1, 400)
        P = rng.choice([1, 2, 5, 37, 74, 132, 148])
        kind = rng.random()
        seq = [0 if rng.random() < 0.1 else (rng.randint(1, 200) if kind < 0.3 else rng.randint(1, 20000)) for _ in range(b)]
        cases.append((seq, P))
    for seq, P in cases:
        for F in (5, 3, 0):
            _same(_three_ways(ref_lib, len(seq), P, 64, F, seqlens=seq), (seq[:8], len(seq), P, F))


def test_reference_kernel_sparse_random(ref_lib):
    rng = random.Random(1)
    for _ in range(60):
        b = rng.randint(1, 300)
        P = rng.choice([1, 3, 37, 74, 148])
        topk = rng.choice([64, 128, 2048, 100, 1])
        tl = [rng.randint(0, topk) for _ in range(b)] if rng.random() < 0.5 else None
        extra_topk = rng.choice([0, 64, 192, 1000])
        etl = [rng.randint(0, extra_topk) for _ in range(b)] if extra_topk and rng.random() < 0.5 else None
        F = rng.choice([5, 5, 3])
        _same(_three_ways(ref_lib, b, P, 64, F, topk=topk, extra_topk=extra_topk, topk_length=tl, extra_topk_length=etl),
              (b, P, topk, extra_topk, tl is not None, etl is not None, F))


@pytest.mark.parametrize("with_sink", [False, True])
@pytest.mark.parametrize("b,s_q,h_q,P", [(5, 2, 11, 74), (128, 1, 128, 74), (9, 3, 64, 148), (3, 1, 8, 20)])
def test_reference_combine_kernel(ref_lib, with_sink, b, s_q, h_q, P):
    """This repository's combine kernel against the reference's own (csrc/smxx/decode/combine/combine.cu, built with the
    reference's flags) on the same partials: requests with 1..P splits, rows without keys (-inf partial LSEs), +-inf sinks.
    The reference kernel handles at most 160 splits per launch configuration and asserts my_num_splits <= its template bound,
    which holds because no request has more splits than there are partitions."""
    from flashmla_b200 import _capi
    ref_lib.ref_combine_bf16.restype = ctypes.c_int
    ref_lib.ref_combine_bf16.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    g = torch.Generator().manual_seed(b * 1000 + h_q + (1 if with_sink else 0))
    dev = torch.device("cuda:0")
    d_v = 512
    counts = [int(x) for x in torch.randint(1, 5, (b,), generator=g)]
    counts[b // 2] = min(P, 40)                               # one request with many splits
    counts[0] = 1                                             # one that is left untouched
    num_splits = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32)
    total = int(num_splits[-1])
    lse_acc = torch.randn(total, s_q, h_q, generator=g) * 3
    o_acc = torch.randn(total, s_q, h_q, d_v, generator=g)
    s0 = int(num_splits[1])                                   # request 1: one partial without keys, one row without any
    lse_acc[s0, 0, 0] = float("-inf")
    o_acc[s0, 0, 0] = 0
    lse_acc[s0:int(num_splits[2]), s_q - 1, h_q - 1] = float("-inf")
    o_acc[s0:int(num_splits[2]), s_q - 1, h_q - 1] = 0
    sink = None
    if with_sink:
        sink = torch.randn(h_q, generator=g)
        sink[0], sink[1], sink[h_q - 1] = float("inf"), float("-inf"), float("inf")
    out_init = torch.randn(b, s_q, h_q, d_v, generator=g).to(torch.bfloat16)
    lse_init = torch.randn(b, s_q, h_q, generator=g)
    lse_acc_d, o_acc_d, ns_d = lse_acc.to(dev), o_acc.to(dev), num_splits.to(dev)
    sink_d = None if sink is None else sink.to(dev)
    meta_d = torch.zeros(P, 8, dtype=torch.int32, device=dev)                 # not read by either kernel
    stream = torch.cuda.current_stream().cuda_stream
    # reference: lse [b, s_q, h_q]
    r_out, r_lse = out_init.to(dev), lse_init.to(dev)
    rc = ref_lib.ref_combine_bf16(b, s_q, h_q, d_v, _ptr(r_lse), _ptr(r_out), _ptr(lse_acc_d), _ptr(o_acc_d), _ptr(meta_d), _ptr(ns_d),
                                  P, _ptr(sink_d), ctypes.c_void_p(stream))
    assert rc == 0
    # this repository: same buffers, lse addressed through strides
    m_out, m_lse = out_init.to(dev), lse_init.to(dev)
    c = _capi.CombineArgs(
        b=b, s_q=s_q, h_q=h_q, d_v=d_v,
        lse=_capi.ptr(m_lse), lse_stride_b=m_lse.stride(0), lse_stride_s=m_lse.stride(1), lse_stride_h=m_lse.stride(2),
        out=_capi.ptr(m_out), o_stride_b=m_out.stride(0), o_stride_s=m_out.stride(1), o_stride_h=m_out.stride(2),
        lse_accum=_capi.ptr(lse_acc_d), o_accum=_capi.ptr(o_acc_d), num_splits=_capi.ptr(ns_d), attn_sink=_capi.ptr(sink_d),
        stream=stream)
    _capi.check(_capi.lib().mla_combine(c), "mla_combine")
    torch.cuda.synchronize()
    ro, mo, rl, ml = r_out.cpu().float(), m_out.cpu().float(), r_lse.cpu(), m_lse.cpu()
    assert torch.equal(torch.isnan(ro), torch.isnan(mo))
    fin = torch.isfinite(ro)
    # (the reference is built with --use_fast_math: its exp2 / log2 are the approximate ones)
    assert torch.allclose(mo[fin], ro[fin], rtol=2 ** -7, atol=2e-5), float((mo[fin] - ro[fin]).abs().max())
    assert float((mo[fin] != ro[fin]).float().mean()) < 0.02                   # almost every value is the same bf16
    assert torch.equal(ml == float("inf"), rl == float("inf"))
    lf = torch.isfinite(rl)
    assert torch.allclose(ml[lf], rl[lf], rtol=1e-5, atol=2e-5)
    # requests with a single split are left as they were by both
    assert torch.equal(m_out[0].cpu(), out_init[0]) and torch.equal(r_out[0].cpu(), out_init[0])
