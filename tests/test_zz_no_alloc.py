"""GPU: the allocation-free dense decode entry point (scratch inside the library) must give the same result as
the regular entry point with caller-provided scratch.

Some users of the C ABI run their decode loop on a memory plan that is fixed at start-up -- allocating there would
synchronise the device or fail -- and some bind the library from a runtime that has no device allocator.  They call
mla_dense_decode_noalloc, which keeps the split-KV scratch in a fixed array of the library.  The array is shared by
every call and keeps old contents, so the check runs two calls in a row with different inputs.
This file is collected last on purpose: a run that stops at the first failure has then seen every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_pair(b, s_q, h_q, seqlens, seed, check_oracle=False):
    import flashmla_b200 as fm
    from flashmla_b200 import _capi
    from tests import workloads as W
    from flashmla_b200.flash_mla_interface import _make_sched_meta
    lib = _capi.lib()
    seq = torch.tensor(seqlens, dtype=torch.int32)
    d = W.dense_decode_inputs(seq, s_q, h_q, 1, seed=seed, device=DEV, poison_unused=True)
    q, kc, bt, sl = d["q"], d["blocked_k"], d["block_table"], d["cache_seqlens"]
    # regular path through the public API (caller-side scratch)
    meta = fm.get_mla_metadata()[0]
    ref_out, ref_lse = fm.flash_mla_with_kvcache(q, kc, bt, sl, 512, meta, None, causal=True)
    # allocation-free path through the C ABI: outputs, metadata and status words are passed in, scratch is not
    P = lib.mla_num_sm_parts(0, _capi.MLA_MODE_DENSE_DECODE, h_q, 1, s_q)
    assert (b + P) * s_q * h_q <= _capi.NOALLOC_MAX_ROWS
    sched, num_splits = _make_sched_meta(b, s_q, P, torch.device(DEV), seqlens_k=sl)
    out = torch.full((b, s_q, h_q, 512), float("nan"), dtype=torch.bfloat16, device=DEV)
    lse = torch.full((b, h_q, s_q), float("nan"), dtype=torch.float32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    a = _capi.DenseDecodeArgs(
        b=b, s_q=s_q, h_q=h_q, h_kv=1, d_qk=576, d_v=512, num_blocks=kc.size(0), page_block_size=64,
        is_causal=int(s_q > 1), softmax_scale=576 ** -0.5,
        q=_capi.ptr(q), q_stride_b=q.stride(0), q_stride_s=q.stride(1), q_stride_h=q.stride(2),
        k_cache=_capi.ptr(kc), k_stride_block=kc.stride(0), k_stride_row=kc.stride(1), k_stride_head=kc.stride(2),
        block_table=_capi.ptr(bt), block_table_stride_b=bt.stride(0), max_blocks_per_seq=bt.size(1), seqlens_k=_capi.ptr(sl),
        out=_capi.ptr(out), o_stride_b=out.stride(0), o_stride_s=out.stride(1), o_stride_h=out.stride(2),
        lse=_capi.ptr(lse), lse_stride_b=lse.stride(0), lse_stride_s=lse.stride(2), lse_stride_h=lse.stride(1),
        meta=_capi.ptr(sched), num_splits=_capi.ptr(num_splits), num_sm_parts=P,
        lse_accum=None, o_accum=None, status=_capi.ptr(status), impl=0, dtype=_capi.MLA_DTYPE_BF16,
        stream=torch.cuda.current_stream().cuda_stream)
    _capi.check(lib.mla_dense_decode_noalloc(a), "mla_dense_decode_noalloc")    # (a device's first call also looks up the array's address)
    torch.cuda.synchronize()
    # a later call must not take device memory from anyone: neither from torch's allocator nor, unseen by it, from the
    # driver (free device memory as the driver reports it stays where it was)
    out.fill_(float("nan"))
    lse.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    _capi.check(lib.mla_dense_decode_noalloc(a), "mla_dense_decode_noalloc")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes across the call"
    assert torch.cuda.memory_allocated() == torch_before
    assert status.tolist() == [0, 0, 0, 0], "a bounded wait ran out inside the allocation-free launch"
    fm.check_status()
    # same kernels, same schedule: identical up to nothing at all
    assert torch.equal(out.view(torch.int16), ref_out.view(torch.int16))
    assert torch.equal(lse, ref_lse)
    if check_oracle:
        from oracle import attention
        from tests.helpers import assert_lse_close, assert_out_close
        o_ref, l_ref = attention.dense_decode(q.cpu(), kc.cpu(), bt.cpu(), sl.cpu(), 512, True)
        assert_out_close("out", out, o_ref)
        assert_lse_close("lse", lse, l_ref)
    return out, lse


def test_no_alloc_matches_regular_entry_point_twice():
    # the first call leaves partial results of a long, heavily split request in the shared scratch;
    # the second call (other lengths, other split pattern) must not be disturbed by them
    _run_pair(3, 1, 128, [9000, 64, 300], seed=21, check_oracle=True)
    _run_pair(4, 1, 128, [130, 5000, 1, 2049], seed=22, check_oracle=True)


def test_no_alloc_admits_the_serving_shape():
    """Batch 128 with 128 heads - (128 + 74) * 128 = 25856 rows of split scratch on a 148-SM part - fits the built-in array."""
    from tests import workloads as W
    seq = W.seqlens_normal(128, 512, 64, 1, 1024, True, seed=3).tolist()
    _run_pair(128, 1, 128, seq, seed=23)


def test_no_alloc_rejects_oversized_requests():
    from flashmla_b200 import _capi
    lib = _capi.lib()
    dummy = torch.zeros(16, device=DEV)
    a = _capi.DenseDecodeArgs(b=4096, s_q=1, h_q=128, h_kv=1, d_qk=576, d_v=512, num_sm_parts=74,
                              q=_capi.ptr(dummy), out=_capi.ptr(dummy), lse=_capi.ptr(dummy))
    assert lib.mla_dense_decode_noalloc(a) == 1
    assert b"exceed the built-in maximum" in lib.mla_last_error()
