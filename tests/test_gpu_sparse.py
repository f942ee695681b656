"""GPU parity of sparse FP8 decode and token-sparse prefill against the CPU oracle, through the public API."""
import os

import pytest
import torch

from oracle import attention, quant
from tests.helpers import assert_lse_close, assert_out_close, non_contiguousify

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(t):
    return None if t is None else t.to(DEV)


def _decode(q, kv, indices, sm_scale, attn_sink=None, topk_length=None, extra_kv=None, extra_indices=None,
            extra_topk_length=None):
    import flashmla_b200 as fm
    meta, _ = fm.get_mla_metadata()
    out, lse = fm.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, sm_scale, False, True, indices, attn_sink,
                                         extra_kv, extra_indices, topk_length, extra_topk_length)
    torch.cuda.synchronize()
    fm.check_status()
    return out, lse


@pytest.mark.parametrize("impl", [1, 2])
def test_sparse_decode_golden_both_kernel_families(golden_dir, impl):
    """The portable kernel (1) and the tcgen05 kernel (2, rows padded to 128) on the reference-generated vectors,
    which cover attn_sink, topk_length, the extra cache and a request without any valid index."""
    import flashmla_b200 as fm
    fm.set_impl(impl)
    try:
        test_sparse_decode_golden(golden_dir)
    finally:
        fm.set_impl(0)


def test_sparse_decode_golden(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "sparse_decode.pt"), weights_only=False):
        kv = c["kv_bytes"].view(torch.float8_e4m3fn)
        out, lse = _decode(_dev(c["q"]), _dev(kv), _dev(c["indices"]), c["sm_scale"], _dev(c["attn_sink"]),
                           _dev(c["topk_length"]),
                           _dev(c["extra_kv_bytes"].view(torch.float8_e4m3fn)) if "extra_kv_bytes" in c else None,
                           _dev(c.get("extra_indices")), _dev(c.get("extra_topk_length")))
        assert_out_close("out", out, c["out"])
        assert_lse_close("lse", lse, c["lse"])


@pytest.mark.parametrize("b,s_q,h_q,s_kv,topk,pow2,sink", [
    (4, 1, 128, 1024, 256, False, False),
    (3, 2, 128, 2048, 512, True, True),
    (5, 1, 64, 512, 128, False, True),
    (2, 3, 16, 640, 192, False, False),
])
def test_sparse_decode_cases(b, s_q, h_q, s_kv, topk, pow2, sink):
    from tests import workloads as W
    d = W.sparse_decode_inputs(b, s_q, h_q, s_kv, topk, seed=b * 10 + s_q, device="cpu", pow2_scale=pow2, pad_rows=1)
    assert d["kv_fp8"].stride(0) == 65 * 656
    kv_deq = quant.dequantize_v32(d["kv_fp8"])
    # the reference's habit: every token no index refers to is NaN in the checker's cache
    attn_sink = None
    if sink:
        attn_sink = torch.randn(h_q, generator=torch.Generator().manual_seed(1))
        attn_sink[0] = float("inf")
        attn_sink[-1] = float("-inf")
    topk_length = torch.randint(0, topk + 1, (b,), generator=torch.Generator().manual_seed(2), dtype=torch.int32) if sink else None
    ref_out, ref_lse = attention.sparse_decode(d["q"], kv_deq, d["indices"], 576 ** -0.5, 512, attn_sink, topk_length)
    idx = non_contiguousify(d["indices"].to(DEV))
    out, lse = _decode(non_contiguousify(d["q"].to(DEV)), d["kv_fp8"].to(DEV), idx, 576 ** -0.5, _dev(attn_sink), _dev(topk_length))
    assert_out_close("out", out, ref_out)
    assert_lse_close("lse", lse, ref_lse)


def test_sparse_decode_lengths_come_and_go_on_one_sched_meta():
    """The reference accepts calls with and without topk_length on the same sched_meta (its partition count does not depend
    on them); here the two cases use different partition rules, so the stored schedule is made again when they switch."""
    import flashmla_b200 as fm
    from tests import workloads as W
    b, s_q, h_q, s_kv, topk = 6, 1, 64, 1024, 512
    d = W.sparse_decode_inputs(b, s_q, h_q, s_kv, topk, seed=3, device="cpu")
    kv_deq = quant.dequantize_v32(d["kv_fp8"])
    tl = torch.tensor([512, 0, 100, 511, 64, 300], dtype=torch.int32)
    meta, _ = fm.get_mla_metadata()
    q, kv, idx = d["q"].to(DEV), d["kv_fp8"].to(DEV), d["indices"].to(DEV)
    for lengths in (None, tl, None, tl):
        out, lse = fm.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, 576 ** -0.5, False, True, idx, None, None, None,
                                             _dev(lengths), None)
        torch.cuda.synchronize()
        fm.check_status()
        ref_out, ref_lse = attention.sparse_decode(d["q"], kv_deq, d["indices"], 576 ** -0.5, 512, None, lengths)
        assert_out_close("out", out, ref_out)
        assert_lse_close("lse", lse, ref_lse)
        assert meta.uniform_costs == (lengths is None)


def test_sparse_decode_all_invalid_and_unused_nan():
    """A request whose indices are all -1 gives out = 0 and lse = +inf; cache rows that no index refers to may
    hold NaN bytes without leaking into the result."""
    from tests import workloads as W
    d = W.sparse_decode_inputs(3, 1, 128, 512, 128, seed=3, device="cpu")
    d["indices"][1] = -1
    kv = d["kv_fp8"].clone()
    used = torch.zeros(kv.size(0) * 64, dtype=torch.bool)
    used[d["indices"][d["indices"] >= 0].long()] = True
    raw = kv.view(torch.uint8).view(-1, 656)
    raw[~used] = 0x7F                      # e4m3 NaN pattern, and NaN-ish scale / RoPE bytes
    kv_deq = quant.dequantize_v32(kv)
    ref_out, ref_lse = attention.sparse_decode(d["q"], kv_deq, d["indices"], 576 ** -0.5, 512)
    out, lse = _decode(d["q"].to(DEV), kv.to(DEV), d["indices"].to(DEV), 576 ** -0.5)
    assert_out_close("out", out, ref_out)
    assert_lse_close("lse", lse, ref_lse)
    assert (out[1] == 0).all() and (lse[1] == float("inf")).all()


@pytest.mark.parametrize("s_kv,topk,page", [(512, 64, 2), (512, 64, 69), (1024, 576, 2), (1024, 576, 61), (2046, 2048, 576), (650, 576, 53)])
@pytest.mark.parametrize("b,s_q", [(4, 1), (74, 3)])
def test_sparse_decode_page_sizes(s_kv, topk, page, b, s_q):
    """Page sizes other than 64, as the reference's grid has them (tests/test_flash_mla_sparse_decoding.py:37-57,
    106-112): the kernel resolves index -> (index / page_size, index % page_size) itself, and a block's stride is not
    page_size * 656 (one spare row per block)."""
    from tests import workloads as W
    d = W.sparse_decode_inputs(b, s_q, 128, s_kv, topk, seed=page + b, device="cpu", pad_rows=1, page_size=page)
    assert d["kv_fp8"].shape[1] == page and d["kv_fp8"].stride(0) == (page + 1) * 656
    kv_deq = quant.dequantize_v32(d["kv_fp8"])
    attn_sink = torch.randn(128, generator=torch.Generator().manual_seed(7))
    topk_length = torch.randint(0, topk + 1, (b,), generator=torch.Generator().manual_seed(8), dtype=torch.int32) if b == 4 else None
    ref_out, ref_lse = attention.sparse_decode(d["q"], kv_deq, d["indices"], 576 ** -0.5, 512, attn_sink, topk_length)
    out, lse = _decode(d["q"].to(DEV), d["kv_fp8"].to(DEV), d["indices"].to(DEV), 576 ** -0.5, attn_sink.to(DEV), _dev(topk_length))
    assert_out_close("out", out, ref_out)
    assert_lse_close("lse", lse, ref_lse)


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("page,extra_page", [(61, 2), (2, 69), (256, 64)])
def test_sparse_decode_extra_cache_page_sizes(page, extra_page, impl):
    """Main and extra cache with different page sizes (the extra one down to 2 tokens per page), per-request lengths
    for both scopes, both kernel families."""
    import flashmla_b200 as fm
    from tests import workloads as W
    b, s_q, h_q = 5, 2, 128
    main = W.sparse_decode_inputs(b, s_q, h_q, 700, 192, seed=page, device="cpu", pad_rows=1, page_size=page)
    extra = W.sparse_decode_inputs(b, s_q, h_q, 300, 128, seed=extra_page + 100, device="cpu", pad_rows=0, page_size=extra_page)
    g = torch.Generator().manual_seed(9)
    topk_length = torch.randint(0, 193, (b,), generator=g, dtype=torch.int32)
    extra_topk_length = torch.randint(0, 129, (b,), generator=g, dtype=torch.int32)
    attn_sink = torch.randn(h_q, generator=g)
    ref_out, ref_lse = attention.sparse_decode(main["q"], quant.dequantize_v32(main["kv_fp8"]), main["indices"], 576 ** -0.5, 512,
                                               attn_sink, topk_length, quant.dequantize_v32(extra["kv_fp8"]), extra["indices"],
                                               extra_topk_length)
    fm.set_impl(impl)
    try:
        out, lse = _decode(main["q"].to(DEV), main["kv_fp8"].to(DEV), main["indices"].to(DEV), 576 ** -0.5, attn_sink.to(DEV),
                           topk_length.to(DEV), extra["kv_fp8"].to(DEV), extra["indices"].to(DEV), extra_topk_length.to(DEV))
    finally:
        fm.set_impl(0)
    assert_out_close("out", out, ref_out)
    assert_lse_close("lse", lse, ref_lse)


def test_sparse_decode_config3_every_request():
    """batch 64, h_q 128, 32768 tokens per sequence, topk 2048 with the last 5% of each row -1, scale = amax/448:
    the whole batch runs on the GPU and EVERY request is checked against the oracle (which de-quantises, request by
    request, the 512 pages that request's block-table row owns)."""
    from tests import workloads as W
    d = W.sparse_decode_inputs(64, 1, 128, 32768, 2048, seed=0, device=DEV, data_on_device=True)
    out, lse = _decode(d["q"], d["kv_fp8"], d["indices"], 576 ** -0.5)
    out_c, lse_c, q_c, idx_c = out.cpu(), lse.cpu(), d["q"].cpu(), d["indices"].cpu()
    for i in range(64):
        idx = idx_c[i:i + 1]
        pages = d["block_table"][i].long()                       # this request's pages, in sequence order
        remap = torch.full((d["kv_fp8"].size(0),), -1, dtype=torch.int64)
        remap[pages] = torch.arange(pages.numel())
        kv_small = quant.dequantize_v32(d["kv_fp8"][pages.to(DEV)].cpu().contiguous())
        idx_small = torch.where(idx >= 0, (remap[(idx.clamp_min(0) // 64).long()] * 64 + idx % 64).to(torch.int32), idx)
        assert (idx_small[idx >= 0] >= 0).all()
        ref_out, ref_lse = attention.sparse_decode(q_c[i:i + 1], kv_small, idx_small, 576 ** -0.5, 512)
        assert_out_close(f"out[{i}]", out_c[i:i + 1], ref_out)
        assert_lse_close(f"lse[{i}]", lse_c[i:i + 1], ref_lse)


def _prefill(q, kv, indices, sm_scale, attn_sink=None, topk_length=None):
    import flashmla_b200 as fm
    out, mx, lse = fm.flash_mla_sparse_fwd(q, kv, indices, sm_scale, 512, attn_sink, topk_length)
    torch.cuda.synchronize()
    fm.check_status()
    return out, mx, lse


def test_sparse_prefill_golden(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "sparse_prefill.pt"), weights_only=False):
        out, mx, lse = _prefill(_dev(c["q"]), _dev(c["kv"]), _dev(c["indices"]), c["sm_scale"], _dev(c["attn_sink"]),
                                _dev(c["topk_length"]))
        assert_out_close("out", out, c["out"])
        assert_lse_close("max_logits", mx, c["max_logits"])
        assert_lse_close("lse", lse, c["lse"])


@pytest.mark.parametrize("impl", [1, 2])
def test_sparse_prefill_golden_both_kernel_families(golden_dir, impl):
    import flashmla_b200 as fm
    fm.set_impl(impl)
    try:
        test_sparse_prefill_golden(golden_dir)
    finally:
        fm.set_impl(0)


@pytest.mark.parametrize("s_q,h_q,s_kv,topk", [(62, 128, 2000, 256), (7, 64, 300, 128), (33, 128, 128, 384)])
def test_sparse_prefill_cases(s_q, h_q, s_kv, topk):
    from tests import workloads as W
    d = W.sparse_prefill_inputs(s_q, h_q, s_kv, topk, seed=s_q, device="cpu")
    zoo = torch.tensor([-2147483648, -123456, -1, s_kv, 114514, 1919810, 2147480000, 2147483647], dtype=torch.int32)
    idx = d["indices"]
    idx[idx < 0] = zoo[torch.arange(int((idx < 0).sum())) % zoo.numel()]
    idx[::5, 0, 3] = s_kv
    ref = attention.sparse_prefill(d["q"], d["kv"], idx, 0.5 * 576 ** -0.5, 512)
    out, mx, lse = _prefill(non_contiguousify(d["q"].to(DEV)), non_contiguousify(d["kv"].to(DEV)),
                            non_contiguousify(idx.to(DEV)), 0.5 * 576 ** -0.5)
    assert_out_close("out", out, ref[0])
    assert_lse_close("max_logits", mx, ref[1])
    assert_lse_close("lse", lse, ref[2])


def test_sparse_prefill_config4_rows():
    """s_kv 32768, topk 2048, h_q 128, causal-valid indices (query t draws from [0, 28672 + t]): a slice of query
    rows at the full KV size is checked against the oracle."""
    from tests import workloads as W
    d = W.sparse_prefill_inputs(48, 128, 32768, 2048, causal_base=28672, seed=0, device="cpu")
    ref = attention.sparse_prefill(d["q"], d["kv"], d["indices"], 576 ** -0.5, 512, row_chunk=8)
    out, mx, lse = _prefill(d["q"].to(DEV), d["kv"].to(DEV), d["indices"].to(DEV), 576 ** -0.5)
    assert_out_close("out", out, ref[0])
    assert_lse_close("max_logits", mx, ref[1])
    assert_lse_close("lse", lse, ref[2])


def test_sparse_prefill_config4_full_size():
    """The whole configuration (4096 query tokens, s_kv 32768, topk 2048) runs on the GPU; every 15th query token -
    274 rows, which hit every CTA pair of the persistent grid (15 and the pair count are coprime) at every depth of
    its stride - is checked against the oracle, the rest through size-independent properties."""
    from tests import workloads as W
    d = W.sparse_prefill_inputs(4096, 128, 32768, 2048, causal_base=28672, seed=0, device=DEV, data_on_device=True)
    out, mx, lse = _prefill(d["q"], d["kv"], d["indices"], 576 ** -0.5)
    rows = torch.arange(0, 4096, 15)
    assert rows.numel() >= 256
    ref = attention.sparse_prefill(d["q"][rows.to(DEV)].cpu(), d["kv"].cpu(), d["indices"][rows.to(DEV)].cpu(), 576 ** -0.5, 512, row_chunk=8)
    assert_out_close("out", out[rows.to(DEV)], ref[0])
    assert_lse_close("max_logits", mx[rows.to(DEV)], ref[1])
    assert_lse_close("lse", lse[rows.to(DEV)], ref[2])
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all() and torch.isfinite(mx).all()
    assert out.float().abs().max() <= d["kv"].float().abs().max()          # a convex combination of value rows
    assert (lse >= mx - 1e-3).all()                                        # log-sum-exp is at least the maximum logit


def test_fp8_cache_writer_bit_exact(golden_dir):
    """The cache-write kernel against the oracle's quantiser, byte for byte: random rows at several magnitudes, an
    all-zero row, padded block strides, both scale conventions, and the reference's own quantised bytes."""
    from flashmla_b200.kvcache import quantize_fp8_kvcache
    g = torch.Generator().manual_seed(3)
    x = torch.randn(7, 64, 1, 576, generator=g)
    x[1] *= 37.0
    x[2] *= 1e-3
    x[3, 5] = 0
    x[4, :, :, 128:256] = 0
    x = x.to(torch.bfloat16)
    for pow2 in (False, True):
        for pad in (0, 1):
            ref = quant.quantize_v32(x, pow2_scale=pow2, pad_rows=pad)
            got = quantize_fp8_kvcache(x.to(DEV), pow2_scale=pow2, pad_rows=pad)
            assert got.stride(0) == (64 + pad) * 656
            assert torch.equal(got.view(torch.uint8).contiguous().cpu(), ref.view(torch.uint8).contiguous()), (pow2, pad)
    # non-contiguous input view (every other block of a larger cache)
    big = torch.randn(6, 64, 1, 576, generator=g).to(torch.bfloat16)
    view = big[::2]
    dev_view = big.to(DEV)[::2]
    assert torch.equal(quantize_fp8_kvcache(dev_view, False).view(torch.uint8).contiguous().cpu(),
                       quant.quantize_v32(view, False, pad_rows=0).view(torch.uint8).contiguous())
    c = torch.load(os.path.join(golden_dir, "quant_v32.pt"), weights_only=False)
    got = quantize_fp8_kvcache(c["x"].to(DEV), pow2_scale=True, pad_rows=1)
    assert got.stride(0) == c["quant_stride0"]
    assert torch.equal(got.view(torch.uint8).contiguous().cpu().reshape(-1), c["quant_bytes"].reshape(-1))


@pytest.mark.parametrize("ragged", [False, True])
def test_sparse_decode_many_requests_per_partition(ragged):
    """More requests than SM partitions: every CTA pair walks several requests (and, with per-request lengths,
    partitions that split requests), so the hand-over of Q, of the K ring and of the accumulators between
    requests is what this checks; two runs must agree bit for bit."""
    from tests import workloads as W
    b, h_q, s_kv, topk = 190, 128, 1024, 256
    d = W.sparse_decode_inputs(b, 1, h_q, s_kv, topk, seed=11, device="cpu")
    kv_deq = quant.dequantize_v32(d["kv_fp8"])
    topk_length = torch.randint(0, topk + 1, (b,), generator=torch.Generator().manual_seed(5), dtype=torch.int32) if ragged else None
    ref_out, ref_lse = attention.sparse_decode(d["q"], kv_deq, d["indices"], 576 ** -0.5, 512, None, topk_length)
    args = (d["q"].to(DEV), d["kv_fp8"].to(DEV), d["indices"].to(DEV), 576 ** -0.5, None, _dev(topk_length))
    out, lse = _decode(*args)
    out2, lse2 = _decode(*args)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    assert_out_close("out", out, ref_out)
    assert_lse_close("lse", lse, ref_lse)


def test_sparse_prefill_many_query_tokens_per_cta_pair():
    """More query tokens than CTA pairs: every pair strides over several tokens, each with its own Q hand-over
    through the K ring; two runs must agree bit for bit."""
    from tests import workloads as W
    d = W.sparse_prefill_inputs(333, 128, 2048, 384, seed=9, device="cpu")
    ref = attention.sparse_prefill(d["q"], d["kv"], d["indices"], 576 ** -0.5, 512)
    args = (d["q"].to(DEV), d["kv"].to(DEV), d["indices"].to(DEV), 576 ** -0.5)
    out, mx, lse = _prefill(*args)
    out2, mx2, lse2 = _prefill(*args)
    assert torch.equal(out, out2) and torch.equal(lse, lse2) and torch.equal(mx, mx2)
    assert_out_close("out", out, ref[0])
    assert_lse_close("max_logits", mx, ref[1])
    assert_lse_close("lse", lse, ref[2])
