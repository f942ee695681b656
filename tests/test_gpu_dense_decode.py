"""GPU parity of dense BF16 MLA decode against the CPU oracle, through the public API
(which calls the C ABI)."""
import os

import pytest
import torch

from oracle import attention
from tests.helpers import assert_lse_close, assert_out_close, non_contiguousify

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(q, blocked_k, block_table, cache_seqlens, d_v, causal, impl=0):
    import flashmla_b200 as fm
    fm.set_impl(impl)
    try:
        meta, _ = fm.get_mla_metadata()
        out, lse = fm.flash_mla_with_kvcache(q, blocked_k, block_table, cache_seqlens, d_v, meta, None, causal=causal)
        # second call re-uses the cached scheduler metadata
        out2, lse2 = fm.flash_mla_with_kvcache(q, blocked_k, block_table, cache_seqlens, d_v, meta, None, causal=causal)
        torch.cuda.synchronize()
        fm.check_status()
        assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    finally:
        fm.set_impl(0)
    return out, lse


def test_golden_fixtures(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "dense_decode.pt"), weights_only=False):
        out, lse = _run(c["q"].to(DEV), c["blocked_k"].to(DEV), c["block_table"].to(DEV), c["cache_seqlens"].to(DEV),
                        c["d_v"], c["causal"])
        assert_out_close("out", out, c["out"])
        assert_lse_close("lse", lse, c["lse"])


def _case(b, s_q, h_q, h_kv, seqlens, causal, seed, noncontig=False, impl=0):
    from tests import workloads as W
    seq = torch.tensor(seqlens, dtype=torch.int32)
    d = W.dense_decode_inputs(seq, s_q, h_q, h_kv, seed=seed, device="cpu", poison_unused=True)
    ref_out, ref_lse = attention.dense_decode(d["q"], d["blocked_k"], d["block_table"], d["cache_seqlens"], 512, causal)
    q, k, bt = d["q"].to(DEV), d["blocked_k"].to(DEV), d["block_table"].to(DEV)
    if noncontig:
        q, k, bt = non_contiguousify(q), non_contiguousify(k), non_contiguousify(bt)
    out, lse = _run(q, k, bt, d["cache_seqlens"].to(DEV), 512, causal, impl)
    assert_out_close("out", out, ref_out)
    assert_lse_close("lse", lse, ref_lse)


def test_config1_tiny():
    """batch 4, s_q 1, h_q 16, seqlens uniform in [64, 512], causal, softmax_scale 576^-0.5."""
    g = torch.Generator().manual_seed(0)
    seq = torch.randint(64, 513, (4,), generator=g).tolist()
    _case(4, 1, 16, 1, seq, True, seed=0)


@pytest.mark.parametrize("s_q,h_q,h_kv,causal", [
    (1, 128, 1, False), (2, 128, 1, True), (1, 64, 1, False), (4, 9, 1, True), (2, 126, 2, True), (1, 3, 3, False),
    (2, 63, 1, True), (1, 1, 1, False),
    # two row blocks: Q boxes of 2 tokens x 64 heads per block / a group size that does not divide a row block
    # (Q is then loaded by the kernel's own threads)
    (4, 64, 1, True), (4, 48, 1, True),
    # eight KV heads: 8 and 16 query heads per KV head
    (1, 64, 8, False), (2, 128, 8, True),
])
def test_shape_grid(s_q, h_q, h_kv, causal):
    seqlens = [140, 4096 // 8 + 3, 20, 0, 64, 1, 1000, 65]
    _case(len(seqlens), s_q, h_q, h_kv, seqlens, causal, seed=s_q * 1000 + h_q, noncontig=(h_q % 2 == 1))


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("s_q,h_q,h_kv,causal", [(1, 128, 1, False), (2, 128, 1, True), (2, 48, 2, True), (1, 16, 1, False),
                                                 (1, 128, 8, True)])
def test_both_kernel_families(impl, s_q, h_q, h_kv, causal):
    """The portable kernel (1) and the tcgen05 kernel (2) must both match the oracle on the same inputs."""
    seqlens = [140, 515, 20, 0, 64, 1, 1000, 65, 4096]
    _case(len(seqlens), s_q, h_q, h_kv, seqlens, causal, seed=11 * s_q + h_q, noncontig=True, impl=impl)


def test_many_splits_long_sequence():
    """One long request next to short ones: the long one is split over many SM partitions."""
    _case(3, 1, 128, 1, [20000, 64, 300], False, seed=5)


def test_serving_shape_every_request():
    """Serving shape (batch 128, h_q 128, seqlens ~ N(4096, 512^2) clipped to [1, 8192], one forced to 8192,
    causal, s_q in {1, 2}): the full batch runs on the GPU and EVERY request is checked against the oracle."""
    from tests import workloads as W
    import flashmla_b200 as fm
    seq = W.seqlens_normal(128, 4096, 512, 1, 8192, True, seed=0)
    for s_q in (1, 2):
        d = W.dense_decode_inputs(seq, s_q, 128, 1, seed=7, device="cpu")
        meta, _ = fm.get_mla_metadata()
        out, lse = fm.flash_mla_with_kvcache(d["q"].to(DEV), d["blocked_k"].to(DEV), d["block_table"].to(DEV),
                                             d["cache_seqlens"].to(DEV), 512, meta, None, causal=True)
        torch.cuda.synchronize()
        fm.check_status()
        ref_out, ref_lse = attention.dense_decode(d["q"], d["blocked_k"], d["block_table"], d["cache_seqlens"], 512, True)
        assert_out_close("out", out, ref_out)
        assert_lse_close("lse", lse, ref_lse)
        # size-independent properties over the whole batch: finite results, and since a softmax output is a
        # convex combination of value rows, |out| is bounded by the largest |value| of the cache
        assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
        assert out.float().abs().max() <= d["blocked_k"].float().abs().max()


def test_fp16_inputs():
    """q and the cache in fp16 (the reference accepts both 16-bit types: csrc/api/dense_decode.h:33): checked against
    the oracle computed from the same fp16 values."""
    from tests import workloads as W
    seqlens = [140, 515, 20, 0, 64, 1, 1000, 65, 4096]
    for s_q, h_q, causal in ((1, 128, False), (2, 128, True), (2, 16, True)):
        d = W.dense_decode_inputs(torch.tensor(seqlens, dtype=torch.int32), s_q, h_q, 1, seed=31 + s_q, device="cpu", poison_unused=True)
        q16, k16 = d["q"].to(torch.float16), d["blocked_k"].to(torch.float16)
        ref_out, ref_lse = attention.dense_decode(q16, k16, d["block_table"], d["cache_seqlens"], 512, causal)
        assert ref_out.dtype == torch.float16
        out, lse = _run(q16.to(DEV), k16.to(DEV), d["block_table"].to(DEV), d["cache_seqlens"].to(DEV), 512, causal)
        assert out.dtype == torch.float16
        assert_out_close("out", out, ref_out)
        assert_lse_close("lse", lse, ref_lse)


@pytest.mark.parametrize("impl", [1, 2])
def test_sequence_longer_than_the_block_table(impl):
    """A cache_seqlens entry beyond 64 * max_blocks_per_seq must not read the block table out of bounds: blocks
    beyond the table's width have no page.  Results for such a request are unspecified (the reference would read out
    of bounds); the other requests must be right and nothing may fault."""
    from tests import workloads as W
    seq = torch.tensor([300, 200, 64], dtype=torch.int32)
    d = W.dense_decode_inputs(seq, 1, 128, 1, seed=41, device="cpu")
    ref_out, ref_lse = attention.dense_decode(d["q"], d["blocked_k"], d["block_table"], d["cache_seqlens"], 512, False)
    bad = seq.clone()
    bad[1] = 64 * d["block_table"].size(1) + 1000                 # far beyond the table
    out, lse = _run(d["q"].to(DEV), d["blocked_k"].to(DEV), d["block_table"].to(DEV), bad.to(DEV), 512, False, impl)
    keep = [0, 2]
    assert_out_close("out", out[keep], ref_out[keep])
    assert_lse_close("lse", lse[keep], ref_lse[keep])
    assert torch.isfinite(out[1].float()).all()


def test_longcontext_shard_sample():
    """Long-context sweep (1024 requests, log-normal lengths with median 8192, sigma 1, clipped to [256, 131072]):
    the shard that one of eight GPUs gets (128 requests) runs in full; the longest, the shortest and three other
    requests are checked against the oracle on their own pages, the whole shard through size-independent properties."""
    from tests import workloads as W
    import flashmla_b200 as fm
    seq_all = W.seqlens_lognormal(1024, 8192, 1.0, 256, 131072, seed=0)
    seq = seq_all[3 * 128:4 * 128].contiguous()
    d = W.dense_decode_inputs(seq, 1, 128, 1, seed=11, device=DEV, data_on_device=True)
    meta, _ = fm.get_mla_metadata()
    out, lse = fm.flash_mla_with_kvcache(d["q"], d["blocked_k"], d["block_table"], d["cache_seqlens"], 512, meta, None, causal=True)
    torch.cuda.synchronize()
    fm.check_status()
    order = torch.argsort(seq)
    sample = sorted({int(order[0]), int(order[-1]), 5, 64, 127})
    for i in sample:
        n = int(seq[i])
        pages = d["block_table"][i, :(n + 63) // 64].long()
        kv_i = d["blocked_k"][pages].cpu()
        bt_i = torch.arange(pages.numel(), dtype=torch.int32).view(1, -1)
        ref_out, ref_lse = attention.dense_decode(d["q"][i:i + 1].cpu(), kv_i, bt_i, seq[i:i + 1], 512, True)
        assert_out_close(f"out[{i}] (len {n})", out[i:i + 1], ref_out)
        assert_lse_close(f"lse[{i}] (len {n})", lse[i:i + 1], ref_lse)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert out.float().abs().max() <= d["blocked_k"].float().abs().max()
    # the log-sum-exp of a longer prefix of the same keys can only grow: compare each request with its own first half
    half = torch.clamp(seq // 2, min=1).to(DEV)
    meta2, _ = fm.get_mla_metadata()
    _, lse_half = fm.flash_mla_with_kvcache(d["q"], d["blocked_k"], d["block_table"], half, 512, meta2, None, causal=True)
    torch.cuda.synchronize()
    fm.check_status()
    assert (lse >= lse_half - 1e-3).all()
