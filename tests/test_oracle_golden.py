"""Pins the CPU oracle (oracle/) against vectors produced by the reference's own
torch code (tests/golden/make_golden.py).  The scheduler's known answers and properties:
tests/test_sched_properties.py."""
import os

import numpy as np
import pytest
import torch

from oracle import attention, quant, sched_meta
from oracle.compare import check_close

# The restatement is not op-for-op identical to the reference (fp32 summation order), so a bf16 output
# may land on the neighbouring representable value: allow one bf16 ulp, and bound the whole tensor by cosine.
BF16_ULP = 2.0 ** -7


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name), weights_only=False)


def test_dense_decode_oracle_matches_reference(golden_dir):
    for c in _load(golden_dir, "dense_decode.pt"):
        out, lse = attention.dense_decode(c["q"], c["blocked_k"], c["block_table"], c["cache_seqlens"], c["d_v"], c["causal"])
        assert check_close("out", out, c["out"], abs_tol=1e-6, rel_tol=BF16_ULP, cos_diff_tol=1e-8)
        assert check_close("lse", lse, c["lse"], abs_tol=2e-6, rel_tol=1e-6)


def test_quant_oracle_matches_reference(golden_dir):
    c = _load(golden_dir, "quant_v32.pt")
    qz = quant.quantize_v32(c["x"], pow2_scale=True)
    assert qz.stride(0) == c["quant_stride0"]
    assert torch.equal(qz.contiguous().view(torch.uint8), c["quant_bytes"])
    dq = quant.dequantize_v32(c["quant_bytes"].view(torch.float8_e4m3fn))
    assert torch.equal(dq.view(torch.int16), c["dequant"].view(torch.int16))
    phys = quant.abs_to_physical_indices(c["abs_indices"], c["block_table"], 64)
    assert torch.equal(phys, c["phys_indices"])


def test_sparse_decode_oracle_matches_reference(golden_dir):
    for c in _load(golden_dir, "sparse_decode.pt"):
        kv = quant.dequantize_v32(c["kv_bytes"].view(torch.float8_e4m3fn))
        extra = None
        if "extra_kv_bytes" in c:
            extra = quant.dequantize_v32(c["extra_kv_bytes"].view(torch.float8_e4m3fn))
        out, lse = attention.sparse_decode(
            c["q"], kv, c["indices"], c["sm_scale"], c["d_v"], c["attn_sink"], c["topk_length"],
            extra, c.get("extra_indices"), c.get("extra_topk_length"))
        assert check_close("out", out, c["out"], abs_tol=1e-6, rel_tol=BF16_ULP, cos_diff_tol=1e-8)
        assert check_close("lse", lse, c["lse"], abs_tol=2e-6, rel_tol=1e-6)


def test_sparse_prefill_oracle_matches_reference(golden_dir):
    for c in _load(golden_dir, "sparse_prefill.pt"):
        out, mx, lse = attention.sparse_prefill(c["q"], c["kv"], c["indices"], c["sm_scale"], c["d_v"],
                                                c["attn_sink"], c["topk_length"], row_chunk=4)
        assert check_close("out", out, c["out"], abs_tol=1e-6, rel_tol=BF16_ULP, cos_diff_tol=1e-8)
        assert check_close("max_logits", mx, c["max_logits"], abs_tol=2e-6, rel_tol=1e-6)
        assert check_close("lse", lse, c["lse"], abs_tol=2e-6, rel_tol=1e-6)


def test_model1_oracle_matches_reference(golden_dir):
    """d_qk = 512: 584-byte records with e8m0 scales (decode) and 512-wide rows (prefill)."""
    from tests.helpers import model1_cache_from_bytes
    m = _load(golden_dir, "model1.pt")
    c = m["quant"]
    qz = quant.quantize_model1(c["x"])
    assert qz.stride(0) == c["quant_stride0"] == quant.model1_block_bytes(64)
    nb, bs = c["x"].shape[:2]
    mine, ref = qz.contiguous().view(torch.uint8).view(nb, -1), c["quant_bytes"].view(nb, -1)
    assert torch.equal(mine[:, :bs * 576], ref[:, :bs * 576])                              # values and RoPE
    assert torch.equal(mine[:, bs * 576:].view(nb, bs, 8)[..., :7], ref[:, bs * 576:].view(nb, bs, 8)[..., :7])   # scales (byte 8 is padding)
    dq = quant.dequantize_model1(model1_cache_from_bytes(c["quant_bytes"], c["quant_stride0"]))
    assert torch.equal(dq.view(torch.int16), c["dequant"].view(torch.int16))
    for c in m["decode"]:
        kv = quant.dequantize_model1(model1_cache_from_bytes(c["kv_bytes"], c["kv_stride0"]))
        extra = None
        if "extra_kv_bytes" in c:
            extra = quant.dequantize_model1(model1_cache_from_bytes(c["extra_kv_bytes"], c["extra_kv_stride0"]))
        out, lse = attention.sparse_decode(
            c["q"], kv, c["indices"], c["sm_scale"], c["d_v"], c["attn_sink"], c["topk_length"],
            extra, c.get("extra_indices"), c.get("extra_topk_length"))
        assert check_close("out", out, c["out"], abs_tol=1e-6, rel_tol=BF16_ULP, cos_diff_tol=1e-8)
        assert check_close("lse", lse, c["lse"], abs_tol=2e-6, rel_tol=1e-6)
    for c in m["prefill"]:
        out, mx, lse = attention.sparse_prefill(c["q"], c["kv"], c["indices"], c["sm_scale"], c["d_v"],
                                                c["attn_sink"], c["topk_length"], row_chunk=4)
        assert check_close("out", out, c["out"], abs_tol=1e-6, rel_tol=BF16_ULP, cos_diff_tol=1e-8)
        assert check_close("max_logits", mx, c["max_logits"], abs_tol=2e-6, rel_tol=1e-6)
        assert check_close("lse", lse, c["lse"], abs_tol=2e-6, rel_tol=1e-6)


def test_sched_meta_oracle_matches_the_reference_kernel(golden_dir):
    """tests/golden/sched_meta_reference.json holds what the reference's own CUDA kernel produced for 71 seeded dense and
    sparse cases (tests/golden/make_sched_golden.py): the restatement has to reproduce every word."""
    import json
    cases = json.load(open(os.path.join(golden_dir, "sched_meta_reference.json")))["cases"]
    assert len(cases) >= 70
    for c in cases:
        if "seqlens" in c:
            meta, ns = sched_meta.get_sched_meta(len(c["seqlens"]), c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"],
                                                 seqlens_k=c["seqlens"])
        else:
            meta, ns = sched_meta.get_sched_meta(c["b"], c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"], topk=c["topk"],
                                                 extra_topk=c["extra_topk"], topk_length=c["topk_length"],
                                                 extra_topk_length=c["extra_topk_length"])
        assert np.asarray(meta)[:, :7].tolist() == c["meta"], c
        assert np.asarray(ns).tolist() == c["num_splits"], c


def test_uniform_costs_one_partition_per_request_never_split():
    """With equal request costs and as many partitions as requests the greedy scheduler cuts at every request boundary
    (the sparse decode path relies on this to skip the combine kernel)."""
    for b in (1, 2, 7, 64, 74):
        for topk in (1, 64, 128, 2048, 2049):
            for extra in (-1, 64, 512):
                meta, ns = sched_meta.get_sched_meta(b, b, 64, 5, topk=topk, extra_topk=extra)
                assert ns.tolist() == list(range(b + 1)), (b, topk, extra)
                assert meta[:, 0].tolist() == list(range(b)) and meta[:, 1].tolist() == list(range(b))
                assert not meta[:, 5].any() and not meta[:, 6].any()
