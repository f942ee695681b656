"""Shared pieces of the GPU parity tests."""
import torch

from oracle.compare import check_close, cos_diff, max_abs_err

# Acceptance bounds of the benchmark specification: bf16 output within a cosine-similarity deficit of
# 1e-5 and a maximum absolute error of 2e-2; LSE within 1e-3.
OUT_COS_TOL = 1e-5
OUT_ABS_TOL = 2e-2
LSE_TOL = 1e-3
# The reference's own test tolerances (tests/test_flash_mla_dense_decoding.py:170-171,
# tests/test_flash_mla_sparse_decoding.py:228-229, tests/test_flash_mla_sparse_prefill.py:46-48): out passes
# element-wise on abs 8e-4..1e-3 OR rel 2.01/128, plus a cosine bound.  Its absolute bound is sized for its
# test data (randn/10, values of std 0.1); the inputs here are N(0,1) as the benchmark configurations ask,
# ten times larger, so the absolute bound scales by ten.  The relative and cosine bounds are scale-free.
REF_OUT = dict(abs_tol=1e-2, rel_tol=2.01 / 128, cos_diff_tol=7e-6)
REF_LSE = dict(abs_tol=1e-5, rel_tol=8.01 / 65536)


def assert_out_close(name, ans, ref, strict=True):
    ans_c, ref_c = ans.detach().cpu().float(), ref.detach().cpu().float()
    assert ans_c.shape == ref_c.shape, f"{name}: shape {tuple(ans_c.shape)} vs {tuple(ref_c.shape)}"
    assert torch.equal(torch.isnan(ans_c), torch.isnan(ref_c)), f"{name}: NaN pattern differs"
    cd = cos_diff(torch.nan_to_num(ans_c), torch.nan_to_num(ref_c))
    mae = max_abs_err(ans_c, ref_c)
    assert abs(cd) <= OUT_COS_TOL, f"{name}: cosine deficit {cd:.3e} > {OUT_COS_TOL}"
    assert mae <= OUT_ABS_TOL, f"{name}: max abs err {mae:.3e} > {OUT_ABS_TOL}"
    if strict:
        assert check_close(name, ans_c, ref_c, **REF_OUT), f"{name}: outside the reference's own tolerance"


def assert_lse_close(name, ans, ref, strict=True):
    ans_c, ref_c = ans.detach().cpu().float(), ref.detach().cpu().float()
    assert ans_c.shape == ref_c.shape, f"{name}: shape {tuple(ans_c.shape)} vs {tuple(ref_c.shape)}"
    for val in (float("inf"), float("-inf")):
        assert torch.equal(ans_c == val, ref_c == val), f"{name}: {val} pattern differs"
    assert torch.equal(torch.isnan(ans_c), torch.isnan(ref_c)), f"{name}: NaN pattern differs"
    mae = max_abs_err(ans_c, ref_c)
    assert mae <= LSE_TOL, f"{name}: max abs err {mae:.3e} > {LSE_TOL}"
    if strict:
        assert check_close(name, ans_c, ref_c, **REF_LSE), f"{name}: outside the reference's own tolerance"


def non_contiguousify(t: torch.Tensor) -> torch.Tensor:
    """Same habit as the reference's tests (tests/kernelkit/generate.py:3-25): the last dimension of the
    backing buffer is 128 longer, every other dimension 1 longer."""
    shape = [d + 128 if i == t.dim() - 1 else d + 1 for i, d in enumerate(t.shape)]
    base = torch.empty(shape, dtype=t.dtype, device=t.device)
    view = base[tuple(slice(0, d) for d in t.shape)]
    view[:] = t
    return view
