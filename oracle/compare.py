"""Tensor comparison used by the parity tests.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Restates tests/kernelkit/compare.py:19-92: positions holding +inf / -inf / NaN
must match exactly and are then zeroed; every other element must pass an
absolute OR a relative bound, and the whole tensor a cosine-difference bound
cos_diff = 1 - 2*sum(a*b)/sum(a^2+b^2).
"""
import torch


def cos_diff(ans: torch.Tensor, ref: torch.Tensor) -> float:
    a, r = ans.double(), ref.double()
    if (r * r).sum().item() < 1e-12:
        return 0.0
    return 1.0 - 2.0 * (a * r).sum().item() / (a * a + r * r).sum().item()


def check_close(name: str, ans: torch.Tensor, ref: torch.Tensor, abs_tol: float, rel_tol: float,
                cos_diff_tol: float = None, quiet: bool = False) -> bool:
    assert ans.shape == ref.shape, f"{name}: shape {tuple(ans.shape)} vs {tuple(ref.shape)}"
    ans = ans.detach().cpu().float().clone()
    ref = ref.detach().cpu().float().clone()
    ok = True
    for val in (float("inf"), float("-inf"), float("nan")):
        rm = (ref == val) if val == val else (ref != ref)
        am = (ans == val) if val == val else (ans != ans)
        if not torch.equal(rm, am):
            if not quiet:
                print(f"{name}: anomaly {val} mismatch: {int(am.sum())} in ans, {int(rm.sum())} in ref")
            ok = False
        ref[rm] = 0.0
        ans[am] = 0.0
    err = (ans - ref).abs()
    rel = err / (ref.abs() + 1e-6)
    passed = (err < abs_tol) | (rel < rel_tol)
    if not bool(passed.all()):
        if not quiet:
            bad = (~passed).sum().item()
            print(f"{name}: {bad} of {passed.numel()} elements out of tolerance; max abs err {err.max().item():.3e}")
        ok = False
    if cos_diff_tol is not None:
        cd = cos_diff(ans, ref)
        if abs(cd) > cos_diff_tol:
            if not quiet:
                print(f"{name}: cosine difference {cd:.3e} > {cos_diff_tol:.1e}")
            ok = False
    return ok


def max_abs_err(ans: torch.Tensor, ref: torch.Tensor) -> float:
    a = ans.detach().cpu().float()
    r = ref.detach().cpu().float()
    finite = torch.isfinite(a) & torch.isfinite(r)
    if not bool(finite.any()):
        return 0.0
    return (a[finite] - r[finite]).abs().max().item()
