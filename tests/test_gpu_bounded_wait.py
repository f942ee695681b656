"""GPU: what an expired barrier wait looks like to the caller.  A one-CTA self-test kernel of the library waits, with
the same helper the attention kernels use, on a barrier nobody arrives on and with nothing else in flight (no TMA, no
MMA, no cluster traffic); after the limit it writes the status words and returns normally - the context stays usable.
No wait is made to run out inside the attention kernels themselves."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_expired_wait_is_reported_and_the_context_survives():
    import flashmla_b200 as fm
    from flashmla_b200 import _capi, flash_mla_interface as fmi
    lib = _capi.lib()
    dev = torch.device(DEV)
    fm.check_status()                                # nothing pending from earlier tests
    status = fmi._status(dev)                        # the words every kernel launch of the Python API reports into
    flag = torch.full((2,), -1, dtype=torch.int32, device=dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.mla_selftest_bounded_wait(1_000_000, 77, _capi.ptr(status), _capi.ptr(flag), torch.cuda.current_stream().cuda_stream)
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()                         # returns: the kernel ended by itself
    assert 0.2 <= t0.elapsed_time(t1) <= 50.0        # about 1e6 cycles at 1-2 GHz, far from the default limit of a second
    assert flag.tolist() == [1, 0]                   # the CTA's abort flag is raised, the wait reported failure
    vals = status.tolist()
    assert vals[0] == 77 and vals[1] == 64           # first code, and every one of the 64 threads counted
    with pytest.raises(RuntimeError, match="gave up a bounded wait \\(code 77, 64 threads\\)"):
        fm.check_status()
    fm.check_status()                                # cleared by the raise
    assert status.tolist()[:2] == [0, 0]
    # the context is intact: an ordinary launch still works
    x = torch.arange(8, device=dev)
    assert int((x * 2).sum()) == 56


def test_selftest_rejects_bad_arguments():
    from flashmla_b200 import _capi
    lib = _capi.lib()
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    assert lib.mla_selftest_bounded_wait(0, 1, _capi.ptr(status), None, None) == 1
    assert lib.mla_selftest_bounded_wait(3_000_000_000, 1, _capi.ptr(status), None, None) == 1
    assert lib.mla_selftest_bounded_wait(1000, 1, None, None, None) == 1
