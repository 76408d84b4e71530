"""The give-up path of the library's bounded waits, made to run out on purpose:
a one-thread kernel waits at most a few hundred polls on a barrier nothing
signals, returns normally, and the status word reports it once."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_that_runs_out_is_reported_once_and_cleared(cuda_dev):
    import torch

    from mamba_rs_b200 import ffi
    lib = ffi.lib()
    h = ffi.default_handle(0)
    h.check_status()  # clean to begin with
    stream = C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)
    rc = lib.mamba_b200_selftest_wait_timeout(h.ptr, stream, 500)
    assert rc == 0, lib.mamba_b200_last_error(h.ptr)
    torch.cuda.synchronize()  # the kernel ended by itself: the context is still usable
    rc = lib.mamba_b200_check_status(h.ptr, stream)
    assert rc == -5  # MAMBA_B200_ERR_KERNEL
    assert b"bounded wait" in lib.mamba_b200_last_error(h.ptr)
    assert lib.mamba_b200_check_status(h.ptr, stream) == 0  # cleared by the read
    # and the library still computes afterwards
    x = torch.ones(1, 8, 16, device=cuda_dev)
    import mamba_rs_b200 as mb
    y = mb.selective_scan_fwd(x, x, x, x, -torch.ones(16, 16, device=cuda_dev), torch.ones(16, device=cuda_dev))
    assert bool(torch.isfinite(y).all())
    assert lib.mamba_b200_selftest_wait_timeout(h.ptr, stream, 0) == -1  # out-of-range limit is refused
