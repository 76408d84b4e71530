"""The allocation-free conv1d backward (scratch built into the library) must
give the same gradients as the regular entry point that takes a caller
workspace.  For engines that may not allocate device memory on this path.

The file name sorts last on purpose: with `pytest -x` every other test has run
before this one.  It goes through the C ABI directly (ctypes), twice in a row,
because all calls share one scratch array that keeps its previous contents."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _args(ffi, mb, x, w, b, d_u, st0, d_x, dW, db, ws):
    a = ffi.Conv1dArgs()
    Bsz, T, D = x.shape
    a.dtype = mb.dtype_code(x.dtype)
    a.B, a.T, a.D, a.K = Bsz, T, D, w.shape[1]
    a.x, a.ld_x = x.data_ptr(), D
    a.conv_w, a.conv_b, a.conv_state = w.data_ptr(), b.data_ptr(), st0.data_ptr()
    a.d_u, a.ld_du = d_u.data_ptr(), D
    a.d_x, a.ld_dx = d_x.data_ptr(), D
    a.dconv_w, a.dconv_b = dW.data_ptr(), db.data_ptr()
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_static_scratch_entry_matches_workspace_entry_twice(cuda_dev, dt):
    import torch

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import ffi
    lib = ffi.lib()
    lib.mamba_b200_conv1d_bwd_static.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(ffi.Conv1dArgs)]
    lib.mamba_b200_conv1d_bwd_static_max_bytes.restype = C.c_longlong
    h = ffi.default_handle(0)
    td = {"f32": torch.float32, "bf16": torch.bfloat16}[dt]
    stream = C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)
    g = torch.Generator(device="cpu").manual_seed(123)
    # two different problems back to back: the second must not see the first's partials
    for (B, T, D, K) in [(3, 200, 96, 4), (2, 70, 40, 3)]:
        x = torch.randn(B, T, D, generator=g).to(cuda_dev).to(td)
        d_u = torch.randn(B, T, D, generator=g).to(cuda_dev).to(td)
        w = (torch.rand(D, K, generator=g) - 0.5).to(cuda_dev)
        b = (0.1 * torch.randn(D, generator=g)).to(cuda_dev)
        st0 = torch.randn(B, D, K, generator=g).to(cuda_dev)
        need = lib.mamba_b200_conv1d_bwd_workspace_bytes(B, T, D, K)
        assert need <= lib.mamba_b200_conv1d_bwd_static_max_bytes()
        ws = torch.empty(need, dtype=torch.uint8, device=cuda_dev)
        outs = []
        for static in (False, True):
            d_x = torch.empty(B, T, D, device=cuda_dev, dtype=td)
            dW = torch.zeros(D, K, device=cuda_dev)
            db = torch.zeros(D, device=cuda_dev)
            a = _args(ffi, mb, x, w, b, d_u, st0, d_x, dW, db, None if static else ws)
            fn = lib.mamba_b200_conv1d_bwd_static if static else lib.mamba_b200_conv1d_bwd
            rc = fn(h.ptr, stream, C.byref(a))
            assert rc == 0, lib.mamba_b200_last_error(h.ptr)
            torch.cuda.synchronize()
            outs.append((d_x.float().cpu().numpy(), dW.cpu().numpy(), db.cpu().numpy()))
        # same kernels, same order of additions: bit-identical (well inside the
        # 1e-4 / 2e-2 parity tolerance the other tests use)
        for got, ref in zip(outs[1], outs[0]):
            np.testing.assert_array_equal(got, ref)


def test_static_scratch_entry_rejects_oversized_problems(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import ffi
    lib = ffi.lib()
    lib.mamba_b200_conv1d_bwd_static.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(ffi.Conv1dArgs)]
    h = ffi.default_handle(0)
    a = ffi.Conv1dArgs()
    a.dtype, a.B, a.T, a.D, a.K = 0, 64, 8192, 5120, 4  # 64*128*5120*5*4 bytes = 838 MB of partials
    rc = lib.mamba_b200_conv1d_bwd_static(h.ptr, None, C.byref(a))
    assert rc == -2
    assert b"built-in" in lib.mamba_b200_last_error(h.ptr)


def test_static_scratch_entry_without_a_handle_on_a_side_stream(cuda_dev):
    """handle == NULL (failures by return code only) and a non-default stream,
    checked against the CPU oracle rather than against the other entry point."""
    import torch

    import mamba_rs_b200 as mb
    import oracle
    from mamba_rs_b200 import ffi
    lib = ffi.lib()
    lib.mamba_b200_conv1d_bwd_static.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(ffi.Conv1dArgs)]
    ffi.default_handle(0)  # the first call on the device has been made before this one
    B, T, D, K = 2, 130, 48, 4
    rng = np.random.default_rng(9)
    xn = rng.standard_normal((B, T, D)).astype(np.float32)
    dun = rng.standard_normal((B, T, D)).astype(np.float32)
    wn = rng.uniform(-0.8, 0.8, (D, K)).astype(np.float32)
    bn = (0.1 * rng.standard_normal(D)).astype(np.float32)
    sn = rng.standard_normal((B, D, K)).astype(np.float32)
    t = lambda a: torch.from_numpy(a).to(cuda_dev)
    x, d_u, w, b, st0 = t(xn), t(dun), t(wn), t(bn), t(sn)
    d_x, dW, db = torch.empty_like(x), torch.zeros(D, K, device=cuda_dev), torch.zeros(D, device=cuda_dev)
    side = torch.cuda.Stream(device=cuda_dev)
    side.wait_stream(torch.cuda.current_stream(cuda_dev))
    a = _args(ffi, mb, x, w, b, d_u, st0, d_x, dW, db, None)
    rc = lib.mamba_b200_conv1d_bwd_static(None, C.c_void_p(side.cuda_stream), C.byref(a))
    assert rc == 0
    side.synchronize()
    ref = oracle.conv1d_bwd(xn, wn, bn, dun, sn)
    den = lambda r: max(np.abs(r).max(), 1e-30)
    assert np.abs(d_x.cpu().numpy() - ref["d_x"]).max() / den(ref["d_x"]) <= 1e-4
    assert np.abs(dW.cpu().numpy() - ref["dconv_w"]).max() / den(ref["dconv_w"]) <= 2e-4
    assert np.abs(db.cpu().numpy() - ref["dconv_b"]).max() / den(ref["dconv_b"]) <= 2e-4
