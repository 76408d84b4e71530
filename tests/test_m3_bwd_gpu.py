"""GPU parity tests of the Mamba-3 SISO SSD backward against the CPU oracle's
sequential BPTT (the oracle follows kernels/mamba3_ssd.cu:558-808).  f32
outputs: 1e-4 of the reference's max-abs; dx in 16-bit storage: 2e-2.  The
tensor-core path (16-bit storage, headdim <= 64 and d_state <= 128 in multiples
of 8, zero-padded to 64 / 128 inside the kernel) rounds its MMA
operands to the storage dtype, so all of its outputs are held to 2e-2."""
import numpy as np
import pytest

import oracle
from helpers import TOL, rel_err, to_dev, torch_dtype
from mamba_rs_b200 import synth

pytestmark = pytest.mark.gpu
ARGS = ("x", "K", "Q", "dt", "trap", "adt", "Dh")
F32_OUT = ("dK", "dQ", "d_adt", "d_dt", "d_trap", "dD")


def case(shape, dt, seed):
    B, T, nh, hd, N = shape
    i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=seed)
    i = {k: (synth.round_to(v, dt) if k in ("x", "K", "Q") else v) for k, v in i.items()}
    dy = synth.round_to(np.random.default_rng(seed + 1).standard_normal(i["x"].shape).astype(np.float32), dt)
    return i, dy


def run_gpu(i, dy, dt, dev, **kw):
    import torch

    import mamba_rs_b200 as mb
    td = torch_dtype(dt)
    out = mb.m3_ssd_bwd(to_dev(i["x"], dev, td), to_dev(i["K"], dev, td), to_dev(i["Q"], dev, td),
                        to_dev(i["dt"], dev), to_dev(i["trap"], dev), to_dev(i["adt"], dev),
                        to_dev(i["Dh"], dev), to_dev(dy, dev, td), **kw)
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    return {k: v.float().cpu().numpy() for k, v in out.items()}


# the reference's unit-parity shape (tests/m3_chunked_fwd_unit_parity.rs:20-31), ragged
# lengths around the 32-step chunk, the reference's limits (hd 32, N 64) and beyond
SHAPES = [(2, 10, 2, 4, 4), (1, 32, 2, 8, 16), (2, 33, 1, 16, 16), (1, 100, 3, 32, 64), (1, 97, 2, 64, 128),
          (2, 1, 2, 8, 8), (1, 160, 1, 24, 40), (2, 128, 2, 64, 128), (1, 300, 3, 64, 128), (1, 513, 1, 64, 128)]


def on_tensor_cores(shape, dt):
    hd, N = shape[3], shape[4]
    return dt != "f32" and hd <= 64 and hd % 8 == 0 and N <= 128 and N % 8 == 0


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "B%dT%dnh%dhd%dN%d" % s)
def test_backward_matches_oracle(cuda_dev, shape, dt):
    i, dy = case(shape, dt, seed=shape[1])
    ref = oracle.m3_ssd_bwd(*[i[k] for k in ARGS], dy)
    got = run_gpu(i, dy, dt, cuda_dev)
    assert rel_err(got["dx"], ref["dx"]) <= TOL[dt]
    tol = TOL[dt] if on_tensor_cores(shape, dt) else 1e-4
    for k in F32_OUT:
        assert rel_err(got[k], ref[k]) <= tol, k


def test_tensor_core_path_matches_cuda_core_path_at_model_size(cuda_dev):
    """bf16, headdim 64, d_state 128, T = 1024: the tcgen05 kernel against the f32
    CUDA-core kernel fed the same bf16-rounded values as f32 tensors."""
    shape = (2, 1024, 4, 64, 128)
    i, dy = case(shape, "bf16", seed=33)
    tcg = run_gpu(i, dy, "bf16", cuda_dev)
    ccg = run_gpu(i, dy, "f32", cuda_dev)
    for k in ("dx", "dK", "dQ", "d_adt", "d_dt", "d_trap", "dD"):
        assert rel_err(tcg[k], ccg[k]) <= TOL["bf16"], k


def test_dD_accumulates_and_rerun_is_identical(cuda_dev):
    import torch
    i, dy = case((2, 70, 2, 16, 32), "f32", seed=9)
    a = run_gpu(i, dy, "f32", cuda_dev)
    pre = torch.full((2,), 3.0, device=cuda_dev)
    b = run_gpu(i, dy, "f32", cuda_dev, dD=pre)
    np.testing.assert_allclose(b["dD"], a["dD"] + 3.0, rtol=1e-6)
    for k in ("dx", "dK", "dQ", "d_adt", "d_dt", "d_trap"):
        np.testing.assert_array_equal(a[k], b[k])


def test_gradient_is_linear_in_dy_at_model_size(cuda_dev):
    """Size-independent property at the benchmark's head geometry (hd 64, N 128,
    T a multiple of the chunk): bwd(a*dy1 + dy2) = a*bwd(dy1) + bwd(dy2)."""
    shape = (2, 512, 4, 64, 128)
    i, dy1 = case(shape, "f32", seed=21)
    dy2 = np.random.default_rng(5).standard_normal(dy1.shape).astype(np.float32)
    g1, g2 = run_gpu(i, dy1, "f32", cuda_dev), run_gpu(i, dy2, "f32", cuda_dev)
    g3 = run_gpu(i, (0.5 * dy1 + dy2).astype(np.float32), "f32", cuda_dev)
    for k in ("dx", "dK", "dQ", "d_adt", "d_dt", "d_trap", "dD"):
        assert rel_err(g3[k], 0.5 * g1[k] + g2[k]) <= 1e-4, k


def test_backward_validation(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    i, dy = case((1, 8, 1, 8, 8), "f32", seed=1)
    t = {k: to_dev(v, cuda_dev) for k, v in i.items() if k in ARGS}
    with pytest.raises(RuntimeError, match="workspace"):
        mb.m3_ssd_bwd(*[t[k] for k in ARGS], to_dev(dy, cuda_dev),
                      workspace=torch.empty(256, dtype=torch.uint8, device=cuda_dev))
    big = synth.m3_ssd_inputs(1, 4, 1, 96, 8, seed=0)
    tb = {k: to_dev(v, cuda_dev) for k, v in big.items() if k in ARGS}
    with pytest.raises(RuntimeError, match="headdim"):
        mb.m3_ssd_bwd(*[tb[k] for k in ARGS], torch.zeros_like(tb["x"]))


def test_tensor_core_backward_is_linear_in_dy_at_config4_size(cuda_dev):
    """Benchmark geometry (B 8, L 4096, 32 heads x 64, d_state 128, bf16):
    bwd(dy1 + dy2) = bwd(dy1) + bwd(dy2), every output, on the tcgen05 path."""
    import torch

    import mamba_rs_b200 as mb
    B, T, nh, hd, N = 8, 4096, 32, 64, 128
    g = torch.Generator(device="cpu").manual_seed(6)
    bf = torch.bfloat16
    dev = cuda_dev
    x = torch.randn(B, T, nh * hd, generator=g).to(dev).to(bf)
    dy1 = torch.randn(B, T, nh * hd, generator=g).to(dev).to(bf)
    dy2 = torch.randn(B, T, nh * hd, generator=g).to(dev).to(bf)
    K = (torch.randn(B, T, nh, N, generator=g) * N ** -0.25).to(dev).to(bf)
    Q = (torch.randn(B, T, nh, N, generator=g) * N ** -0.25).to(dev).to(bf)
    A = -torch.exp(torch.rand(nh, generator=g) * np.log(16.0))
    dt = torch.nn.functional.softplus(0.5 * torch.randn(B, T, nh, generator=g) - 4.0)
    trap = torch.sigmoid(torch.randn(B, T, nh, generator=g))
    adt = (A * dt).to(dev).contiguous()
    dt, trap = dt.to(dev).contiguous(), trap.to(dev).contiguous()
    Dh = torch.ones(nh, device=dev)
    ws = torch.empty(mb.ffi.lib().mamba_b200_m3_ssd_bwd_workspace_bytes(B, T, nh, hd, N), dtype=torch.uint8,
                     device=dev)
    run = lambda dy: mb.m3_ssd_bwd(x, K, Q, dt, trap, adt, Dh, dy, workspace=ws)
    g1, g2 = run(dy1), run(dy2)
    g12 = run((dy1.float() + dy2.float()).to(bf))
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    for k in ("dx", "dK", "dQ", "d_adt", "d_dt", "d_trap", "dD"):
        want = g1[k].float() + g2[k].float()
        err = float((g12[k].float() - want).abs().max() / want.abs().max())
        assert err <= TOL["bf16"], (k, err)
