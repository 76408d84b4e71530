"""GPU parity tests of the Mamba-3 SISO SSD forward against the CPU oracle's
sequential definition.  Tolerances as for Mamba-1: 1e-4 (f32 storage), 2e-2
(bf16 / f16 storage), max-abs relative to the max-abs reference."""
import numpy as np
import pytest

import oracle
from helpers import TOL, rel_err, to_dev, torch_dtype
from mamba_rs_b200 import synth

pytestmark = pytest.mark.gpu
ARGS = ("x", "K", "Q", "dt", "trap", "adt", "Dh")


def rounded(i, dt):
    return {k: (synth.round_to(v, dt) if k in ("x", "K", "Q") else v) for k, v in i.items()}


def run_gpu(i, dt, dev, **kw):
    import torch

    import mamba_rs_b200 as mb
    td = torch_dtype(dt)
    B, T, nh, N = i["K"].shape
    hd = i["x"].shape[2] // nh
    ssm = torch.zeros(B, nh, hd, N, device=dev)
    ks = torch.zeros(B, nh, N, device=dev)
    vs = torch.zeros(B, nh, hd, device=dev)
    y = mb.m3_ssd_fwd(to_dev(i["x"], dev, td), to_dev(i["K"], dev, td), to_dev(i["Q"], dev, td),
                      to_dev(i["dt"], dev), to_dev(i["trap"], dev), to_dev(i["adt"], dev), to_dev(i["Dh"], dev),
                      ssm_state=ssm, k_state=ks, v_state=vs, **kw)
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    return y.float().cpu().numpy(), ssm.cpu().numpy(), ks.cpu().numpy(), vs.cpu().numpy()


# shapes of the reference's own unit parity test (tests/m3_chunked_fwd_unit_parity.rs:20-31:
# B=2,T=10,nh=2,hd=4,ds=4), its limits (hd 32, N 64), and beyond them
SEQ_SHAPES = [(2, 10, 2, 4, 4), (1, 64, 3, 16, 16), (2, 100, 2, 32, 64), (1, 70, 2, 64, 128), (1, 33, 1, 8, 24)]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", SEQ_SHAPES, ids=lambda s: "B%dT%dnh%dhd%dN%d" % s)
def test_sequential_kernel_matches_oracle(cuda_dev, shape, dt):
    B, T, nh, hd, N = shape
    i = rounded(synth.m3_ssd_inputs(B, T, nh, hd, N, seed=T), dt)
    ref = oracle.m3_ssd_fwd(*[i[k] for k in ARGS])
    y, ssm, ks, vs = run_gpu(i, dt, cuda_dev, force_sequential=True)
    assert rel_err(y, ref["y"]) <= TOL[dt]
    assert rel_err(ssm, ref["ssm_state"]) <= 1e-4
    np.testing.assert_array_equal(ks, ref["k_state"])
    np.testing.assert_array_equal(vs, ref["v_state"])


def test_sequential_kernel_carries_state(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    i = synth.m3_ssd_inputs(1, 60, 2, 16, 32, seed=5)
    whole = oracle.m3_ssd_fwd(*[i[k] for k in ARGS])
    dev = cuda_dev
    ssm = torch.zeros(1, 2, 16, 32, device=dev)
    ks = torch.zeros(1, 2, 32, device=dev)
    vs = torch.zeros(1, 2, 16, device=dev)
    ys = []
    for lo, hi, carry in ((0, 25, False), (25, 60, True)):
        sl = {k: (np.ascontiguousarray(i[k][:, lo:hi]) if k != "Dh" else i[k]) for k in ARGS}
        ys.append(mb.m3_ssd_fwd(*[to_dev(sl[k], dev) for k in ARGS], ssm_state=ssm, k_state=ks, v_state=vs,
                                carry_in=carry))
    torch.cuda.synchronize()
    assert rel_err(torch.cat(ys, 1).cpu().numpy(), whole["y"]) <= 1e-5
    assert rel_err(ssm.cpu().numpy(), whole["ssm_state"]) <= 1e-5


# tensor-core path: hd = 64, N = 128, 16-bit storage; T around the 128-step chunk
TC_SHAPES = [(1, 128, 1), (2, 256, 2), (1, 1, 1), (1, 100, 2), (1, 129, 1), (2, 300, 3), (1, 1000, 2)]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("shape", TC_SHAPES, ids=lambda s: "B%dT%dnh%d" % s)
def test_tensor_core_kernel_matches_oracle(cuda_dev, shape, dt):
    B, T, nh = shape
    i = rounded(synth.m3_ssd_inputs(B, T, nh, 64, 128, seed=T + 1), dt)
    ref = oracle.m3_ssd_fwd(*[i[k] for k in ARGS])
    y, ssm, ks, vs = run_gpu(i, dt, cuda_dev)
    assert rel_err(y, ref["y"]) <= TOL[dt]
    assert rel_err(ssm, ref["ssm_state"]) <= TOL[dt]  # 16-bit operands feed the state GEMM
    np.testing.assert_array_equal(ks, ref["k_state"])
    np.testing.assert_array_equal(vs, ref["v_state"])


# the reference's own limits (headdim 32, d_state 64) and other multiples of 8: the
# kernel pads its tiles to 64 / 128 columns with zeros
PADDED_SHAPES = [(2, 200, 2, 32, 64), (1, 130, 3, 8, 8), (1, 300, 2, 24, 40), (1, 129, 1, 64, 16), (1, 64, 2, 16, 128)]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("shape", PADDED_SHAPES, ids=lambda s: "B%dT%dnh%dhd%dN%d" % s)
def test_tensor_core_kernel_with_padded_head_and_state_dims(cuda_dev, shape, dt):
    B, T, nh, hd, N = shape
    i = rounded(synth.m3_ssd_inputs(B, T, nh, hd, N, seed=T + hd), dt)
    ref = oracle.m3_ssd_fwd(*[i[k] for k in ARGS])
    y, ssm, ks, vs = run_gpu(i, dt, cuda_dev)
    assert rel_err(y, ref["y"]) <= TOL[dt]
    assert rel_err(ssm, ref["ssm_state"]) <= TOL[dt]
    np.testing.assert_array_equal(ks, ref["k_state"])
    np.testing.assert_array_equal(vs, ref["v_state"])
    y2, ssm2, _, _ = run_gpu(i, dt, cuda_dev, force_sequential=True)
    assert rel_err(y, y2) <= TOL[dt]


def test_tensor_core_and_sequential_kernels_agree(cuda_dev):
    i = rounded(synth.m3_ssd_inputs(2, 520, 4, 64, 128, seed=9), "bf16")
    y1, s1, _, _ = run_gpu(i, "bf16", cuda_dev)
    y2, s2, _, _ = run_gpu(i, "bf16", cuda_dev, force_sequential=True)
    assert rel_err(y1, y2) <= TOL["bf16"]
    assert rel_err(s1, s2) <= TOL["bf16"]


def test_tensor_core_kernel_at_config4_size_agrees_with_sequential_and_is_linear_in_x(cuda_dev):
    """Benchmark geometry (B 8, L 4096, 32 heads x 64, d_state 128, bf16): the
    tcgen05 kernel against the sequential kernel on the same device tensors, and
    the size-independent property y(x1 + x2) = y(x1) + y(x2) - y(0) with y(0) = 0."""
    import torch

    import mamba_rs_b200 as mb
    B, T, nh, hd, N = 8, 4096, 32, 64, 128
    g = torch.Generator(device="cpu").manual_seed(4)
    bf = torch.bfloat16
    dev = cuda_dev
    x1 = torch.randn(B, T, nh * hd, generator=g).to(dev).to(bf)
    x2 = torch.randn(B, T, nh * hd, generator=g).to(dev).to(bf)
    K = (torch.randn(B, T, nh, N, generator=g) * N ** -0.25).to(dev).to(bf)
    Q = (torch.randn(B, T, nh, N, generator=g) * N ** -0.25).to(dev).to(bf)
    A = -torch.exp(torch.rand(nh, generator=g) * np.log(16.0))
    dt = torch.nn.functional.softplus(0.5 * torch.randn(B, T, nh, generator=g) - 4.0)
    trap = torch.sigmoid(torch.randn(B, T, nh, generator=g))
    adt = (A * dt).to(dev).contiguous()
    dt, trap = dt.to(dev).contiguous(), trap.to(dev).contiguous()
    Dh = torch.ones(nh, device=dev)
    s_tc = torch.zeros(B, nh, hd, N, device=dev)
    s_seq = torch.zeros(B, nh, hd, N, device=dev)
    y_tc = mb.m3_ssd_fwd(x1, K, Q, dt, trap, adt, Dh, ssm_state=s_tc).float()
    y_seq = mb.m3_ssd_fwd(x1, K, Q, dt, trap, adt, Dh, ssm_state=s_seq, force_sequential=True).float()
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    den = y_seq.abs().max()
    assert float((y_tc - y_seq).abs().max() / den) <= TOL["bf16"]
    assert float((s_tc - s_seq).abs().max() / s_seq.abs().max()) <= TOL["bf16"]
    del y_seq
    x12 = (x1.float() + x2.float()).to(bf)  # rounding of the sum stays inside the tolerance
    y2 = mb.m3_ssd_fwd(x2, K, Q, dt, trap, adt, Dh).float()
    y12 = mb.m3_ssd_fwd(x12, K, Q, dt, trap, adt, Dh).float()
    torch.cuda.synchronize()
    assert float((y12 - (y_tc + y2)).abs().max() / y12.abs().max()) <= TOL["bf16"]
