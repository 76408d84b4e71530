"""GPU parity tests of the decode step and the standalone conv1d kernels
against the CPU oracle (tolerances as in test_m1_fwd_gpu.py)."""
import numpy as np
import pytest

import oracle
from helpers import TOL, quantised_inputs, random_states, rel_err, to_dev, torch_dtype
from mamba_rs_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(1, 32, 16, 4), (3, 100, 16, 4), (2, 48, 8, 3), (2, 7, 12, 2), (4, 64, 64, 4)],
                         ids=lambda s: "B%dD%dN%dK%d" % s)
def test_decode_steps_track_oracle(cuda_dev, shape, dt):
    """A run of decode steps from a random state: every step's y and the final
    states match the oracle's step function (cpu/inference.rs:88-210)."""
    import torch

    import mamba_rs_b200 as mb
    B, D, N, K = shape
    steps = 6
    q = quantised_inputs(B, steps, D, N, K, dt, seed=D + N, a_mode="random")
    ssm0, cst0 = random_states(B, D, N, K, seed=5)
    td = torch_dtype(dt)
    ssm, cst = to_dev(ssm0, cuda_dev), to_dev(cst0, cuda_dev)
    a, Dp = to_dev(q["a_neg"], cuda_dev), to_dev(q["Dp"], cuda_dev)
    cw, cb = to_dev(q["conv_w"], cuda_dev), to_dev(q["conv_b"], cuda_dev)
    rs, rc = ssm0, cst0
    for t in range(steps):
        ref = oracle.m1_step(q["x"][:, t], q["delta_raw"][:, t], q["Bm"][:, t], q["Cm"][:, t], q["z"][:, t],
                             q["a_neg"], q["Dp"], q["conv_w"], q["conv_b"], rc, rs)
        rs, rc = ref["ssm_state"], ref["conv_state"]
        y = mb.selective_scan_step(to_dev(q["x"][:, t], cuda_dev, td), to_dev(q["delta_raw"][:, t], cuda_dev, td),
                                   to_dev(q["Bm"][:, t], cuda_dev, td), to_dev(q["Cm"][:, t], cuda_dev, td),
                                   a, Dp, ssm, to_dev(q["z"][:, t], cuda_dev, td), conv_w=cw, conv_b=cb,
                                   conv_state=cst)
        torch.cuda.synchronize()
        assert rel_err(y.float().cpu().numpy(), ref["y"]) <= TOL[dt]
    assert rel_err(ssm.cpu().numpy(), rs) <= 1e-4
    np.testing.assert_array_equal(cst.cpu().numpy(), rc)


def test_prefill_then_decode_handoff(cuda_dev):
    """Sequence forward followed by decode steps == one longer sequence forward
    (GpuMambaBackbone prefill_sequence -> step)."""
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N, K, extra = 2, 50, 64, 16, 4, 5
    q = quantised_inputs(B, T + extra, D, N, K, "f32", seed=77)
    whole = oracle.m1_fused_fwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q["z"], q["a_neg"], q["Dp"],
                                q["conv_w"], q["conv_b"])
    d = lambda a: to_dev(a, cuda_dev)
    ssm = torch.zeros(B, D, N, device=cuda_dev)
    cst = torch.zeros(B, D, K, device=cuda_dev)
    c = lambda a: d(np.ascontiguousarray(a[:, :T]))
    y0 = mb.selective_scan_fwd(c(q["x"]), c(q["delta_raw"]), c(q["Bm"]), c(q["Cm"]), d(q["a_neg"]), d(q["Dp"]),
                               c(q["z"]), conv_w=d(q["conv_w"]), conv_b=d(q["conv_b"]), conv_state=cst,
                               ssm_state=ssm)
    ys = [y0]
    for t in range(T, T + extra):
        ys.append(mb.selective_scan_step(d(q["x"][:, t]), d(q["delta_raw"][:, t]), d(q["Bm"][:, t]),
                                         d(q["Cm"][:, t]), d(q["a_neg"]), d(q["Dp"]), ssm, d(q["z"][:, t]),
                                         conv_w=d(q["conv_w"]), conv_b=d(q["conv_b"]), conv_state=cst)[:, None])
    torch.cuda.synchronize()
    got = torch.cat(ys, dim=1).cpu().numpy()
    assert rel_err(got, whole["y"]) <= 1e-4
    assert rel_err(ssm.cpu().numpy(), whole["ssm_state"]) <= 1e-4
    np.testing.assert_array_equal(cst.cpu().numpy(), whole["conv_state"])


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(2, 1, 16, 4), (1, 3, 5, 4), (2, 64, 48, 4), (1, 65, 130, 4), (2, 200, 33, 3),
                                   (1, 130, 8, 2), (1, 70, 12, 1), (1, 129, 20, 8), (1, 100, 1024, 4), (2, 40, 520, 3)],
                         ids=lambda s: "B%dT%dD%dK%d" % s)
def test_conv1d_forward_and_backward_match_oracle(cuda_dev, shape, dt):
    import torch

    import mamba_rs_b200 as mb
    B, T, D, K = shape
    rng = np.random.default_rng(T * 7 + D)
    x = synth.round_to(rng.standard_normal((B, T, D)).astype(np.float32), dt)
    w = rng.uniform(-0.8, 0.8, (D, K)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(D)).astype(np.float32)
    st0 = synth.round_to(rng.standard_normal((B, D, K)).astype(np.float32), dt)
    d_u = synth.round_to(rng.standard_normal((B, T, D)).astype(np.float32), dt)
    td = torch_dtype(dt)
    ref_f = oracle.conv1d_fwd(x, w, bias, st0)
    ref_b = oracle.conv1d_bwd(x, w, bias, d_u, st0)
    st = to_dev(st0, cuda_dev)
    u = mb.conv1d_fwd(to_dev(x, cuda_dev, td), to_dev(w, cuda_dev), to_dev(bias, cuda_dev), st)
    g = mb.conv1d_bwd(to_dev(x, cuda_dev, td), to_dev(w, cuda_dev), to_dev(bias, cuda_dev),
                      to_dev(d_u, cuda_dev, td), to_dev(st0, cuda_dev))
    torch.cuda.synchronize()
    tol = TOL[dt]
    assert rel_err(u.float().cpu().numpy(), ref_f["u"]) <= tol
    np.testing.assert_array_equal(st.cpu().numpy(), ref_f["conv_state"])
    assert rel_err(g["d_x"].float().cpu().numpy(), ref_b["d_x"]) <= tol
    assert rel_err(g["dconv_w"].cpu().numpy(), ref_b["dconv_w"]) <= max(tol, 2e-4)
    assert rel_err(g["dconv_b"].cpu().numpy(), ref_b["dconv_b"]) <= max(tol, 2e-4)


def test_conv_then_scan_equals_fused_conv_scan(cuda_dev):
    """conv1d_fwd followed by the scan on u == the scan with the conv fused in."""
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N, K = 2, 120, 64, 16, 4
    q = quantised_inputs(B, T, D, N, K, "f32", seed=8)
    d = lambda a: to_dev(a, cuda_dev)
    args = (d(q["delta_raw"]), d(q["Bm"]), d(q["Cm"]), d(q["a_neg"]), d(q["Dp"]), d(q["z"]))
    y_fused = mb.selective_scan_fwd(d(q["x"]), *args, conv_w=d(q["conv_w"]), conv_b=d(q["conv_b"]))
    u = mb.conv1d_fwd(d(q["x"]), d(q["conv_w"]), d(q["conv_b"]))
    y_split = mb.selective_scan_fwd(u, *args)
    torch.cuda.synchronize()
    assert rel_err(y_split.cpu().numpy(), y_fused.cpu().numpy()) <= 1e-6


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_decode_step_with_state_slices_that_are_only_4_byte_aligned(cuda_dev, dt):
    """a_neg and ssm_state as slices of flat f32 arenas (the reference keeps weights and
    state that way): bases 4 bytes off a 16-byte boundary take the scalar state path."""
    import torch

    import mamba_rs_b200 as mb
    B, D, N, K = 3, 40, 16, 4
    q = quantised_inputs(B, 1, D, N, K, dt, seed=77, a_mode="random")
    ssm0, cst0 = random_states(B, D, N, K, seed=78)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    arena_a = torch.zeros(D * N + 1, device=cuda_dev)
    arena_h = torch.zeros(B * D * N + 1, device=cuda_dev)
    a_neg = arena_a[1:].view(D, N)
    ssm = arena_h[1:].view(B, D, N)
    a_neg.copy_(d(q["a_neg"]))
    ssm.copy_(d(ssm0))
    assert a_neg.data_ptr() % 16 == 4 and ssm.data_ptr() % 16 == 4
    cst = d(cst0)
    y = mb.selective_scan_step(d(q["x"][:, 0], td), d(q["delta_raw"][:, 0], td), d(q["Bm"][:, 0], td),
                               d(q["Cm"][:, 0], td), a_neg, d(q["Dp"]), ssm, d(q["z"][:, 0], td),
                               conv_w=d(q["conv_w"]), conv_b=d(q["conv_b"]), conv_state=cst)
    torch.cuda.synchronize()
    ref = oracle.m1_step(q["x"][:, 0], q["delta_raw"][:, 0], q["Bm"][:, 0], q["Cm"][:, 0], q["z"][:, 0], q["a_neg"],
                         q["Dp"], q["conv_w"], q["conv_b"], cst0, ssm0)
    assert rel_err(y.float().cpu().numpy(), ref["y"]) <= TOL[dt]
    assert rel_err(ssm.cpu().numpy(), ref["ssm_state"]) <= 1e-4
