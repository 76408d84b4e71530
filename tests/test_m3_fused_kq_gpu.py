"""Mamba-3 SSD forward with the per-head K / Q built inside the kernel (bias + RoPE from the
group-level rows) against (1) the oracle's K / Q generation followed by the oracle scan and
(2) this library's own kernel fed the materialised K / Q."""
import numpy as np
import pytest

import oracle
from mamba_rs_b200 import synth
from tests.helpers import TOL, rel_err

pytestmark = pytest.mark.gpu


def _case(B, T, nh, ng, hd, N, na, seed):
    i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=seed)
    g = synth.m3_group_inputs(B, T, nh, ng, N, na, i["dt"], seed=seed)
    return i, g


@pytest.mark.parametrize("dt_name", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [
    # B, T, nh, ng, hd, N, n_angles
    (2, 300, 4, 1, 64, 128, 32),    # rope_fraction 0.5 at the tensor-core geometry
    (1, 260, 4, 2, 64, 128, 64),    # rope_fraction 1.0, two groups
    (2, 129, 2, 1, 32, 64, 16),     # the reference's own limits (hd 32, N 64)
    (1, 200, 2, 2, 16, 32, 8),
    (1, 70, 2, 1, 64, 128, 0),      # no rotation: bias add only
    (1, 1000, 2, 1, 64, 128, 32),   # eight chunks: the carried angle
])
def test_fused_kq_forward_matches_oracle_and_unfused(cuda_dev, shape, dt_name):
    import torch

    import mamba_rs_b200 as mb
    B, T, nh, ng, hd, N, na = shape
    i, g = _case(B, T, nh, ng, hd, N, na, seed=11)
    rnd = lambda a: synth.round_to(a, dt_name)
    x, Bn, Cn = rnd(i["x"]), rnd(g["Bn"]), rnd(g["Cn"])
    tdt = torch.bfloat16 if dt_name == "bf16" else torch.float16
    t = lambda a, d=None: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_dev).to(d or torch.float32)
    vel = g["angle_vel"] if na else None
    Kr, Qr, ang_ref = oracle.m3_kq_from_groups(Bn, Cn, g["b_bias"], g["c_bias"], vel, i["dt"],
                                               g["angle_state"] if na else None)
    Kq, Qq = rnd(Kr), rnd(Qr)  # what the unfused pipeline would store
    ref = oracle.m3_ssd_fwd(x, Kq, Qq, i["dt"], i["trap"], i["adt"], i["Dh"])

    ang = t(g["angle_state"]) if na else None
    ssm = torch.zeros(B, nh, hd, N, device=cuda_dev)
    kst = torch.zeros(B, nh, N, device=cuda_dev)
    vst = torch.zeros(B, nh, hd, device=cuda_dev)
    y = mb.ops.m3_ssd_fwd_fused_kq(t(x, tdt), t(Bn, tdt), t(Cn, tdt), t(g["b_bias"]), t(g["c_bias"]),
                                   t(vel) if na else None, t(i["dt"]), t(i["trap"]), t(i["adt"]), t(i["Dh"]),
                                   angle_state=ang, ssm_state=ssm, k_state=kst, v_state=vst)
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    tol = TOL[dt_name]
    assert rel_err(y.float().cpu().numpy(), ref["y"]) <= tol
    assert rel_err(ssm.cpu().numpy(), ref["ssm_state"]) <= tol
    assert rel_err(kst.cpu().numpy(), Kq[:, -1]) <= tol
    np.testing.assert_array_equal(vst.cpu().numpy(), x[:, -1].reshape(B, nh, hd))
    if na:
        # angles are compared on the circle
        d = np.abs(ang.cpu().numpy() - ang_ref)
        d = np.minimum(d, 2 * np.pi - d)
        assert d.max() <= 1e-3, d.max()

    # the same kernel reading the materialised K / Q
    y2 = mb.m3_ssd_fwd(t(x, tdt), t(Kq, tdt), t(Qq, tdt), t(i["dt"]), t(i["trap"]), t(i["adt"]), t(i["Dh"]))
    assert rel_err(y.float().cpu().numpy(), y2.float().cpu().numpy()) <= tol


def test_fused_kq_refuses_shapes_outside_the_tensor_core_path(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    B, T, nh, ng, hd, N, na = 1, 40, 2, 1, 16, 32, 8
    i, g = _case(B, T, nh, ng, hd, N, na, seed=3)
    t = lambda a, d=None: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_dev).to(d or torch.float32)
    with pytest.raises(Exception):  # f32 storage has no tensor-core path
        mb.ops.m3_ssd_fwd_fused_kq(t(i["x"]), t(g["Bn"]), t(g["Cn"]), t(g["b_bias"]), t(g["c_bias"]),
                                   t(g["angle_vel"]), t(i["dt"]), t(i["trap"]), t(i["adt"]), t(i["Dh"]))
    bf = torch.bfloat16
    with pytest.raises(Exception):  # n_angles must be a multiple of 4
        mb.ops.m3_ssd_fwd_fused_kq(t(i["x"], bf), t(g["Bn"], bf), t(g["Cn"], bf), t(g["b_bias"]), t(g["c_bias"]),
                                   t(g["angle_vel"][:, :, :6]), t(i["dt"]), t(i["trap"]), t(i["adt"]), t(i["Dh"]))
