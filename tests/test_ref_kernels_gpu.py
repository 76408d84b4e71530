"""Cross-check against the reference's OWN CUDA kernels (compiled from its
sources into oracle/_ref by oracle/build_ref.py and run on this GPU): the CPU
oracle, the reference kernels and this library must agree on the unfused scan
and conv contracts.  Skipped when oracle/_ref was not built."""
import numpy as np
import pytest

import oracle
from helpers import TOL, rel_err, to_dev, torch_dtype
from mamba_rs_b200 import synth
from oracle import ref_kernels

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_kernels.available(), reason="oracle/_ref not built")]


@pytest.fixture(scope="module")
def rk():
    return ref_kernels.RefKernels()


def scan_inputs(B, T, D, N, dt, seed):
    inp = synth.m1_scan_inputs(B, T, D, N, 0, seed, "random", z=False)
    delta = np.log1p(np.exp(inp["delta_raw"].astype(np.float64))).astype(np.float32)
    q = {k: synth.round_to(v, dt) for k, v in dict(u=inp["x"], delta=delta, Bm=inp["Bm"], Cm=inp["Cm"]).items()}
    q["a_neg"], q["Dp"] = inp["a_neg"], inp["Dp"]
    return q


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("kernel", ["parallel", "sequential"])
@pytest.mark.parametrize("shape", [(2, 300, 24, 16), (1, 1500, 4, 8), (2, 256, 8, 16), (1, 40, 40, 16)],
                         ids=lambda s: "B%dT%dD%dN%d" % s)
def test_reference_scan_kernels_agree_with_oracle_and_library(cuda_dev, rk, shape, kernel, dt):
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N = shape
    q = scan_inputs(B, T, D, N, dt, seed=T)
    h0 = np.random.default_rng(T).standard_normal((B, D, N)).astype(np.float32)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    args = (d(q["delta"], td), d(q["u"], td), d(q["Bm"], td), d(q["Cm"], td), d(q["a_neg"]), d(q["Dp"]))
    h_ref, y_ref = d(h0), torch.empty(B, T, D, device=cuda_dev, dtype=td)
    fn = rk.ssm_parallel_scan_fwd_nosave if kernel == "parallel" else rk.ssm_burnin_forward_nosave
    fn(dt, h_ref, y_ref, *args)
    h_lib, y_lib = d(h0), torch.empty(B, T, D, device=cuda_dev, dtype=td)
    mb.ssm_parallel_scan_fwd_nosave(h_lib, y_lib, *args)
    torch.cuda.synchronize()
    orc = oracle.m1_fused_fwd(q["u"], q["delta"], q["Bm"], q["Cm"], None, q["a_neg"], q["Dp"], ssm_state=h0,
                              delta_softplus=False)
    y_ref_n, y_lib_n = y_ref.float().cpu().numpy(), y_lib.float().cpu().numpy()
    # reference GPU kernel vs the CPU restatement: pins the oracle on the reference's own code
    assert rel_err(y_ref_n, orc["y"]) <= TOL[dt]
    assert rel_err(h_ref.cpu().numpy(), orc["ssm_state"]) <= 1e-4
    # this library vs the reference GPU kernel, same arguments
    assert rel_err(y_lib_n, y_ref_n) <= TOL[dt]
    assert rel_err(h_lib.cpu().numpy(), h_ref.cpu().numpy()) <= 1e-4


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_reference_conv_kernel_agrees(cuda_dev, rk, dt):
    import torch

    import mamba_rs_b200 as mb
    B, T, D, K = 2, 150, 40, 4
    rng = np.random.default_rng(3)
    x = synth.round_to(rng.standard_normal((B, T, D)).astype(np.float32), dt)
    w = rng.uniform(-0.8, 0.8, (D, K)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(D)).astype(np.float32)
    st0 = synth.round_to(rng.standard_normal((B, D, K)).astype(np.float32), dt)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    st_ref, u_ref = d(st0), torch.empty(B, T, D, device=cuda_dev, dtype=td)
    rk.conv1d_burnin_forward_nosave(dt, u_ref, st_ref, d(x, td), d(w), d(bias))
    st_lib = d(st0)
    u_lib = mb.conv1d_fwd(d(x, td), d(w), d(bias), st_lib)
    torch.cuda.synchronize()
    orc = oracle.conv1d_fwd(x, w, bias, st0)
    assert rel_err(u_ref.float().cpu().numpy(), orc["u"]) <= TOL[dt]
    assert rel_err(u_lib.float().cpu().numpy(), u_ref.float().cpu().numpy()) <= TOL[dt]
    np.testing.assert_array_equal(st_ref.cpu().numpy(), orc["conv_state"])
    np.testing.assert_array_equal(st_lib.cpu().numpy(), st_ref.cpu().numpy())
