"""GPU parity of the rows around the scan: fused residual + RMSNorm (forward and
backward), embedding gather, softmax cross-entropy and AdamW, against the numpy
restatements in oracle/ (which cite the reference kernels they follow).
Tolerances: 1e-4 of the reference's max-abs for f32 results, 2e-2 for 16-bit ones."""
import numpy as np
import pytest

import oracle
from helpers import TOL, rel_err, to_dev, torch_dtype
from mamba_rs_b200 import synth

pytestmark = pytest.mark.gpu


def host(t):
    return t.float().cpu().numpy()


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(7, 128), (64, 768), (33, 2560), (5, 100), (3, 1), (2, 8192)],
                         ids=lambda s: "rows%d_dim%d" % s)
def test_residual_rmsnorm_forward_and_backward(cuda_dev, shape, dt):
    import torch

    import mamba_rs_b200 as mb
    rows, dim = shape
    rng = np.random.default_rng(rows + dim)
    res0 = rng.standard_normal((rows, dim)).astype(np.float32)
    branch = synth.round_to(rng.standard_normal((rows, dim)).astype(np.float32), dt)
    scale = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    dy = synth.round_to(rng.standard_normal((rows, dim)).astype(np.float32), dt)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    res = d(res0)
    y, rms = mb.residual_rmsnorm_fwd(res, d(branch, td), d(scale), eps=1e-5)
    x_ref, y_ref, rms_ref = oracle.residual_rmsnorm_fwd(res0, branch, scale, 1e-5)
    assert rel_err(host(res), x_ref) <= 1e-6
    assert rel_err(host(rms), rms_ref) <= 1e-5
    assert rel_err(host(y), y_ref) <= TOL[dt]
    # plain RMSNorm (no branch) leaves the residual untouched
    res2 = d(res0)
    y2, _ = mb.residual_rmsnorm_fwd(res2, None, d(scale), out_dtype=td)
    np.testing.assert_array_equal(host(res2), res0)
    assert rel_err(host(y2), oracle.residual_rmsnorm_fwd(res0, None, scale)[1]) <= TOL[dt]
    # backward: += into both outputs
    g0 = rng.standard_normal((rows, dim)).astype(np.float32)
    ds0 = rng.standard_normal(dim).astype(np.float32)
    d_res, d_scale = d(g0), d(ds0)
    mb.residual_rmsnorm_bwd(d(dy, td), res, d(scale), rms, d_res, d_scale)
    torch.cuda.synchronize()
    dx_ref, dsc_ref = oracle.residual_rmsnorm_bwd(dy, host(res), scale, host(rms))
    assert rel_err(host(d_res) - g0, dx_ref) <= 1e-4
    assert rel_err(host(d_scale) - ds0, dsc_ref) <= 1e-4
    mb.ffi.default_handle(0).check_status()


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_embedding_gather(cuda_dev, dt):
    import torch

    import mamba_rs_b200 as mb
    V, dim, rows = 1000, 772, 300
    rng = np.random.default_rng(1)
    table = synth.round_to(rng.standard_normal((V, dim)).astype(np.float32), dt)
    ids = rng.integers(0, V, rows).astype(np.int32)
    ids[5], ids[6] = -1, V  # out of range: zero rows
    out = mb.embedding_gather(to_dev(table, cuda_dev, torch_dtype(dt)), to_dev(ids, cuda_dev))
    torch.cuda.synchronize()
    ref = table[np.clip(ids, 0, V - 1)]
    ref[[5, 6]] = 0.0
    np.testing.assert_array_equal(host(out), ref)


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(9, 50280), (33, 1000), (4, 77), (2, 120000)], ids=lambda s: "rows%d_V%d" % s)
def test_softmax_cross_entropy(cuda_dev, shape, dt):
    import torch

    import mamba_rs_b200 as mb
    rows, V = shape
    rng = np.random.default_rng(V)
    logits = synth.round_to((3.0 * rng.standard_normal((rows, V))).astype(np.float32), dt)
    tg = rng.integers(0, V, rows).astype(np.int32)
    tg[0] = -1  # a row that does not count
    loss, dl = mb.softmax_xent(to_dev(logits, cuda_dev, torch_dtype(dt)), to_dev(tg, cuda_dev), grad_scale=0.5)
    only_loss, none = mb.softmax_xent(to_dev(logits, cuda_dev, torch_dtype(dt)), to_dev(tg, cuda_dev), want_grad=False)
    torch.cuda.synchronize()
    loss_ref, g_ref = oracle.softmax_xent(logits, tg, 0.5)
    assert none is None
    assert rel_err(host(loss), loss_ref) <= 1e-5
    assert rel_err(host(only_loss), loss_ref) <= 1e-5
    assert rel_err(host(dl), g_ref) <= TOL[dt]
    assert float(host(dl)[0].max()) == 0.0 and float(host(loss)[0]) == 0.0
    mb.ffi.default_handle(0).check_status()


@pytest.mark.parametrize("lp", [None, "bf16", "f16"])
def test_adamw_matches_the_reference_update_rule(cuda_dev, lp):
    import torch

    import mamba_rs_b200 as mb
    n = 100003
    rng = np.random.default_rng(2)
    p0, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    m0, v0 = (0.1 * rng.standard_normal(n)).astype(np.float32), rng.random(n).astype(np.float32)
    hp = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
    p_ref, m_ref, v_ref, bc = oracle.adamw_step(p0, g, m0, v0, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["wd"], 7)
    d = lambda a: to_dev(a, cuda_dev)
    p, m, v = d(p0), d(m0), d(v0)
    lp_t = None if lp is None else torch.empty(n, device=cuda_dev, dtype=torch_dtype(lp))
    mb.adamw_step(p, d(g), m, v, d(np.array(bc, np.float32)), lr=hp["lr"], beta1=hp["beta1"], beta2=hp["beta2"],
                  eps=hp["eps"], weight_decay=hp["wd"], param_lp=lp_t)
    torch.cuda.synchronize()
    assert rel_err(host(p), p_ref) <= 1e-6
    assert rel_err(host(m), m_ref) <= 1e-6
    assert rel_err(host(v), v_ref) <= 1e-6
    if lp is not None:
        np.testing.assert_array_equal(host(lp_t), synth.round_to(host(p), lp))
