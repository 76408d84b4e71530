"""Pins the backward oracle and the Mamba-3 oracle on the reference's OWN CUDA
kernels (compiled unchanged from its sources into oracle/_ref by
oracle/build_ref.py and launched on this GPU with the reference's grids):

    reference kernel  ~  CPU oracle  ~  this library

on the shapes of the reference's kernel-parity tests
(tests/m1_parallel_bwd_parity.rs:290-366, tests/m3_chunked_fwd_unit_parity.rs:20-31)
plus larger ones inside the reference's limits (headdim <= 32, d_state <= 64,
chunk 64).  Tolerances: max-abs error / max-abs reference <= 1e-4 for f32
storage, 2e-2 for bf16 / f16 storage.  Skipped when oracle/_ref was not built."""
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


def host(t):
    return t.float().cpu().numpy()


# ---------------------------------------------------------------- Mamba-1 scan backward

# (1,32,4,4) ... (1,3072,4,8): the reference's own parallel-vs-sequential backward shapes
M1_BWD_SHAPES = [(1, 32, 4, 4), (1, 2048, 4, 8), (1, 1500, 4, 8), (2, 256, 8, 16), (1, 3072, 4, 8),
                 (2, 300, 24, 16)]


def m1_case(B, T, D, N, dt, seed):
    inp = synth.m1_scan_inputs(B, T, D, N, 0, seed, "random", z=False)
    delta = np.log1p(np.exp(inp["delta_raw"].astype(np.float64))).astype(np.float32)
    q = {k: synth.round_to(v, dt) for k, v in dict(u=inp["x"], delta=delta, Bm=inp["Bm"], Cm=inp["Cm"]).items()}
    q["a_neg"], q["Dp"] = inp["a_neg"], inp["Dp"]
    rng = np.random.default_rng(seed + 7)
    q["dy"] = synth.round_to(rng.standard_normal((B, T, D)).astype(np.float32), dt)
    q["h0"] = rng.standard_normal((B, D, N)).astype(np.float32)
    return q


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("kind", ["parallel", "sequential"])
@pytest.mark.parametrize("shape", M1_BWD_SHAPES, ids=lambda s: "B%dT%dD%dN%d" % s)
def test_reference_scan_backward_agrees_with_oracle_and_library(cuda_dev, rk, shape, kind, dt):
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N = shape
    q = m1_case(B, T, D, N, dt, seed=T + N)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    delta, u, Bm, Cm, dy = (d(q[k], td) for k in ("delta", "u", "Bm", "Cm", "dy"))
    a_neg, Dp = d(q["a_neg"]), d(q["Dp"])
    # reference: saving forward (h_saved [B,T+1,D,N]) then its backward + reducers
    h = d(q["h0"])
    y_ref = torch.empty(B, T, D, device=cuda_dev, dtype=td)
    h_saved = torch.empty(B, T + 1, D, N, device=cuda_dev)
    fwd = rk.ssm_parallel_scan_fwd if kind == "parallel" else rk.ssm_burnin_forward
    fwd(dt, h, y_ref, h_saved, delta, u, Bm, Cm, a_neg, Dp)
    ref = rk.ssm_scan_bwd(kind, dt, h_saved, delta, u, Bm, Cm, a_neg, Dp, dy)
    # this library: forward saving block-boundary states, then the fused backward
    S = 32
    cs = torch.empty(B, (T + S - 1) // S, D, N, device=cuda_dev)
    mb.selective_scan_fwd(u, delta, Bm, Cm, a_neg, Dp, None, ssm_state=d(q["h0"]), chunk_states=cs,
                          save_stride=S, delta_softplus=False)
    lib = mb.selective_scan_bwd(u, delta, Bm, Cm, a_neg, Dp, dy, cs, S, None, delta_softplus=False)
    torch.cuda.synchronize()
    orc = oracle.m1_fused_bwd(q["u"], q["delta"], q["Bm"], q["Cm"], None, q["a_neg"], q["Dp"], q["dy"],
                              ssm_state0=q["h0"], delta_softplus=False)
    tol = TOL[dt]
    pairs = (("d_u", "d_x"), ("d_delta", "d_delta"), ("dB", "dB"), ("dC", "dC"), ("dA_log", "dA_log"),
             ("dD", "dD"))
    for gk, ok in pairs:
        # the reference's own kernels pin the CPU restatement ...
        assert rel_err(host(ref[gk]), orc[ok]) <= tol, ("reference vs oracle", gk)
        # ... and this library matches the reference kernels on the same arguments
        assert rel_err(host(lib[gk]), host(ref[gk])) <= tol, ("library vs reference", gk)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 256, 8, 16), (1, 1500, 4, 8), (2, 300, 24, 16)], ids=lambda s: "B%dT%dD%dN%d" % s)
def test_entry_points_on_the_reference_kernels_own_buffers(cuda_dev, rk, shape, dt):
    """mamba_b200_ssm_scan_bwd reads the block-boundary rows straight out of the h_saved the
    REFERENCE's saving forward wrote, and out of the sparse h_saved this library's
    mamba_b200_ssm_scan_fwd_save writes: both must give the reference backward's gradients."""
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N = shape
    q = m1_case(B, T, D, N, dt, seed=T + 3 * N)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    delta, u, Bm, Cm, dy = (d(q[k], td) for k in ("delta", "u", "Bm", "Cm", "dy"))
    a_neg, Dp = d(q["a_neg"]), d(q["Dp"])
    h_ref, y_ref = d(q["h0"]), torch.empty(B, T, D, device=cuda_dev, dtype=td)
    hs_ref = torch.empty(B, T + 1, D, N, device=cuda_dev)
    rk.ssm_parallel_scan_fwd(dt, h_ref, y_ref, hs_ref, delta, u, Bm, Cm, a_neg, Dp)
    ref = rk.ssm_scan_bwd("parallel", dt, hs_ref, delta, u, Bm, Cm, a_neg, Dp, dy)
    h_lib, y_lib = d(q["h0"]), torch.empty(B, T, D, device=cuda_dev, dtype=td)
    hs_lib = torch.full((B, T + 1, D, N), float("nan"), device=cuda_dev)
    mb.ssm_scan_fwd_save(h_lib, y_lib, hs_lib, delta, u, Bm, Cm, a_neg, Dp)
    g_on_ref = mb.ssm_scan_bwd(hs_ref, delta, u, Bm, Cm, a_neg, Dp, dy)
    g_on_lib = mb.ssm_scan_bwd(hs_lib, delta, u, Bm, Cm, a_neg, Dp, dy)
    torch.cuda.synchronize()
    tol = TOL[dt]
    assert rel_err(host(y_lib), host(y_ref)) <= tol
    assert rel_err(host(h_lib), host(h_ref)) <= 1e-4
    rows = list(range(0, T, 32))
    assert rel_err(host(hs_lib[:, rows]), host(hs_ref[:, rows])) <= 1e-4   # the rows that are written
    assert bool(torch.isnan(hs_lib[:, 1]).all())                          # and nothing else
    for g in (g_on_ref, g_on_lib):
        for k in ("d_delta", "d_u", "dB", "dC", "dD", "dA_log"):
            assert rel_err(host(g[k]), host(ref[k])) <= tol, k


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_conv_nosave_entry_point_on_the_reference_argument_list(cuda_dev, rk, dt):
    import torch

    import mamba_rs_b200 as mb
    B, T, D, K = 2, 130, 40, 4
    rng = np.random.default_rng(5)
    x = synth.round_to(rng.standard_normal((B, T, D)).astype(np.float32), dt)
    w = rng.uniform(-0.8, 0.8, (D, K)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(D)).astype(np.float32)
    st0 = rng.standard_normal((B, D, K)).astype(np.float32)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    st_ref, u_ref = d(st0), torch.empty(B, T, D, device=cuda_dev, dtype=td)
    rk.conv1d_burnin_forward_nosave(dt, u_ref, st_ref, d(x, td), d(w), d(bias))
    st_lib, u_lib = d(st0), torch.empty(B, T, D, device=cuda_dev, dtype=td)
    mb.conv1d_fwd_nosave(u_lib, st_lib, d(x, td), d(w), d(bias))
    torch.cuda.synchronize()
    assert rel_err(host(u_lib), host(u_ref)) <= TOL[dt]
    np.testing.assert_array_equal(host(st_lib), host(st_ref))


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(2, 150, 40, 4), (1, 700, 24, 4), (3, 64, 8, 2)],
                         ids=lambda s: "B%dT%dD%dK%d" % s)
def test_reference_conv_backward_agrees(cuda_dev, rk, shape, dt):
    import torch

    import mamba_rs_b200 as mb
    B, T, D, K = shape
    rng = np.random.default_rng(T)
    x = synth.round_to(rng.standard_normal((B, T, D)).astype(np.float32), dt)
    d_u = synth.round_to(rng.standard_normal((B, T, D)).astype(np.float32), dt)
    w = rng.uniform(-0.8, 0.8, (D, K)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(D)).astype(np.float32)
    st0 = rng.standard_normal((B, D, K)).astype(np.float32)
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    ref = rk.conv1d_fwd_bwd(dt, d(st0), d(x, td), d(w), d(bias), d(d_u, td))
    lib = mb.conv1d_bwd(d(x, td), d(w), d(bias), d(d_u, td), d(st0))
    torch.cuda.synchronize()
    orc = oracle.conv1d_bwd(x, w, bias, d_u, st0)
    tol = TOL[dt]
    for k in ("d_x", "dconv_w", "dconv_b"):
        assert rel_err(host(ref[k]), orc[k]) <= tol, ("reference vs oracle", k)
        assert rel_err(host(lib[k]), host(ref[k])) <= tol, ("library vs reference", k)


# ---------------------------------------------------------------- Mamba-3

M3_ARGS = ("x", "K", "Q", "dt", "trap", "adt", "Dh")


def m3_case(shape, dt, seed):
    B, T, nh, hd, N = shape
    i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=seed)
    i = {k: (synth.round_to(v, dt) if k in ("x", "K", "Q") else v) for k, v in i.items()}
    i["dy"] = synth.round_to(np.random.default_rng(seed + 1).standard_normal(i["x"].shape).astype(np.float32), dt)
    alpha = np.exp(i["adt"].astype(np.float64)).astype(np.float32)
    i["alpha"] = alpha
    i["beta"] = (alpha * i["dt"] * (1.0 - i["trap"])).astype(np.float32)
    i["gamma"] = (i["trap"] * i["dt"]).astype(np.float32)
    return i


def m3_dev(i, dt, dev):
    td = torch_dtype(dt)
    out = {k: to_dev(i[k], dev, td) for k in ("x", "K", "Q", "dy")}
    out.update({k: to_dev(i[k], dev) for k in ("dt", "trap", "adt", "Dh", "alpha", "beta", "gamma")})
    return out


# first: the reference's unit-parity geometry (partial last chunk of 4 comes with CS = 4 below)
M3_SEQ_SHAPES = [(2, 10, 2, 4, 4), (1, 64, 2, 16, 16), (2, 200, 2, 32, 64), (1, 257, 3, 8, 32)]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", M3_SEQ_SHAPES, ids=lambda s: "B%dT%dnh%dhd%dN%d" % s)
def test_reference_m3_sequential_forward(cuda_dev, rk, shape, dt):
    """m3_burnin_fwd[_{dt}] from a random carried state ~ oracle ~ library (carry_in)."""
    import torch

    import mamba_rs_b200 as mb
    B, T, nh, hd, N = shape
    i = m3_case(shape, dt, seed=T)
    g = m3_dev(i, dt, cuda_dev)
    rng = np.random.default_rng(T + 3)
    s0 = rng.standard_normal((B, nh, hd, N)).astype(np.float32)
    k0 = rng.standard_normal((B, nh, N)).astype(np.float32)
    v0 = rng.standard_normal((B, nh, hd)).astype(np.float32)
    d = lambda a: to_dev(a, cuda_dev)
    rs, rks, rvs = d(s0), d(k0), d(v0)
    ref = rk.m3_burnin_fwd(dt, rs, rks, rvs, g["x"], g["K"], g["Q"], g["alpha"], g["beta"], g["gamma"], g["Dh"])
    ls, lks, lvs = d(s0), d(k0), d(v0)
    y_lib = mb.m3_ssd_fwd(g["x"], g["K"], g["Q"], g["dt"], g["trap"], g["adt"], g["Dh"], ssm_state=ls,
                          k_state=lks, v_state=lvs, carry_in=True)
    torch.cuda.synchronize()
    orc = oracle.m3_ssd_fwd(*[i[k] for k in M3_ARGS], ssm=s0, kst=k0, vst=v0)
    tol = TOL[dt]
    assert rel_err(host(ref["y"]), orc["y"]) <= tol
    assert rel_err(host(y_lib), host(ref["y"])) <= tol
    for r, l, o in ((rs, ls, "ssm_state"), (rks, lks, "k_state"), (rvs, lvs, "v_state")):
        assert rel_err(host(r), orc[o]) <= 1e-4, o
        assert rel_err(host(l), host(r)) <= 1e-4, o


@pytest.mark.parametrize("shape", M3_SEQ_SHAPES, ids=lambda s: "B%dT%dnh%dhd%dN%d" % s)
def test_reference_m3_sequential_backward(cuda_dev, rk, shape):
    """m3_backward_seq (f32 only in the reference) ~ oracle BPTT on every gradient it emits;
    the library's dx / dK / dQ / dD match it as well."""
    import torch

    import mamba_rs_b200 as mb
    B, T, nh, hd, N = shape
    i = m3_case(shape, "f32", seed=T + 11)
    g = m3_dev(i, "f32", cuda_dev)
    z = lambda *s: torch.zeros(*s, device=cuda_dev)
    saves = rk.m3_burnin_fwd("f32", z(B, nh, hd, N), z(B, nh, N), z(B, nh, hd), g["x"], g["K"], g["Q"],
                             g["alpha"], g["beta"], g["gamma"], g["Dh"])
    ref = rk.m3_backward_seq(saves, g["x"], g["K"], g["Q"], g["alpha"], g["beta"], g["gamma"], g["Dh"], g["dy"])
    lib = mb.m3_ssd_bwd(g["x"], g["K"], g["Q"], g["dt"], g["trap"], g["adt"], g["Dh"], g["dy"])
    torch.cuda.synchronize()
    orc = oracle.m3_ssd_bwd(*[i[k] for k in M3_ARGS], i["dy"])
    for k in ("dx", "dK", "dQ", "d_alpha", "d_beta", "d_gamma", "dD"):
        assert rel_err(host(ref[k]), orc[k]) <= 1e-4, ("reference vs oracle", k)
    for k in ("dx", "dK", "dQ", "dD"):
        assert rel_err(host(lib[k]), host(ref[k])) <= 1e-4, ("library vs reference", k)


# (shape, chunk): the reference's unit test runs chunk 4 over T = 10 (ragged last chunk)
M3_CHUNK_CASES = [((2, 10, 2, 4, 4), 4), ((2, 200, 2, 32, 64), 64), ((1, 256, 4, 16, 32), 64),
                  ((1, 130, 2, 8, 16), 64)]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("case", M3_CHUNK_CASES, ids=lambda c: "B%dT%dnh%dhd%dN%d" % c[0] + "cs%d" % c[1])
def test_reference_m3_chunked_forward_and_backward(cuda_dev, rk, case, dt):
    """The reference's chunked chain (preprocess -> dA cumsum -> chunk state -> state passing
    -> chunk scan; extract -> dqkv -> dqktheta with no RoPE angles -> ddt_dtrap) ~ oracle ~
    library, forward and backward.  16-bit storage with headdim and d_state multiples of 8
    takes the library's tcgen05 path."""
    import torch

    import mamba_rs_b200 as mb
    shape, CS = case
    B, T, nh, hd, N = shape
    i = m3_case(shape, dt, seed=T + CS)
    g = m3_dev(i, dt, cuda_dev)
    fw = rk.m3_chunked_fwd(dt, g["x"], g["K"], g["Q"], g["dt"], g["trap"], g["adt"], g["Dh"], CS)
    gq = rk.m3_dqkv(dt, fw, g["x"], g["Q"], g["Dh"], g["dy"], CS)
    tail = rk.m3_dqk_tail(dt, fw, gq, g["K"], g["Q"], g["dt"], g["trap"], CS)
    ls = torch.zeros(B, nh, hd, N, device=cuda_dev)
    y_lib = mb.m3_ssd_fwd(g["x"], g["K"], g["Q"], g["dt"], g["trap"], g["adt"], g["Dh"], ssm_state=ls)
    lib = mb.m3_ssd_bwd(g["x"], g["K"], g["Q"], g["dt"], g["trap"], g["adt"], g["Dh"], g["dy"])
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    of = oracle.m3_ssd_fwd(*[i[k] for k in M3_ARGS])
    ob = oracle.m3_ssd_bwd(*[i[k] for k in M3_ARGS], i["dy"])
    tol = TOL[dt]
    # forward
    assert rel_err(host(fw["y"]), of["y"]) <= tol
    assert rel_err(host(y_lib), host(fw["y"])) <= tol
    assert rel_err(host(fw["final_state"]), of["ssm_state"]) <= tol
    assert rel_err(host(ls), host(fw["final_state"])) <= tol
    # backward: reference chain vs oracle, library vs reference chain
    sig = i["trap"] * (1.0 - i["trap"])  # the reference emits d(trap) before its sigmoid
    ref_b = dict(dx=host(gq["dV"]), dK=host(tail["dK"]), dQ=host(tail["dQ"]), d_adt=host(gq["dADT"]),
                 d_dt=host(tail["d_dt"]), d_trap_raw=host(tail["d_trap_raw"]), dD=host(gq["dD"]))
    orc_b = dict(ob, d_trap_raw=ob["d_trap"] * sig)
    lib_b = {k: host(v) for k, v in lib.items()}
    lib_b["d_trap_raw"] = lib_b["d_trap"] * sig
    for k in ("dx", "dK", "dQ", "d_adt", "d_dt", "d_trap_raw", "dD"):
        assert rel_err(ref_b[k], orc_b[k]) <= tol, ("reference vs oracle", k)
        assert rel_err(lib_b[k], ref_b[k]) <= tol, ("library vs reference", k)


# --- Mamba-3 per-head K / Q: reference chain bc_bias_add -> m3_angle_dt_fwd_seq -> rope_fwd ---
@pytest.mark.parametrize("shape", [(2, 300, 4, 1, 128, 32), (1, 129, 4, 2, 64, 32), (2, 70, 2, 1, 32, 8)])
def test_reference_m3_kq_chain_agrees_with_oracle_and_fused_kernel(cuda_dev, rk, shape):
    """reference kernels ~ oracle.m3_kq_from_groups (f32, 1e-4), and the tensor-core kernel
    that builds K / Q itself ~ the scan oracle fed the reference kernels' K / Q (bf16, 2e-2)."""
    import torch

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import synth
    B, T, nh, ng, N, na = shape
    hd = 32
    i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=21)
    g = synth.m3_group_inputs(B, T, nh, ng, N, na, i["dt"], seed=21)
    raw = np.random.default_rng(5).standard_normal((B, T, na)).astype(np.float32)
    vel = (np.tanh(raw) * np.float32(np.pi)).astype(np.float32)
    bf = lambda a: synth.round_to(a, "bf16")
    Bn, Cn, x = bf(g["Bn"]), bf(g["Cn"]), bf(i["x"])
    t = lambda a, d=None: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_dev).to(d or torch.float32)
    ang_ref = t(g["angle_state"])
    Kr, Qr, cum = rk.m3_kq_from_groups(t(Bn), t(Cn), t(g["b_bias"]), t(g["c_bias"]), t(raw), t(i["dt"]), ang_ref)
    torch.cuda.synchronize()
    Ko, Qo, ang_o = oracle.m3_kq_from_groups(Bn, Cn, g["b_bias"], g["c_bias"], vel, i["dt"], g["angle_state"])
    assert rel_err(Kr.cpu().numpy(), Ko) <= 1e-4
    assert rel_err(Qr.cpu().numpy(), Qo) <= 1e-4
    d = np.abs(ang_ref.cpu().numpy() - ang_o)
    assert np.minimum(d, 2 * np.pi - d).max() <= 1e-4

    ref = oracle.m3_ssd_fwd(x, bf(Kr.cpu().numpy()), bf(Qr.cpu().numpy()), i["dt"], i["trap"], i["adt"], i["Dh"])
    tb = torch.bfloat16
    ang = t(g["angle_state"])
    y = mb.ops.m3_ssd_fwd_fused_kq(t(x, tb), t(Bn, tb), t(Cn, tb), t(g["b_bias"]), t(g["c_bias"]), t(vel),
                                   t(i["dt"]), t(i["trap"]), t(i["adt"]), t(i["Dh"]), angle_state=ang)
    torch.cuda.synchronize()
    assert rel_err(y.float().cpu().numpy(), ref["y"]) <= TOL["bf16"]
    d = np.abs(ang.cpu().numpy() - ang_ref.cpu().numpy())
    assert np.minimum(d, 2 * np.pi - d).max() <= 1e-3
