"""GPU parity tests of the fused Mamba-1 forward, through the C ABI, against
the CPU oracle on identical (storage-rounded) inputs.

Bar: max-abs error / max-abs reference <= 1e-4 for f32 storage, <= 2e-2 for
bf16 / f16 storage, for y and the final SSM state; the conv window is a copy
of inputs and must match exactly."""
import numpy as np
import pytest

import oracle
from helpers import (GOLDEN_CASES, TOL, golden_inputs, load_golden, quantised_inputs, random_states,
                     rel_err, to_dev, torch_dtype)

pytestmark = pytest.mark.gpu


def run_gpu(q, dt, dev, ssm0=None, cst0=None, **kw):
    import torch

    import mamba_rs_b200 as mb
    td = torch_dtype(dt)
    ssm = to_dev(ssm0, dev)
    cst = to_dev(cst0, dev)
    y = mb.selective_scan_fwd(to_dev(q["x"], dev, td), to_dev(q["delta_raw"], dev, td),
                              to_dev(q["Bm"], dev, td), to_dev(q["Cm"], dev, td), to_dev(q["a_neg"], dev),
                              to_dev(q["Dp"], dev), to_dev(q.get("z"), dev, td),
                              conv_w=to_dev(q.get("conv_w"), dev), conv_b=to_dev(q.get("conv_b"), dev),
                              conv_state=cst, ssm_state=ssm, **kw)
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    return (y.float().cpu().numpy(), None if ssm is None else ssm.cpu().numpy(),
            None if cst is None else cst.cpu().numpy())


def run_ref(q, ssm0=None, cst0=None, **kw):
    return oracle.m1_fused_fwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q.get("z"), q["a_neg"], q["Dp"],
                               q.get("conv_w"), q.get("conv_b"), cst0, ssm0, **kw)


SHAPES = [
    # B, T, D, N, K — T around the 16-step chunk and 4-step block edges, ragged D, every N variant
    (2, 40, 64, 16, 0), (2, 100, 48, 16, 4), (1, 1, 32, 16, 4), (1, 3, 5, 16, 4), (1, 15, 33, 16, 4),
    (1, 16, 64, 16, 0), (1, 17, 130, 16, 4), (3, 65, 7, 4, 3), (1, 33, 20, 8, 4), (1, 50, 12, 12, 2),
    (1, 50, 12, 64, 4), (1, 20, 6, 32, 4), (1, 9, 3, 128, 2), (2, 300, 256, 16, 4), (1, 257, 64, 16, 4),
    (1, 40, 2, 256, 0), (1, 70, 3, 200, 4),
]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("a_mode", ["s4d", "random"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "B%dT%dD%dN%dK%d" % s)
def test_fused_forward_matches_oracle(cuda_dev, shape, a_mode, dt):
    B, T, D, N, K = shape
    q = quantised_inputs(B, T, D, N, K, dt, seed=B * 1000 + T, a_mode=a_mode)
    ssm0, cst0 = random_states(B, D, N, K, seed=T)
    ref = run_ref(q, ssm0, cst0)
    y, ssm, cst = run_gpu(q, dt, cuda_dev, ssm0, cst0)
    assert rel_err(y, ref["y"]) <= TOL[dt]
    assert rel_err(ssm, ref["ssm_state"]) <= 1e-4  # state is f32 for every storage dtype
    if K:
        np.testing.assert_array_equal(cst, ref["conv_state"])


@pytest.mark.parametrize("case", GOLDEN_CASES, ids=[c[0] for c in GOLDEN_CASES])
def test_fused_forward_matches_golden(cuda_dev, case):
    q, ssm0, cst0, _ = golden_inputs(case)
    gold = load_golden(case[0])
    dt = case[6]
    y, ssm, cst = run_gpu(q, dt, cuda_dev, ssm0, cst0)
    assert rel_err(y, gold["y"]) <= TOL[dt]
    assert rel_err(ssm, gold["ssm_state"]) <= 1e-4
    if case[5]:
        np.testing.assert_array_equal(cst, gold["conv_state"])


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_modes_no_gate_pre_softplus_and_ready_gate(cuda_dev, dt):
    import torch
    q = quantised_inputs(2, 70, 40, 16, 0, dt, seed=21, a_mode="random")
    # no gate, delta already activated (the unfused reference kernel's contract)
    q2 = dict(q)
    q2["delta_raw"] = np.log1p(np.exp(q["delta_raw"].astype(np.float64))).astype(np.float32)
    from mamba_rs_b200 import synth
    q2["delta_raw"] = synth.round_to(q2["delta_raw"], dt)
    q2["z"] = None
    ref = run_ref(q2, delta_softplus=False)
    y, _, _ = run_gpu(q2, dt, cuda_dev, delta_softplus=False)
    assert rel_err(y, ref["y"]) <= TOL[dt]
    # z_mode 2: the gate tensor already holds SiLU(gate)
    q3 = dict(q)
    g = q["z"].astype(np.float64)
    q3["z"] = synth.round_to((g / (1 + np.exp(-g))).astype(np.float32), dt)
    ref3 = run_ref(dict(q3, z=None))
    y3, _, _ = run_gpu(q3, dt, cuda_dev, z_mode=2)
    assert rel_err(y3, ref3["y"] * q3["z"]) <= TOL[dt]


def test_compat_entry_point_matches_reference_kernel_contract(cuda_dev):
    """mamba_b200_ssm_scan_fwd_nosave == ssm_parallel_scan_fwd_nosave_{dt}:
    shapes of tests/m1_parallel_bwd_parity.rs:290-366, det_rand inputs."""
    import torch

    import mamba_rs_b200 as mb
    for (B, T, D, N) in [(1, 32, 4, 4), (1, 2048, 4, 8), (1, 1500, 4, 8), (2, 256, 8, 16), (1, 3072, 4, 8)]:
        u = oracle.det_rand(B * T * D, 1).reshape(B, T, D)
        delta = (np.abs(oracle.det_rand(B * T * D, 2)) * 0.2 + 0.01).reshape(B, T, D).astype(np.float32)
        Bm = oracle.det_rand(B * T * N, 3).reshape(B, T, N)
        Cm = oracle.det_rand(B * T * N, 4).reshape(B, T, N)
        a_neg = -np.exp(oracle.det_rand(D * N, 5).reshape(D, N) + 0.5).astype(np.float32)
        Dp = (oracle.det_rand(D, 6) + 1.0).astype(np.float32)
        h0 = oracle.det_rand(B * D * N, 7).reshape(B, D, N)
        ref = oracle.m1_fused_fwd(u, delta, Bm, Cm, None, a_neg, Dp, ssm_state=h0, delta_softplus=False)
        h = to_dev(h0, cuda_dev)
        y = torch.empty(B, T, D, device=cuda_dev)
        mb.ssm_parallel_scan_fwd_nosave(h, y, to_dev(delta, cuda_dev), to_dev(u, cuda_dev),
                                        to_dev(Bm, cuda_dev), to_dev(Cm, cuda_dev), to_dev(a_neg, cuda_dev),
                                        to_dev(Dp, cuda_dev))
        torch.cuda.synchronize()
        assert rel_err(y.cpu().numpy(), ref["y"]) <= 1e-4
        assert rel_err(h.cpu().numpy(), ref["ssm_state"]) <= 1e-4


def test_in_place_strided_views_of_proj_and_xdbl(cuda_dev):
    """x and z read in place from proj[B*T, 2D], B and C from xdbl[B*T, dt_rank+2N]
    (the reference gathers them into scratch buffers first)."""
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N, K, dr = 2, 77, 48, 16, 4, 8
    q = quantised_inputs(B, T, D, N, K, "bf16", seed=31)
    td = torch.bfloat16
    proj = torch.cat([to_dev(q["x"], cuda_dev, td), to_dev(q["z"], cuda_dev, td)], dim=-1)
    xdbl = torch.cat([torch.zeros(B, T, dr, device=cuda_dev, dtype=td), to_dev(q["Bm"], cuda_dev, td),
                      to_dev(q["Cm"], cuda_dev, td)], dim=-1)
    ref = run_ref(q)
    u_out = torch.empty(B, T, D, device=cuda_dev, dtype=td)
    y = mb.selective_scan_fwd(proj[..., :D], to_dev(q["delta_raw"], cuda_dev, td), xdbl[..., dr:dr + N],
                              xdbl[..., dr + N:], to_dev(q["a_neg"], cuda_dev), to_dev(q["Dp"], cuda_dev),
                              proj[..., D:], conv_w=to_dev(q["conv_w"], cuda_dev),
                              conv_b=to_dev(q["conv_b"], cuda_dev), u_out=u_out)
    torch.cuda.synchronize()
    assert rel_err(y.float().cpu().numpy(), ref["y"]) <= TOL["bf16"]
    refu = run_ref(q, want_u=True)["u"]
    assert rel_err(u_out.float().cpu().numpy(), refu) <= TOL["bf16"]


def test_misaligned_rows_use_plain_load_path(cuda_dev):
    """Odd row strides and an odd base offset break every TMA layout rule; the
    kernel must fall back to plain loads and stores and still match."""
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N = 1, 45, 19, 16
    q = quantised_inputs(B, T, D, N, 0, "f16", seed=41)
    td = torch.float16

    def odd(a, cols):
        buf = torch.zeros(B, T, cols + 3, device=cuda_dev, dtype=td)
        buf[..., 1:1 + cols] = to_dev(a, cuda_dev, td)
        return buf[..., 1:1 + cols]

    ybuf = torch.zeros(B, T, D + 3, device=cuda_dev, dtype=td)
    y = mb.selective_scan_fwd(odd(q["x"], D), odd(q["delta_raw"], D), odd(q["Bm"], N), odd(q["Cm"], N),
                              to_dev(q["a_neg"], cuda_dev), to_dev(q["Dp"], cuda_dev), odd(q["z"], D),
                              y=ybuf[..., 1:1 + D])
    torch.cuda.synchronize()
    ref = run_ref(q)
    assert rel_err(y.float().cpu().numpy(), ref["y"]) <= TOL["f16"]
    assert float(ybuf[..., 0].abs().max()) == 0.0 and float(ybuf[..., 1 + D:].abs().max()) == 0.0


def test_split_sequence_equals_whole_on_gpu(cuda_dev):
    """Prefill in two calls with state carried == one call (tests/prefill.rs:174-232)."""
    q = quantised_inputs(2, 90, 32, 16, 4, "f32", seed=51)
    whole_y, whole_h, whole_c = run_gpu(q, "f32", cuda_dev, np.zeros((2, 32, 16), np.float32),
                                        np.zeros((2, 32, 4), np.float32))
    cut = 37
    first = {k: (v[:, :cut] if k in ("x", "z", "delta_raw", "Bm", "Cm") else v) for k, v in q.items()}
    second = {k: (v[:, cut:] if k in ("x", "z", "delta_raw", "Bm", "Cm") else v) for k, v in q.items()}
    y1, h1, c1 = run_gpu(first, "f32", cuda_dev, np.zeros((2, 32, 16), np.float32),
                         np.zeros((2, 32, 4), np.float32))
    y2, h2, c2 = run_gpu(second, "f32", cuda_dev, h1, c1)
    assert rel_err(np.concatenate([y1, y2], axis=1), whole_y) <= 1e-6
    assert rel_err(h2, whole_h) <= 1e-6
    np.testing.assert_array_equal(c2, whole_c)


def test_chunk_states_are_the_states_entering_each_block(cuda_dev):
    import torch
    B, T, D, N, S = 2, 200, 24, 16, 64
    q = quantised_inputs(B, T, D, N, 0, "f32", seed=61)
    ssm0, _ = random_states(B, D, N, 0, 62)
    ref = run_ref(q, ssm0, want_h=True)
    nblk = (T + S - 1) // S
    cs = torch.full((B, nblk, D, N), float("nan"), device=cuda_dev)
    run_gpu(q, "f32", cuda_dev, ssm0, chunk_states=cs, save_stride=S)
    got = cs.cpu().numpy()
    for k in range(nblk):
        assert rel_err(got[:, k], ref["h_all"][:, k * S]) <= 1e-4


def test_argument_errors_are_reported_not_launched(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    x = torch.zeros(1, 8, 16, device=cuda_dev)
    bc = torch.zeros(1, 8, 16, device=cuda_dev)
    a = torch.zeros(16, 16, device=cuda_dev)
    Dp = torch.zeros(16, device=cuda_dev)
    with pytest.raises(RuntimeError, match="d_state"):
        mb.selective_scan_fwd(x, x, torch.zeros(1, 8, 300, device=cuda_dev),
                              torch.zeros(1, 8, 300, device=cuda_dev), torch.zeros(16, 300, device=cuda_dev), Dp)
    with pytest.raises(RuntimeError, match="d_conv"):
        mb.selective_scan_fwd(x, x, bc, bc, a, Dp, conv_w=torch.zeros(16, 9, device=cuda_dev),
                              conv_b=torch.zeros(16, device=cuda_dev))
    for bad in (10, 16, 128):
        with pytest.raises(RuntimeError, match="save_stride"):
            mb.selective_scan_fwd(x, x, bc, bc, a, Dp, chunk_states=torch.zeros(1, 1, 16, 16, device=cuda_dev),
                                  save_stride=bad)
    # empty batch / empty sequence: accepted, nothing to do
    e = torch.zeros(0, 8, 16, device=cuda_dev)
    assert mb.selective_scan_fwd(e, e, e, e, a, Dp).shape == (0, 8, 16)


def test_full_size_linearity_and_split_at_config2(cuda_dev):
    """The benchmark shape (B=16, D=1536, N=16, L=2048, bf16) is too large for the
    CPU oracle in a unit test; check size-independent properties instead:
    (1) with z fixed the op is linear in u: f(2u) == 2 f(u) up to bf16 rounding,
    (2) two half-length calls with the state carried == one call,
    (3) a CPU-oracle spot check of 3 channels x 1 sample drawn from the tensor."""
    import torch

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import synth
    B, T, D, N = 16, 2048, 1536, 16
    inp = synth.m1_scan_inputs(B, T, D, N, 0, seed=2, a_mode="s4d")
    td = torch.bfloat16
    x, dl, Bm, Cm, z = [to_dev(inp[k], cuda_dev, td) for k in ("x", "delta_raw", "Bm", "Cm", "z")]
    a, Dp = to_dev(inp["a_neg"], cuda_dev), to_dev(inp["Dp"], cuda_dev)
    h = torch.zeros(B, D, N, device=cuda_dev)
    y1 = mb.selective_scan_fwd(x, dl, Bm, Cm, a, Dp, z, ssm_state=h)
    h2 = torch.zeros(B, D, N, device=cuda_dev)
    y2 = mb.selective_scan_fwd(x * 2, dl, Bm, Cm, a, Dp, z, ssm_state=h2)
    torch.cuda.synchronize()
    scale = float(y1.float().abs().max())
    assert float((y2.float() - 2 * y1.float()).abs().max()) <= 2e-2 * 2 * scale
    assert float((h2 - 2 * h).abs().max()) <= 1e-4 * float(h2.abs().max())
    ha = torch.zeros(B, D, N, device=cuda_dev)
    c = lambda t_, lo, hi: t_[:, lo:hi].contiguous()  # the ABI takes [B*T, ld] row-major blocks
    ya = mb.selective_scan_fwd(c(x, 0, 1000), c(dl, 0, 1000), c(Bm, 0, 1000), c(Cm, 0, 1000), a, Dp,
                               c(z, 0, 1000), ssm_state=ha)
    yb = mb.selective_scan_fwd(c(x, 1000, T), c(dl, 1000, T), c(Bm, 1000, T), c(Cm, 1000, T), a, Dp,
                               c(z, 1000, T), ssm_state=ha)
    torch.cuda.synchronize()
    assert float((torch.cat([ya, yb], 1).float() - y1.float()).abs().max()) <= 2e-2 * scale
    assert float((ha - h).abs().max()) <= 1e-4 * float(h.abs().max())
    # spot check against the oracle
    bsel, dsel = 5, [0, 777, 1535]
    f = lambda t_: t_[bsel:bsel + 1].float().cpu().numpy()
    ref = oracle.m1_fused_fwd(f(x)[..., dsel], f(dl)[..., dsel], f(Bm), f(Cm), f(z)[..., dsel],
                              inp["a_neg"][dsel], inp["Dp"][dsel])
    assert rel_err(f(y1)[..., dsel], ref["y"]) <= TOL["bf16"]
    assert rel_err(h[bsel, dsel].cpu().numpy(), ref["ssm_state"][0]) <= 1e-4


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", [(1, 2048, 40, 16, 4), (2, 1100, 24, 16, 0), (1, 4100, 8, 8, 3), (1, 1500, 16, 64, 4)],
                         ids=lambda s: "B%dT%dD%dN%dK%d" % s)
def test_time_segments_with_exact_carry_match_oracle(cuda_dev, shape, dt):
    """A small batch with a lent workspace is cut into time segments that run side by
    side (state-only pass, carry, full pass).  Fused conv, conv / ssm state updated in
    place, training saves: everything must match the one-piece oracle."""
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N, K = shape
    q = quantised_inputs(B, T, D, N, K, dt, seed=T + D, a_mode="random")
    ssm0, cst0 = random_states(B, D, N, K, seed=T)
    ref = oracle.m1_fused_fwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q["z"], q["a_neg"], q["Dp"],
                              q.get("conv_w"), q.get("conv_b"), cst0, ssm0, want_h=True)
    td = torch_dtype(dt)
    d = lambda a_, t_=None: to_dev(a_, cuda_dev, t_)
    ssm = d(ssm0)
    cst = d(cst0) if K else None
    S = 32
    cs = torch.empty(B, (T + S - 1) // S, D, N, device=cuda_dev)
    ws = torch.empty(mb.selective_scan_fwd_workspace_bytes(B, T, D, N), dtype=torch.uint8, device=cuda_dev)
    y = mb.selective_scan_fwd(d(q["x"], td), d(q["delta_raw"], td), d(q["Bm"], td), d(q["Cm"], td), d(q["a_neg"]),
                              d(q["Dp"]), d(q["z"], td), conv_w=d(q.get("conv_w")), conv_b=d(q.get("conv_b")),
                              conv_state=cst, ssm_state=ssm, chunk_states=cs, save_stride=S, workspace=ws)
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    assert rel_err(y.float().cpu().numpy(), ref["y"]) <= TOL[dt]
    assert rel_err(ssm.cpu().numpy(), ref["ssm_state"]) <= 1e-4
    if K:
        np.testing.assert_array_equal(cst.cpu().numpy(), ref["conv_state"])
    got = cs.cpu().numpy()
    for k in range(got.shape[1]):
        assert rel_err(got[:, k], ref["h_all"][:, k * S]) <= 1e-4, k
    # and the same call without a workspace (one segment) gives the same numbers
    ssm1 = d(ssm0)
    y1 = mb.selective_scan_fwd(d(q["x"], td), d(q["delta_raw"], td), d(q["Bm"], td), d(q["Cm"], td), d(q["a_neg"]),
                               d(q["Dp"]), d(q["z"], td), conv_w=d(q.get("conv_w")), conv_b=d(q.get("conv_b")),
                               conv_state=d(cst0) if K else None, ssm_state=ssm1)
    torch.cuda.synchronize()
    assert rel_err(y.float().cpu().numpy(), y1.float().cpu().numpy()) <= TOL[dt]
    assert rel_err(ssm.cpu().numpy(), ssm1.cpu().numpy()) <= 1e-4
