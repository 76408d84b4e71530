"""CPU tests of the Mamba-3 SISO SSD oracle: the sequential definition against
its f64 shadow, the chunked reformulation against the sequential definition
(tests/m3_cpu_gpu_train_parity.rs:550-571 pins chunked vs sequential at T=256),
split == whole, and the analytic backward against f64 central differences
(tests/m3_test_correctness.rs:147-201)."""
import numpy as np
import pytest

import oracle
from helpers import rel_err
from mamba_rs_b200 import synth

ARGS = ("x", "K", "Q", "dt", "trap", "adt", "Dh")


def test_sequential_matches_f64_shadow():
    i = synth.m3_ssd_inputs(2, 80, 3, 8, 16, seed=1)
    r = oracle.m3_ssd_fwd(*[i[k] for k in ARGS])
    y64 = oracle.m3_ssd_fwd_f64(*[i[k] for k in ARGS])
    assert rel_err(r["y"], y64) < 2e-6


@pytest.mark.parametrize("shape", [(2, 256, 2, 8, 16, 64), (1, 10, 2, 4, 4, 4), (1, 100, 2, 16, 32, 64),
                                   (1, 130, 1, 64, 128, 64)], ids=str)
def test_chunked_reformulation_equals_sequential(shape):
    B, T, nh, hd, N, CS = shape
    i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=T)
    seq = oracle.m3_ssd_fwd(*[i[k] for k in ARGS])
    chk = oracle.m3_ssd_fwd_chunked(*[i[k] for k in ARGS], chunk=CS)
    assert rel_err(chk["y"], seq["y"]) < 1e-5
    assert rel_err(chk["ssm_state"], seq["ssm_state"]) < 1e-5


def test_split_sequence_equals_whole_bitwise():
    i = synth.m3_ssd_inputs(1, 60, 2, 8, 16, seed=2)
    whole = oracle.m3_ssd_fwd(*[i[k] for k in ARGS])
    cut = 23
    a = oracle.m3_ssd_fwd(*[i[k][:, :cut] if k != "Dh" else i[k] for k in ARGS])
    b = oracle.m3_ssd_fwd(*[i[k][:, cut:] if k != "Dh" else i[k] for k in ARGS], ssm=a["ssm_state"],
                          kst=a["k_state"], vst=a["v_state"])
    np.testing.assert_array_equal(np.concatenate([a["y"], b["y"]], axis=1), whole["y"])
    np.testing.assert_array_equal(b["ssm_state"], whole["ssm_state"])
    np.testing.assert_array_equal(b["k_state"], i["K"][:, -1])
    np.testing.assert_array_equal(b["v_state"].reshape(1, -1), i["x"][:, -1])


def test_backward_matches_f64_finite_differences():
    rng = np.random.default_rng(0)
    B, T, nh, hd, N = 1, 20, 2, 4, 8
    i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=3)
    dy = rng.standard_normal((B, T, nh * hd)).astype(np.float32)
    g = oracle.m3_ssd_bwd(*[i[k] for k in ARGS], dy)
    base = {k: i[k].astype(np.float64) for k in ARGS}

    def loss(**kw):
        a = dict(base)
        a.update(kw)
        return float((oracle.m3_ssd_fwd_f64(*[a[k] for k in ARGS]) * dy).sum())

    eps = 1e-5
    for name, gname in (("x", "dx"), ("K", "dK"), ("Q", "dQ"), ("dt", "d_dt"), ("trap", "d_trap"),
                        ("adt", "d_adt"), ("Dh", "dD")):
        for _ in range(5):
            idx = tuple(int(rng.integers(0, s)) for s in base[name].shape)
            ap, am = base[name].copy(), base[name].copy()
            ap[idx] += eps
            am[idx] -= eps
            fd = (loss(**{name: ap}) - loss(**{name: am})) / (2 * eps)
            an = float(g[gname][idx])
            assert abs(fd - an) <= 5e-3 * max(abs(fd), abs(an)) + 5e-5, (name, idx, fd, an)
