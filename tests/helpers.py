"""Shared helpers of the parity tests: seeded inputs rounded to the storage
dtype, device transfer, and the error measure the tolerances are stated in."""
import numpy as np

from mamba_rs_b200 import synth

# Tolerances of the parity bar: max-abs error relative to the max-abs reference
# value, 1e-4 for f32 storage and 2e-2 for bf16 / f16 storage.
TOL = {"f32": 1e-4, "bf16": 2e-2, "f16": 2e-2}
ACT_KEYS = ("x", "z", "delta_raw", "Bm", "Cm")


def rel_err(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = max(np.abs(ref).max(), 1e-30)
    return float(np.abs(got - ref).max() / den)


def quantised_inputs(B, T, D, N, K, dtype, seed=0, a_mode="s4d", z=True):
    inp = synth.m1_scan_inputs(B, T, D, N, K, seed, a_mode, z)
    return {k: (synth.round_to(v, dtype) if k in ACT_KEYS else v) for k, v in inp.items()}


def random_states(B, D, N, K, seed):
    rng = np.random.default_rng(seed)
    ssm = rng.standard_normal((B, D, N)).astype(np.float32)
    cst = rng.standard_normal((B, D, K)).astype(np.float32) if K else None
    return ssm, cst


def torch_dtype(name):
    import torch
    return {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[name]


def to_dev(a, dev, dtype=None):
    import torch
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t.to(dtype) if dtype is not None else t


# Committed golden fixtures (tests/golden/m1_fused_<name>.npz, made by
# tests/golden/gen_golden.py): name, B, T, D, N, K, dtype, a_mode, seed
GOLDEN_CASES = [
    ("f32_s4d_conv", 2, 37, 24, 16, 4, "f32", "s4d", 11),
    ("bf16_rand_conv", 1, 50, 40, 16, 4, "bf16", "random", 12),
    ("f16_s4d_noconv", 2, 20, 16, 8, 0, "f16", "s4d", 13),
    ("f32_rand_n4", 1, 33, 10, 4, 3, "f32", "random", 14),
]


def golden_inputs(case):
    """Inputs, entering states and upstream gradient of one golden case."""
    name, B, T, D, N, K, dt, a_mode, seed = case
    q = quantised_inputs(B, T, D, N, K, dt, seed, a_mode)
    ssm0, cst0 = random_states(B, D, N, K, seed + 100)
    dg = np.random.default_rng(seed + 200).standard_normal((B, T, D)).astype(np.float32)
    return q, ssm0, cst0, dg


def load_golden(name):
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"m1_fused_{name}.npz")
    return dict(np.load(path))
