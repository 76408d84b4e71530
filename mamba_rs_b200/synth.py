"""Seeded synthetic workloads for the selective-scan path.

The reference measures on no public dataset; these generators reproduce the
shapes and value distributions of the configurations the benchmarks and parity
tests are quoted on (numpy Generator, PCG64, seed stated per call).
"""
from __future__ import annotations

import numpy as np


def inv_softplus(y):
    y = np.asarray(y, dtype=np.float64)
    return np.where(y > 20.0, y, np.log(np.expm1(y)))


def m1_scan_inputs(B, T, D, N, K=0, seed=0, a_mode="s4d", z=True, dt_min=1e-3, dt_max=1e-1):
    """Inputs of the standalone fused op (float32 numpy arrays).

    u|x, z ~ N(0,1); delta_raw = 0.5*N(0,1) + dt_bias[d] with
    dt_bias = inv_softplus(log-uniform[dt_min, dt_max]); B, C ~ N(0,1);
    a_neg[d,n] = -(n+1) ("s4d", the reference init) or a random negative
    matrix ("random": -exp(U[ln 0.5, ln 16]), as after training); D = 1.
    With K > 0, x is the pre-conv branch and conv_w ~ U(-sqrt(3/K), sqrt(3/K)),
    conv_b ~ 0.1*N(0,1)."""
    rng = np.random.default_rng(seed)
    f = np.float32
    x = rng.standard_normal((B, T, D), dtype=f)
    zz = rng.standard_normal((B, T, D), dtype=f) if z else None
    dt = np.exp(rng.uniform(np.log(dt_min), np.log(dt_max), size=D))
    dt_bias = inv_softplus(dt).astype(f)
    delta_raw = (0.5 * rng.standard_normal((B, T, D), dtype=f) + dt_bias[None, None, :]).astype(f)
    Bm = rng.standard_normal((B, T, N), dtype=f)
    Cm = rng.standard_normal((B, T, N), dtype=f)
    if a_mode == "s4d":
        a_neg = -np.tile(np.arange(1, N + 1, dtype=f), (D, 1))
    elif a_mode == "random":
        a_neg = -np.exp(rng.uniform(np.log(0.5), np.log(16.0), size=(D, N))).astype(f)
    else:
        raise ValueError(a_mode)
    out = dict(x=x, z=zz, delta_raw=delta_raw, Bm=Bm, Cm=Cm, a_neg=np.ascontiguousarray(a_neg),
               Dp=np.ones(D, f))
    if K:
        bound = np.sqrt(3.0 / K)
        out["conv_w"] = rng.uniform(-bound, bound, size=(D, K)).astype(f)
        out["conv_b"] = (0.1 * rng.standard_normal(D)).astype(f)
    return out


def round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round a float32 array to the storage dtype and back (float32 values that
    the device sees exactly)."""
    if a is None or dtype == "f32":
        return a
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a))
    td = {"bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    return t.to(td).to(torch.float32).numpy()


def m1_fwd_algorithmic_bytes(B, T, D, N, esize, K=0, z=True):
    """Bytes the fused forward must move once: x|u, delta, [z], y activations,
    B and C, a_neg and D, state in and out, [conv state in/out, conv w, b]."""
    streams = 3 + (1 if z else 0)
    total = streams * esize * B * T * D + 2 * esize * B * T * N + 4 * D * (N + 1) + 2 * 4 * B * D * N
    if K:
        total += 2 * 4 * B * D * K + 4 * D * (K + 1)
    return total


def m3_ssd_inputs(B, T, nh, hd, N, seed=0):
    """Inputs of the Mamba-3 SISO SSD op (float32): x, K, Q ~ N(0,1) (K and Q
    scaled by N^-1/4 each so q.k stays O(1)); per-head A = -exp(U[ln 1, ln 16]);
    dt = softplus(0.5*N(0,1) + dt_bias), dt_bias as for Mamba-1; trap =
    sigmoid(N(0,1)); adt = A*dt; D = 1."""
    rng = np.random.default_rng(seed)
    f = np.float32
    x = rng.standard_normal((B, T, nh * hd), dtype=f)
    sc = f(N) ** f(-0.25)
    K = rng.standard_normal((B, T, nh, N), dtype=f) * sc
    Q = rng.standard_normal((B, T, nh, N), dtype=f) * sc
    A = -np.exp(rng.uniform(np.log(1.0), np.log(16.0), size=nh)).astype(f)
    dt_bias = inv_softplus(np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=nh))).astype(f)
    raw = 0.5 * rng.standard_normal((B, T, nh), dtype=f) + dt_bias
    dt = np.log1p(np.exp(raw.astype(np.float64))).astype(f)
    trap = (1.0 / (1.0 + np.exp(-rng.standard_normal((B, T, nh))))).astype(f)
    adt = (A[None, None, :] * dt).astype(f)
    return dict(x=x, K=K, Q=Q, dt=dt, trap=trap, adt=adt, Dh=np.ones(nh, f), A=A)


def m3_group_inputs(B, T, nh, ng, N, n_angles, dt, seed=0):
    """Group-level inputs of the Mamba-3 K / Q generation: Bn, Cn [B,T,ng,N] ~ N(0,1)
    * N^-1/4 (what BCNorm leaves, scaled like K and Q above), per-head biases ~ 0.1 N(0,1),
    angle_vel = tanh(N(0,1)) * pi [B,T,n_angles], a starting angle in [0, 2 pi)."""
    rng = np.random.default_rng(seed + 7919)
    f = np.float32
    sc = f(N) ** f(-0.25)
    Bn = rng.standard_normal((B, T, ng, N), dtype=f) * sc
    Cn = rng.standard_normal((B, T, ng, N), dtype=f) * sc
    b_bias = (0.1 * rng.standard_normal((nh, N), dtype=f) * sc).astype(f)
    c_bias = (0.1 * rng.standard_normal((nh, N), dtype=f) * sc).astype(f)
    vel = (np.tanh(rng.standard_normal((B, T, max(n_angles, 1)), dtype=f)) * f(np.pi)).astype(f)[:, :, :n_angles]
    ang0 = rng.uniform(0.0, 2 * np.pi, size=(B, nh, max(n_angles, 1))).astype(f)[:, :, :n_angles]
    return dict(Bn=Bn, Cn=Cn, b_bias=b_bias, c_bias=c_bias, angle_vel=np.ascontiguousarray(vel),
                angle_state=np.ascontiguousarray(ang0))


def m3_fused_kq_algorithmic_bytes(B, T, nh, ng, hd, N, n_angles, esize):
    """x and y, the group-level Bn and Cn once each, angle_vel, dt/trap/adt f32, biases,
    final state out."""
    return (2 * esize * B * T * nh * hd + 2 * esize * B * T * ng * N + 4 * B * T * n_angles
            + 3 * 4 * B * T * nh + 2 * 4 * nh * N + 4 * B * nh * hd * N)


def m3_fwd_algorithmic_bytes(B, T, nh, hd, N, esize):
    """x and y, K and Q once each, dt/trap/adt f32, final state out."""
    return (2 * esize * B * T * nh * hd + 2 * esize * B * T * nh * N + 3 * 4 * B * T * nh
            + 4 * B * nh * hd * N)
