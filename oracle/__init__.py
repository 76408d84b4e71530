"""ctypes front-end of the CPU oracle (``liboracle.so``).

Test infrastructure only: imported by ``tests/``, by the smoke check and by the
CPU-baseline / reference legs of ``bench.py``; the product package never
imports it.  All arrays are C-contiguous numpy ``float32`` (``float64`` for the
shadow).  See ``m1_oracle.c`` / ``m3_oracle.c`` for the reference citations.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the committed Makefile (gcc only)."""
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith(".c")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_fast_exp_scalar.restype = C.c_float
        _lib.orc_fast_exp_scalar.argtypes = [C.c_float]
        _lib.orc_fast_exp_simd_lane.restype = C.c_float
        _lib.orc_fast_exp_simd_lane.argtypes = [C.c_float]
        _lib.orc_m1_layer_floats.restype = C.c_long
        _lib.orc_m1_weights_floats.restype = C.c_long
    return _lib


class M1Shape(C.Structure):
    _fields_ = [("B", C.c_int), ("T", C.c_int), ("D", C.c_int), ("N", C.c_int),
                ("K", C.c_int), ("ld_x", C.c_long), ("ld_delta", C.c_long),
                ("ld_z", C.c_long), ("ld_bc", C.c_long), ("ld_y", C.c_long),
                ("delta_softplus", C.c_int), ("has_z", C.c_int)]


class M1Config(C.Structure):
    _fields_ = [("d_model", C.c_int), ("n_layers", C.c_int), ("d_state", C.c_int),
                ("d_conv", C.c_int), ("expand", C.c_int), ("dt_rank", C.c_int),
                ("input_dim", C.c_int)]

    @property
    def d_inner(self):
        return self.expand * self.d_model

    @property
    def xdbl_dim(self):
        return self.dt_rank + 2 * self.d_state


def _p(a, dtype=np.float32):
    if a is None:
        return None
    assert a.dtype == dtype and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def fast_exp(x, simd: bool = False) -> np.ndarray:
    x = np.atleast_1d(np.asarray(x, dtype=np.float32))
    f = lib().orc_fast_exp_simd_lane if simd else lib().orc_fast_exp_scalar
    return np.array([f(float(v)) for v in x.ravel()], dtype=np.float32).reshape(x.shape)


def fast_exp_inplace(buf: np.ndarray) -> np.ndarray:
    buf = np.ascontiguousarray(buf, dtype=np.float32).copy()
    lib().orc_fast_exp_inplace(_p(buf), C.c_long(buf.size))
    return buf


def _shape(x, delta, Bm, z, N, K, delta_softplus):
    B, T, D = delta.shape
    return M1Shape(B, T, D, N, K, x.shape[-1], delta.shape[-1],
                   z.shape[-1] if z is not None else 0, Bm.shape[-1], D,
                   int(delta_softplus), int(z is not None))


def m1_fused_fwd(x, delta, Bm, Cm, z, a_neg, Dp, conv_w=None, conv_b=None,
                 conv_state=None, ssm_state=None, delta_softplus=True,
                 want_u=False, want_h=False):
    """Fused forward.  x/delta/z: [B,T,D]; Bm/Cm: [B,T,N]; a_neg [D,N]; Dp [D];
    conv_w [D,K], conv_b [D], conv_state [B,D,K], ssm_state [B,D,N] (copied).
    Returns dict(y, ssm_state, conv_state, u, delta, h_all)."""
    x, delta, Bm, Cm, z = map(_f32, (x, delta, Bm, Cm, z))
    a_neg, Dp, conv_w, conv_b = map(_f32, (a_neg, Dp, conv_w, conv_b))
    B, T, D = delta.shape
    N = a_neg.shape[1]
    K = 0 if conv_w is None else conv_w.shape[1]
    s = _shape(x, delta, Bm, z, N, K, delta_softplus)
    ssm = np.zeros((B, D, N), np.float32) if ssm_state is None else _f32(ssm_state).copy()
    cst = None
    if K:
        cst = np.zeros((B, D, K), np.float32) if conv_state is None else _f32(conv_state).copy()
    y = np.empty((B, T, D), np.float32)
    u = np.empty((B, T, D), np.float32) if want_u else None
    dl = np.empty((B, T, D), np.float32) if want_u else None
    h_all = np.empty((B, T + 1, D, N), np.float32) if want_h else None
    lib().orc_m1_fused_fwd(C.byref(s), _p(x), _p(delta), _p(Bm), _p(Cm), _p(z), _p(a_neg),
                           _p(Dp), _p(conv_w), _p(conv_b), _p(cst), _p(ssm), _p(y), _p(u),
                           _p(dl), _p(h_all))
    return dict(y=y, ssm_state=ssm, conv_state=cst, u=u, delta=dl, h_all=h_all)


def m1_fused_fwd_f64(x, delta, Bm, Cm, z, a_neg, Dp, conv_w=None, conv_b=None,
                     conv_state=None, ssm_state=None, delta_softplus=True):
    f64 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float64)
    x, delta, Bm, Cm, z, a_neg, Dp, conv_w, conv_b = map(
        f64, (x, delta, Bm, Cm, z, a_neg, Dp, conv_w, conv_b))
    B, T, D = delta.shape
    N = a_neg.shape[1]
    K = 0 if conv_w is None else conv_w.shape[1]
    s = _shape(x, delta, Bm, z, N, K, delta_softplus)
    ssm = np.zeros((B, D, N)) if ssm_state is None else f64(ssm_state).copy()
    cst = None
    if K:
        cst = np.zeros((B, D, K)) if conv_state is None else f64(conv_state).copy()
    y = np.empty((B, T, D))
    d = np.float64
    lib().orc_m1_fused_fwd_f64(C.byref(s), _p(x, d), _p(delta, d), _p(Bm, d), _p(Cm, d),
                               _p(z, d), _p(a_neg, d), _p(Dp, d), _p(conv_w, d),
                               _p(conv_b, d), _p(cst, d), _p(ssm, d), _p(y, d))
    return dict(y=y, ssm_state=ssm, conv_state=cst)


def m1_fused_bwd(x, delta, Bm, Cm, z, a_neg, Dp, dg, conv_w=None, conv_b=None,
                 conv_state0=None, ssm_state0=None, delta_softplus=True, d_u_extra=None):
    """Fused backward.  Returns dict(d_x, d_delta, d_z, dB, dC, dA_log, dD,
    dconv_w, dconv_b); parameter gradients start from zero."""
    x, delta, Bm, Cm, z, dg = map(_f32, (x, delta, Bm, Cm, z, dg))
    a_neg, Dp, conv_w, conv_b = map(_f32, (a_neg, Dp, conv_w, conv_b))
    conv_state0, ssm_state0, d_u_extra = map(_f32, (conv_state0, ssm_state0, d_u_extra))
    B, T, D = delta.shape
    N = a_neg.shape[1]
    K = 0 if conv_w is None else conv_w.shape[1]
    s = _shape(x, delta, Bm, z, N, K, delta_softplus)
    d_x = np.zeros((B, T, D), np.float32)
    d_delta = np.zeros((B, T, D), np.float32)
    d_z = np.zeros((B, T, D), np.float32)
    dB = np.zeros((B, T, N), np.float32)
    dC = np.zeros((B, T, N), np.float32)
    dA = np.zeros((D, N), np.float32)
    dD = np.zeros((D,), np.float32)
    dcw = np.zeros((D, max(K, 1)), np.float32)
    dcb = np.zeros((D,), np.float32)
    lib().orc_m1_fused_bwd(C.byref(s), _p(x), _p(delta), _p(Bm), _p(Cm), _p(z), _p(a_neg),
                           _p(Dp), _p(conv_w), _p(conv_b), _p(conv_state0), _p(ssm_state0),
                           _p(dg), _p(d_u_extra), _p(d_x), _p(d_delta), _p(d_z), _p(dB),
                           _p(dC), _p(dA), _p(dD), _p(dcw), _p(dcb))
    return dict(d_x=d_x, d_delta=d_delta, d_z=d_z, dB=dB, dC=dC, dA_log=dA, dD=dD,
                dconv_w=dcw[:, :K] if K else None, dconv_b=dcb if K else None)


def m1_step(x, delta, Bm, Cm, z, a_neg, Dp, conv_w=None, conv_b=None, conv_state=None,
            ssm_state=None, delta_softplus=True):
    """T=1 decode step.  x/delta/z: [B,D]; Bm/Cm: [B,N]."""
    x, delta, Bm, Cm, z = map(_f32, (x, delta, Bm, Cm, z))
    a_neg, Dp, conv_w, conv_b = map(_f32, (a_neg, Dp, conv_w, conv_b))
    B, D = delta.shape
    N = a_neg.shape[1]
    K = 0 if conv_w is None else conv_w.shape[1]
    s = M1Shape(B, 1, D, N, K, x.shape[-1], D, D if z is not None else 0, Bm.shape[-1], D,
                int(delta_softplus), int(z is not None))
    ssm = _f32(ssm_state).copy()
    cst = _f32(conv_state).copy() if K else None
    y = np.empty((B, D), np.float32)
    lib().orc_m1_step(C.byref(s), _p(x), _p(delta), _p(Bm), _p(Cm), _p(z), _p(a_neg), _p(Dp),
                      _p(conv_w), _p(conv_b), _p(cst), _p(ssm), _p(y))
    return dict(y=y, ssm_state=ssm, conv_state=cst)


# -- full backbone (d_model 128, 2 layers, B 4 x T 512 in the tests) --------

def m1_config(d_model=128, n_layers=2, d_state=16, d_conv=4, expand=2, dt_rank=None,
              input_dim=None) -> M1Config:
    dt_rank = dt_rank if dt_rank is not None else (d_model + 15) // 16
    return M1Config(d_model, n_layers, d_state, d_conv, expand, dt_rank,
                    input_dim if input_dim is not None else d_model)


def m1_weights_init(cfg: M1Config, seed: int) -> np.ndarray:
    w = np.empty(lib().orc_m1_weights_floats(C.byref(cfg)), np.float32)
    lib().orc_m1_weights_init(C.byref(cfg), C.c_uint64(seed), _p(w))
    return w


def m1_layer_views(cfg: M1Config, w: np.ndarray):
    """Named views of the flat weight buffer produced by m1_weights_init."""
    dm, di, N, K, dr = cfg.d_model, cfg.d_inner, cfg.d_state, cfg.d_conv, cfg.dt_rank
    xd = cfg.xdbl_dim
    o = 0

    def take(*shape):
        nonlocal o
        n = int(np.prod(shape))
        v = w[o:o + n].reshape(shape)
        o += n
        return v

    out = dict(input_proj_w=take(cfg.input_dim, dm), input_proj_b=take(dm), layers=[])
    for _ in range(cfg.n_layers):
        out["layers"].append(dict(
            norm_w=take(dm), in_proj_w=take(dm, 2 * di), conv_w=take(di, K), conv_b=take(di),
            x_proj_w=take(di, xd), dt_proj_w=take(dr, di), dt_proj_b=take(di),
            a_log=take(di, N), a_neg=take(di, N), d_param=take(di), out_proj_w=take(di, dm)))
    out["norm_f"] = take(dm)
    assert o == w.size
    return out


def m1_prefill(cfg: M1Config, w, inp, conv_state=None, ssm_state=None, taps=False):
    """One-sample backbone prefill.  inp [T,input_dim] -> out [T,d_model]."""
    inp = _f32(inp)
    T = inp.shape[0]
    L, di, N, K = cfg.n_layers, cfg.d_inner, cfg.d_state, cfg.d_conv
    cst = np.zeros((L, di, K), np.float32) if conv_state is None else _f32(conv_state).copy()
    ssm = np.zeros((L, di, N), np.float32) if ssm_state is None else _f32(ssm_state).copy()
    out = np.empty((T, cfg.d_model), np.float32)
    tp = dict(proj=np.empty((L, T, 2 * di), np.float32),
              delta_raw=np.empty((L, T, di), np.float32),
              xdbl=np.empty((L, T, cfg.xdbl_dim), np.float32),
              gated=np.empty((L, T, di), np.float32)) if taps else {}
    lib().orc_m1_prefill(C.byref(cfg), _p(w), _p(inp), C.c_int(T), _p(cst), _p(ssm), _p(out),
                         _p(tp.get("proj")), _p(tp.get("delta_raw")), _p(tp.get("xdbl")),
                         _p(tp.get("gated")))
    return dict(out=out, conv_state=cst, ssm_state=ssm, **tp)


def m1_prefill_batch(cfg: M1Config, w, inp):
    """Batch prefill, one OpenMP task per sample.  inp [B,T,input_dim]."""
    inp = _f32(inp)
    B, T = inp.shape[:2]
    L, di = cfg.n_layers, cfg.d_inner
    cst = np.zeros((B, L, di, cfg.d_conv), np.float32)
    ssm = np.zeros((B, L, di, cfg.d_state), np.float32)
    out = np.empty((B, T, cfg.d_model), np.float32)
    nthr = lib().orc_m1_prefill_batch(C.byref(cfg), _p(w), _p(inp), C.c_int(B), C.c_int(T),
                                      _p(cst), _p(ssm), _p(out))
    return dict(out=out, conv_state=cst, ssm_state=ssm, threads=nthr)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int | None = None) -> int:
    """Use `n` OpenMP threads from now on (default: every core this process may run
    on), whatever OMP_NUM_THREADS said when the library was loaded.  Returns n."""
    if n is None:
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
    lib().orc_set_num_threads(C.c_int(int(n)))
    return int(n)


# -- seeded test inputs ------------------------------------------------------

def det_rand(n: int, seed: int) -> np.ndarray:
    """xorshift32 stream in [-0.5, 0.5) used by the reference's kernel parity
    tests (tests/m1_parallel_bwd_parity.rs:15-25)."""
    s = np.uint32(seed)
    out = np.empty(n, np.float32)
    s = int(s)
    for i in range(n):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = np.float32(s & 0xFFFF) / np.float32(65536.0) - np.float32(0.5)
    return out


def conv1d_fwd(x, w, bias, conv_state=None):
    """Standalone conv1d + SiLU.  x [B,T,D]; returns dict(u, conv_state)."""
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    B, T, D = x.shape
    K = w.shape[1]
    cst = np.zeros((B, D, K), np.float32) if conv_state is None else _f32(conv_state).copy()
    u = np.empty((B, T, D), np.float32)
    lib().orc_conv1d_fwd(B, T, D, K, _p(x), C.c_long(D), _p(w), _p(bias), _p(cst), _p(u))
    return dict(u=u, conv_state=cst)


def conv1d_bwd(x, w, bias, d_u, conv_state0=None):
    """Backward of conv1d + SiLU.  Returns dict(d_x, dconv_w, dconv_b)."""
    x, w, bias, d_u, conv_state0 = map(_f32, (x, w, bias, d_u, conv_state0))
    B, T, D = x.shape
    K = w.shape[1]
    d_x = np.empty((B, T, D), np.float32)
    dW = np.zeros((D, K), np.float32)
    db = np.zeros((D,), np.float32)
    lib().orc_conv1d_bwd(B, T, D, K, _p(x), C.c_long(D), _p(w), _p(bias), _p(conv_state0), _p(d_u),
                         _p(d_x), _p(dW), _p(db))
    return dict(d_x=d_x, dconv_w=dW, dconv_b=db)


# -- Mamba-3 SISO SSD ---------------------------------------------------------

class M3Shape(C.Structure):
    _fields_ = [("B", C.c_int), ("T", C.c_int), ("nh", C.c_int), ("hd", C.c_int), ("N", C.c_int)]


def m3_ssd_fwd(x, K, Q, dt, trap, adt, Dh, ssm=None, kst=None, vst=None, want_h=False):
    """Sequential definition.  x [B,T,nh*hd]; K,Q [B,T,nh,N]; dt,trap,adt [B,T,nh];
    Dh [nh].  Returns dict(y, ssm_state [B,nh,hd,N], k_state, v_state, h_all)."""
    x, K, Q, dt, trap, adt, Dh = map(_f32, (x, K, Q, dt, trap, adt, Dh))
    B, T, nh, N = K.shape
    hd = x.shape[2] // nh
    s = M3Shape(B, T, nh, hd, N)
    ssm = np.zeros((B, nh, hd, N), np.float32) if ssm is None else _f32(ssm).copy()
    kst = np.zeros((B, nh, N), np.float32) if kst is None else _f32(kst).copy()
    vst = np.zeros((B, nh, hd), np.float32) if vst is None else _f32(vst).copy()
    y = np.empty((B, T, nh * hd), np.float32)
    h_all = np.empty((B, T + 1, nh, hd, N), np.float32) if want_h else None
    lib().orc_m3_ssd_fwd(C.byref(s), _p(x), _p(K), _p(Q), _p(dt), _p(trap), _p(adt), _p(Dh), _p(ssm),
                         _p(kst), _p(vst), _p(y), _p(h_all))
    return dict(y=y, ssm_state=ssm, k_state=kst, v_state=vst, h_all=h_all)


def m3_ssd_fwd_f64(x, K, Q, dt, trap, adt, Dh):
    f = lambda a: np.ascontiguousarray(a, dtype=np.float64)
    x, K, Q, dt, trap, adt, Dh = map(f, (x, K, Q, dt, trap, adt, Dh))
    B, T, nh, N = K.shape
    s = M3Shape(B, T, nh, x.shape[2] // nh, N)
    y = np.empty((B, T, x.shape[2]))
    d = np.float64
    lib().orc_m3_ssd_fwd_f64(C.byref(s), _p(x, d), _p(K, d), _p(Q, d), _p(dt, d), _p(trap, d), _p(adt, d),
                             _p(Dh, d), _p(y, d))
    return y


def m3_ssd_fwd_chunked(x, K, Q, dt, trap, adt, Dh, chunk=64):
    x, K, Q, dt, trap, adt, Dh = map(_f32, (x, K, Q, dt, trap, adt, Dh))
    B, T, nh, N = K.shape
    hd = x.shape[2] // nh
    s = M3Shape(B, T, nh, hd, N)
    y = np.empty((B, T, nh * hd), np.float32)
    fs = np.empty((B, nh, hd, N), np.float32)
    lib().orc_m3_ssd_fwd_chunked(C.byref(s), C.c_int(chunk), _p(x), _p(K), _p(Q), _p(dt), _p(trap),
                                 _p(adt), _p(Dh), _p(y), _p(fs))
    return dict(y=y, ssm_state=fs)


def m3_ssd_bwd(x, K, Q, dt, trap, adt, Dh, dy):
    x, K, Q, dt, trap, adt, Dh, dy = map(_f32, (x, K, Q, dt, trap, adt, Dh, dy))
    B, T, nh, N = K.shape
    hd = x.shape[2] // nh
    s = M3Shape(B, T, nh, hd, N)
    z = lambda *sh: np.zeros(sh, np.float32)
    out = dict(dx=z(B, T, nh * hd), dK=z(B, T, nh, N), dQ=z(B, T, nh, N), d_alpha=z(B, T, nh),
               d_beta=z(B, T, nh), d_gamma=z(B, T, nh), d_adt=z(B, T, nh), d_dt=z(B, T, nh),
               d_trap=z(B, T, nh), dD=z(nh))
    lib().orc_m3_ssd_bwd(C.byref(s), _p(x), _p(K), _p(Q), _p(dt), _p(trap), _p(adt), _p(Dh), _p(dy),
                         *[_p(out[k]) for k in ("dx", "dK", "dQ", "d_alpha", "d_beta", "d_gamma", "d_adt",
                                                "d_dt", "d_trap", "dD")])
    return out


# -- the rows around the scan: residual + RMSNorm, loss, optimiser (numpy) -----------

def m3_kq_from_groups(Bn, Cn, b_bias, c_bias, angle_vel, dt, angle_state=None):
    """Per-head K and Q of the Mamba-3 SISO layer from the group-level rows, restating
    src/mamba3_siso/cpu/forward.rs:336-375 (bias add :341-347, angle accumulation in f64
    modulo 2 pi rounded to f32 per step :352-359, rotation of the pairs (2a, 2a+1) :360-372;
    the GPU kernels bc_bias_add / m3_angle_dt_fwd_seq / rope_fwd of kernels/mamba3_ops.cu
    compute the same).  Bn, Cn [B,T,ng,N]; b_bias, c_bias [nh,N]; angle_vel [B,T,n_angles]
    = tanh(angles_raw) * pi; dt [B,T,nh]; angle_state [B,nh,n_angles] (None = zeros).
    Returns K, Q [B,T,nh,N] f32 and the angle after the window [B,nh,n_angles] f32."""
    f = np.float32
    Bn, Cn = np.asarray(Bn, f), np.asarray(Cn, f)
    Bsz, T, ng, N = Bn.shape
    nh = b_bias.shape[0]
    na = angle_vel.shape[2] if angle_vel is not None else 0
    grp = np.arange(nh) // (nh // ng)
    K = (Bn[:, :, grp, :] + np.asarray(b_bias, f)[None, None]).astype(f)
    Q = (Cn[:, :, grp, :] + np.asarray(c_bias, f)[None, None]).astype(f)
    ang = np.zeros((Bsz, nh, max(na, 1)), f) if angle_state is None else np.array(angle_state, f)
    if na:
        two_pi = 2.0 * np.pi
        vel, dtf = np.asarray(angle_vel, f), np.asarray(dt, f)
        for t in range(T):
            delta = (vel[:, t, None, :] * dtf[:, t, :, None]).astype(f)      # f32 product, forward.rs:354
            acc = ang[:, :, :na].astype(np.float64) + delta.astype(np.float64)
            acc -= two_pi * np.floor(acc / two_pi)
            ang[:, :, :na] = acc.astype(f)
            a32 = ang[:, :, :na]
            sn, cs = np.sin(a32).astype(f), np.cos(a32).astype(f)
            for X in (K, Q):
                x0, x1 = X[:, t, :, 0:2 * na:2].copy(), X[:, t, :, 1:2 * na:2].copy()
                X[:, t, :, 0:2 * na:2] = cs * x0 - sn * x1
                X[:, t, :, 1:2 * na:2] = sn * x0 + cs * x1
    return K, Q, ang[:, :, :na].copy()


def residual_rmsnorm_fwd(residual, branch, scale, eps=1e-5):
    """residual_add_f32_{dt} (kernels/elementwise.cu:367-377) followed by
    rmsnorm_forward_f32in_{dt} (kernels/norms.cu:126-168), in f32: returns the new
    residual, y = x / rms * scale, and rms = sqrt(mean(x^2) + eps) per row."""
    x = np.asarray(residual, np.float32)
    if branch is not None:
        x = (x + np.asarray(branch, np.float32)).astype(np.float32)
    rms = np.sqrt((x.astype(np.float64) ** 2).mean(axis=1) + eps).astype(np.float32)
    rms = np.where(np.isfinite(rms) & (rms >= 1e-20), rms, np.float32(1.0))
    y = x * (np.float32(1.0) / rms)[:, None] * np.asarray(scale, np.float32)[None, :]
    return x, y.astype(np.float32), rms


def residual_rmsnorm_bwd(dy, x, scale, rms):
    """rmsnorm_backward (kernels/norms.cu:181-240): dx = (scale*dy - x_hat*mean(dy*y_hat)) /
    rms; d_scale = sum over rows of dy * x_hat.  f64 arithmetic."""
    dy, x, scale, rms = (np.asarray(a, np.float64) for a in (dy, x, scale, rms))
    inv = 1.0 / rms[:, None]
    xh = x * inv
    mean = (dy * xh * scale[None, :]).mean(axis=1, keepdims=True)
    dx = (scale[None, :] * dy - xh * mean) * inv
    return dx, (dy * xh).sum(axis=0)


def softmax_xent(logits, targets, grad_scale=1.0):
    """Cross-entropy per row and its gradient (softmax - onehot) * grad_scale; rows with a
    negative target do not count.  f64 arithmetic."""
    l = np.asarray(logits, np.float64)
    m = l.max(axis=1, keepdims=True)
    e = np.exp(l - m)
    S = e.sum(axis=1, keepdims=True)
    counted = np.asarray(targets) >= 0
    tsafe = np.where(counted, targets, 0)
    loss = (m[:, 0] + np.log(S[:, 0])) - l[np.arange(l.shape[0]), tsafe]
    g = e / S
    g[np.arange(l.shape[0]), tsafe] -= 1.0
    g *= grad_scale
    g[~counted] = 0.0
    return np.where(counted, loss, 0.0), g


def adamw_step(param, grad, m, v, lr, beta1, beta2, eps, wd, step):
    """adamw_step_f32 (kernels/adamw.cu:63-95) in f32, the reference's operation order."""
    f = np.float32
    p, g, m, v = (np.asarray(a, f).copy() for a in (param, grad, m, v))
    bc1 = f(1.0 / (1.0 - beta1 ** step))
    bc2 = f(1.0 / (1.0 - beta2 ** step))
    m = m * f(beta1) + f(1.0 - f(beta1)) * g
    v = v * f(beta2) + f(1.0 - f(beta2)) * g * g
    p = f(1.0 - f(lr) * f(wd)) * p - f(lr) * (m * bc1) / (np.sqrt(v * bc2) + f(eps))
    return p.astype(f), m.astype(f), v.astype(f), (bc1, bc2)
