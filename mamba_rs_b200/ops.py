"""Operator layer over the C ABI, on torch CUDA tensors.

Names and argument meaning follow the reference's launch sites
(src/mamba_ssm/gpu/forward_mixed.rs:433-758, prefill.rs:676-961): activations
are ``[B, T, D]`` row-major views (a last-dim stride of 1 and any row stride, so
the x / z halves of ``proj[B*T, 2D]`` and the B / C columns of ``xdbl`` are
passed in place), state tensors are f32.  torch is used for device memory and
streams only; every compute call goes through ``libmamba_b200.so``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import ffi

__all__ = ["selective_scan_fwd", "ssm_parallel_scan_fwd_nosave", "dtype_code"]


def dtype_code(dt: torch.dtype) -> int:
    try:
        return {torch.float32: ffi.F32, torch.float16: ffi.F16, torch.bfloat16: ffi.BF16}[dt]
    except KeyError:
        raise TypeError(f"unsupported storage dtype {dt} (WeightDtype is f32 / f16 / bf16)")


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mamba_rs_b200 ops take CUDA tensors only (no CPU fallback)")


def _rows(t: torch.Tensor, name: str) -> int:
    """Row stride (elements) of a [B, T, C] or [B*T, C] activation view."""
    if t.stride(-1) != 1:
        raise ValueError(f"{name}: last dimension must be contiguous")
    ld = t.stride(-2)
    if t.dim() == 3 and t.shape[0] > 1 and t.stride(0) != t.shape[1] * ld:
        raise ValueError(f"{name}: batch stride must equal T * row stride")
    return ld


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def selective_scan_fwd(x, delta, Bm, Cm, a_neg, Dp, z=None, *, z_mode=None,
                       delta_softplus=True, conv_w=None, conv_b=None, conv_state=None,
                       ssm_state=None, y=None, u_out=None, chunk_states=None, save_stride=0,
                       handle=None):
    """Fused forward ``[conv1d+SiLU] -> softplus -> scan -> +D*u -> *SiLU(z)``.

    x, delta, z: [B,T,D]; Bm, Cm: [B,T,N]; a_neg [D,N] f32; Dp [D] f32.
    conv_state [B,D,K] / ssm_state [B,D,N] f32 are updated in place.
    Returns y [B,T,D] in the storage dtype of x."""
    _require_cuda(x, delta, Bm, Cm, a_neg, Dp, z, conv_w, conv_b, conv_state, ssm_state, y, u_out)
    Bsz, T, D = delta.shape
    N = a_neg.shape[1]
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    if y is None:
        y = torch.empty((Bsz, T, D), dtype=x.dtype, device=dev)
    if z_mode is None:
        z_mode = 0 if z is None else 1
    a = ffi.SscanFwdArgs()
    a.dtype = dtype_code(x.dtype)
    for t, nm in ((delta, "delta"), (Bm, "B"), (Cm, "C"), (z, "z"), (y, "y"), (u_out, "u_out")):
        if t is not None and t.dtype != x.dtype:
            raise TypeError(f"{nm} dtype {t.dtype} != x dtype {x.dtype}")
    for t, nm in ((a_neg, "a_neg"), (Dp, "D"), (conv_w, "conv_w"), (conv_b, "conv_b"),
                  (conv_state, "conv_state"), (ssm_state, "ssm_state"), (chunk_states, "chunk_states")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError(f"{nm} must be contiguous float32")
    a.B, a.T, a.D, a.N = Bsz, T, D, N
    a.x, a.ld_x = _ptr(x), _rows(x, "x")
    a.delta, a.ld_delta, a.delta_softplus = _ptr(delta), _rows(delta, "delta"), int(delta_softplus)
    if _rows(Bm, "B") != _rows(Cm, "C"):
        raise ValueError("B and C must share a row stride")
    a.Bm, a.Cm, a.ld_bc = _ptr(Bm), _ptr(Cm), _rows(Bm, "B")
    a.z, a.ld_z, a.z_mode = _ptr(z), (_rows(z, "z") if z is not None else 0), int(z_mode)
    a.a_neg, a.Dp = _ptr(a_neg), _ptr(Dp)
    a.conv_w, a.conv_b, a.conv_state = _ptr(conv_w), _ptr(conv_b), _ptr(conv_state)
    a.K = conv_w.shape[1] if conv_w is not None else 0
    a.ssm_state = _ptr(ssm_state)
    a.y, a.ld_y = _ptr(y), _rows(y, "y")
    a.u_out, a.ld_u = _ptr(u_out), (_rows(u_out, "u_out") if u_out is not None else 0)
    a.chunk_states, a.save_stride = _ptr(chunk_states), int(save_stride)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_sscan_fwd(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_sscan_fwd")
    return y


def ssm_parallel_scan_fwd_nosave(h_state, y_out, delta, u, Bm, Cm, a_neg, Dp, *, handle=None):
    """Drop-in for the reference kernel ``ssm_parallel_scan_fwd_nosave_{dt}``
    (kernels/mamba_ssm_parallel.cu:544-553): contiguous tensors, delta already
    softplus'ed, ``h_state`` [B,D,N] f32 updated in place, ``y_out`` written."""
    _require_cuda(h_state, y_out, delta, u, Bm, Cm, a_neg, Dp)
    Bsz, T, D = delta.shape
    N = a_neg.shape[1]
    dev = delta.device
    hd = handle or ffi.default_handle(dev.index or 0)
    for t in (y_out, delta, u, Bm, Cm, a_neg, Dp, h_state):
        if not t.is_contiguous():
            raise ValueError("compat entry point takes contiguous tensors")
    fn = ffi.lib().mamba_b200_ssm_scan_fwd_nosave
    with torch.cuda.device(dev):
        rc = fn(hd.ptr, _stream(dev), C.c_int(dtype_code(delta.dtype)), _ptr(h_state), _ptr(y_out),
                _ptr(delta), _ptr(u), _ptr(Bm), _ptr(Cm), _ptr(a_neg), _ptr(Dp), C.c_int(Bsz),
                C.c_int(T), C.c_int(D), C.c_int(N))
    hd.check(rc, "mamba_b200_ssm_scan_fwd_nosave")
    return y_out
