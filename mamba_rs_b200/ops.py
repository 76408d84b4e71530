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

__all__ = ["selective_scan_fwd", "selective_scan_fwd_workspace_bytes", "selective_scan_bwd",
           "selective_scan_bwd_workspace_bytes",
           "residual_rmsnorm_fwd", "residual_rmsnorm_bwd", "embedding_gather", "softmax_xent", "adamw_step",
           "ssm_parallel_scan_fwd_nosave", "ssm_scan_fwd_save", "ssm_scan_bwd", "conv1d_fwd_nosave", "selective_scan_step", "conv1d_fwd", "conv1d_bwd", "m3_ssd_fwd", "m3_ssd_fwd_fused_kq", "m3_ssd_bwd", "dtype_code"]


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
                       workspace=None, handle=None):
    """Fused forward ``[conv1d+SiLU] -> softplus -> scan -> +D*u -> *SiLU(z)``.

    x, delta, z: [B,T,D]; Bm, Cm: [B,T,N]; a_neg [D,N] f32; Dp [D] f32.
    conv_state [B,D,K] / ssm_state [B,D,N] f32 are updated in place.
    workspace: optional uint8 scratch of selective_scan_fwd_workspace_bytes(...)
    bytes; with it a small batch is cut into time segments that run side by side.
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
    if workspace is not None:
        _require_cuda(workspace)
        a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel() * workspace.element_size()
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


def ssm_scan_fwd_save(h_state, y_out, h_saved, delta, u, Bm, Cm, a_neg, Dp, *, handle=None):
    """Drop-in for the reference's saving forward ``ssm_parallel_scan_fwd_{dt}``
    (kernels/mamba_ssm_parallel.cu:777-790): same tensors; of ``h_saved``
    [B, T+1, D, N] only rows 0, 32, 64, ... are written (what ssm_scan_bwd reads)."""
    _require_cuda(h_state, y_out, h_saved, delta, u, Bm, Cm, a_neg, Dp)
    Bsz, T, D = delta.shape
    N = a_neg.shape[1]
    dev = delta.device
    hd = handle or ffi.default_handle(dev.index or 0)
    if tuple(h_saved.shape) != (Bsz, T + 1, D, N) or h_saved.dtype != torch.float32 or not h_saved.is_contiguous():
        raise ValueError("h_saved must be contiguous float32 [B, T+1, D, N]")
    for t in (y_out, delta, u, Bm, Cm, a_neg, Dp, h_state):
        if not t.is_contiguous():
            raise ValueError("compat entry point takes contiguous tensors")
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_ssm_scan_fwd_save(
            hd.ptr, _stream(dev), C.c_int(dtype_code(delta.dtype)), _ptr(h_state), _ptr(y_out), _ptr(h_saved),
            _ptr(delta), _ptr(u), _ptr(Bm), _ptr(Cm), _ptr(a_neg), _ptr(Dp), Bsz, T, D, N)
    hd.check(rc, "mamba_b200_ssm_scan_fwd_save")
    return y_out


def ssm_scan_bwd(h_saved, delta, u, Bm, Cm, a_neg, Dp, dy, *, d_D=None, d_a_log=None, workspace=None,
                 handle=None):
    """Drop-in for ``ssm_parallel_scan_bwd_{dt}`` / ``ssm_backward_local_{dt}`` plus the four
    reducers (kernels/mamba_ssm_parallel.cu:1182-1200, kernels/mamba_ssm.cu:466-763), on the
    reference's own buffers.  Returns dict(d_delta, d_u, dB, dC, dD, dA_log); d_D / d_a_log
    are accumulated into the tensors passed in (zeros otherwise)."""
    _require_cuda(h_saved, delta, u, Bm, Cm, a_neg, Dp, dy, d_D, d_a_log, workspace)
    Bsz, T, D = delta.shape
    N = a_neg.shape[1]
    dev = delta.device
    hd = handle or ffi.default_handle(dev.index or 0)
    for t in (h_saved, delta, u, Bm, Cm, a_neg, Dp, dy):
        if not t.is_contiguous():
            raise ValueError("compat entry point takes contiguous tensors")
    f32 = dict(dtype=torch.float32, device=dev)
    d_delta, d_u = torch.empty_like(delta), torch.empty_like(u)
    dB, dC = torch.empty((Bsz, T, N), **f32), torch.empty((Bsz, T, N), **f32)
    d_D = torch.zeros(D, **f32) if d_D is None else d_D
    d_a_log = torch.zeros((D, N), **f32) if d_a_log is None else d_a_log
    if workspace is None:
        workspace = torch.empty(max(selective_scan_bwd_workspace_bytes(Bsz, T, D, N), 1), dtype=torch.uint8,
                                device=dev)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_ssm_scan_bwd(
            hd.ptr, _stream(dev), C.c_int(dtype_code(delta.dtype)), _ptr(h_saved), _ptr(delta), _ptr(u), _ptr(Bm),
            _ptr(Cm), _ptr(a_neg), _ptr(Dp), _ptr(dy), _ptr(d_delta), _ptr(d_u), _ptr(dB), _ptr(dC), _ptr(d_D),
            _ptr(d_a_log), Bsz, T, D, N, _ptr(workspace), C.c_longlong(workspace.numel()))
    hd.check(rc, "mamba_b200_ssm_scan_bwd")
    return dict(d_delta=d_delta, d_u=d_u, dB=dB, dC=dC, dD=d_D, dA_log=d_a_log)


def conv1d_fwd_nosave(u_out, state, x, conv_w, conv_b, *, handle=None):
    """Drop-in for ``conv1d_burnin_forward_nosave_{dt}`` (kernels/conv1d.cu:284-296)."""
    _require_cuda(u_out, state, x, conv_w, conv_b)
    Bsz, T, D = x.shape
    dev = x.device
    hd = handle or ffi.default_handle(dev.index or 0)
    for t in (u_out, state, x, conv_w, conv_b):
        if not t.is_contiguous():
            raise ValueError("compat entry point takes contiguous tensors")
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_conv1d_fwd_nosave(hd.ptr, _stream(dev), C.c_int(dtype_code(x.dtype)), _ptr(u_out),
                                                    _ptr(state), _ptr(x), _ptr(conv_w), _ptr(conv_b), Bsz, T, D,
                                                    conv_w.shape[1])
    hd.check(rc, "mamba_b200_conv1d_fwd_nosave")
    return u_out


def selective_scan_fwd_workspace_bytes(B, T, D, N) -> int:
    """Bytes of the optional forward scratch (segment hand-over states)."""
    return int(ffi.lib().mamba_b200_sscan_fwd_workspace_bytes(B, T, D, N))


def selective_scan_bwd_workspace_bytes(B, T, D, N) -> int:
    """Bytes of caller-owned scratch the backward needs (per-tile dB/dC partials
    and per-sample dA_log / dD partials)."""
    return int(ffi.lib().mamba_b200_sscan_bwd_workspace_bytes(B, T, D, N))


def selective_scan_bwd(u, delta, Bm, Cm, a_neg, Dp, dy, chunk_states, save_stride, z=None, *,
                       z_mode=None, delta_softplus=True, dA_log=None, dD=None, workspace=None,
                       handle=None):
    """Fused backward (BPTT by recomputation from the saved block-boundary
    states).  Returns dict(d_u, d_delta, d_z, dB, dC, dA_log, dD); dA_log and
    dD are accumulated into the tensors passed in (zeros if none are passed)."""
    _require_cuda(u, delta, Bm, Cm, a_neg, Dp, dy, chunk_states, z)
    Bsz, T, D = delta.shape
    N = a_neg.shape[1]
    dev = u.device
    h = handle or ffi.default_handle(dev.index or 0)
    if z_mode is None:
        z_mode = 0 if z is None else 1
    f32 = dict(dtype=torch.float32, device=dev)
    d_u = torch.empty((Bsz, T, D), dtype=u.dtype, device=dev)
    d_delta = torch.empty((Bsz, T, D), dtype=u.dtype, device=dev)
    d_z = torch.empty((Bsz, T, D), dtype=u.dtype, device=dev) if z_mode else None
    dB = torch.empty((Bsz, T, N), **f32)
    dC = torch.empty((Bsz, T, N), **f32)
    dA_log = torch.zeros((D, N), **f32) if dA_log is None else dA_log
    dD = torch.zeros((D,), **f32) if dD is None else dD
    need = selective_scan_bwd_workspace_bytes(Bsz, T, D, N)
    if workspace is None:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
    a = ffi.SscanBwdArgs()
    a.dtype = dtype_code(u.dtype)
    a.B, a.T, a.D, a.N = Bsz, T, D, N
    a.u, a.ld_u = _ptr(u), _rows(u, "u")
    a.delta, a.ld_delta, a.delta_softplus = _ptr(delta), _rows(delta, "delta"), int(delta_softplus)
    a.Bm, a.Cm, a.ld_bc = _ptr(Bm), _ptr(Cm), _rows(Bm, "B")
    a.z, a.ld_z, a.z_mode = _ptr(z), (_rows(z, "z") if z is not None else 0), int(z_mode)
    a.a_neg, a.Dp = _ptr(a_neg), _ptr(Dp)
    a.chunk_states, a.save_stride = _ptr(chunk_states), int(save_stride)
    a.dy, a.ld_dy = _ptr(dy), _rows(dy, "dy")
    a.d_u, a.ld_du = _ptr(d_u), D
    a.d_delta, a.ld_ddelta = _ptr(d_delta), D
    a.d_z, a.ld_dz = _ptr(d_z), D
    a.dBm, a.dCm, a.dA_log, a.dD = _ptr(dB), _ptr(dC), _ptr(dA_log), _ptr(dD)
    a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel()
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_sscan_bwd(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_sscan_bwd")
    return dict(d_u=d_u, d_delta=d_delta, d_z=d_z, dB=dB, dC=dC, dA_log=dA_log, dD=dD)


def selective_scan_step(x, delta, Bm, Cm, a_neg, Dp, ssm_state, z=None, *, z_mode=None,
                        delta_softplus=True, conv_w=None, conv_b=None, conv_state=None, y=None,
                        u_out=None, handle=None):
    """T = 1 decode step (GpuMambaBackbone::step inner kernels).  x, delta, z:
    [B,D]; Bm, Cm: [B,N] (views of xdbl are fine); states updated in place."""
    _require_cuda(x, delta, Bm, Cm, a_neg, Dp, ssm_state, z, conv_w, conv_b, conv_state)
    Bsz, D = delta.shape
    N = a_neg.shape[1]
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    if y is None:
        y = torch.empty((Bsz, D), dtype=x.dtype, device=dev)
    if z_mode is None:
        z_mode = 0 if z is None else 1
    a = ffi.SscanStepArgs()
    a.dtype = dtype_code(x.dtype)
    a.B, a.D, a.N = Bsz, D, N
    a.x, a.ld_x = _ptr(x), x.stride(0)
    a.delta, a.ld_delta, a.delta_softplus = _ptr(delta), delta.stride(0), int(delta_softplus)
    a.Bm, a.Cm, a.ld_bc = _ptr(Bm), _ptr(Cm), Bm.stride(0)
    a.z, a.ld_z, a.z_mode = _ptr(z), (z.stride(0) if z is not None else 0), int(z_mode)
    a.a_neg, a.Dp = _ptr(a_neg), _ptr(Dp)
    a.conv_w, a.conv_b, a.conv_state = _ptr(conv_w), _ptr(conv_b), _ptr(conv_state)
    a.K = conv_w.shape[1] if conv_w is not None else 0
    a.ssm_state = _ptr(ssm_state)
    a.y, a.ld_y = _ptr(y), y.stride(0)
    a.u_out, a.ld_u = _ptr(u_out), (u_out.stride(0) if u_out is not None else 0)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_sscan_step(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_sscan_step")
    return y


def conv1d_fwd(x, conv_w, conv_b, conv_state=None, u=None, *, handle=None):
    """Depthwise causal conv1d + SiLU over [B,T,D]; conv_state [B,D,K] in/out."""
    _require_cuda(x, conv_w, conv_b, conv_state, u)
    Bsz, T, D = x.shape
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    if u is None:
        u = torch.empty((Bsz, T, D), dtype=x.dtype, device=dev)
    a = ffi.Conv1dArgs()
    a.dtype = dtype_code(x.dtype)
    a.B, a.T, a.D, a.K = Bsz, T, D, conv_w.shape[1]
    a.x, a.ld_x = _ptr(x), _rows(x, "x")
    a.conv_w, a.conv_b, a.conv_state = _ptr(conv_w), _ptr(conv_b), _ptr(conv_state)
    a.u, a.ld_u = _ptr(u), _rows(u, "u")
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_conv1d_fwd(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_conv1d_fwd")
    return u


def conv1d_bwd(x, conv_w, conv_b, d_u, conv_state0=None, *, dconv_w=None, dconv_b=None,
               workspace=None, handle=None):
    """Backward of conv1d + SiLU by recomputation.  Returns dict(d_x, dconv_w,
    dconv_b); the parameter gradients are accumulated into the tensors given."""
    _require_cuda(x, conv_w, conv_b, d_u, conv_state0)
    Bsz, T, D = x.shape
    K = conv_w.shape[1]
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    d_x = torch.empty((Bsz, T, D), dtype=x.dtype, device=dev)
    dconv_w = torch.zeros((D, K), dtype=torch.float32, device=dev) if dconv_w is None else dconv_w
    dconv_b = torch.zeros((D,), dtype=torch.float32, device=dev) if dconv_b is None else dconv_b
    need = int(ffi.lib().mamba_b200_conv1d_bwd_workspace_bytes(Bsz, T, D, K))
    if workspace is None:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
    a = ffi.Conv1dArgs()
    a.dtype = dtype_code(x.dtype)
    a.B, a.T, a.D, a.K = Bsz, T, D, K
    a.x, a.ld_x = _ptr(x), _rows(x, "x")
    a.conv_w, a.conv_b, a.conv_state = _ptr(conv_w), _ptr(conv_b), _ptr(conv_state0)
    a.d_u, a.ld_du = _ptr(d_u), _rows(d_u, "d_u")
    a.d_x, a.ld_dx = _ptr(d_x), D
    a.dconv_w, a.dconv_b = _ptr(dconv_w), _ptr(dconv_b)
    a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel()
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_conv1d_bwd(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_conv1d_bwd")
    return dict(d_x=d_x, dconv_w=dconv_w, dconv_b=dconv_b)


def m3_ssd_fwd(x, K, Q, dt, trap, adt, Dh, *, ssm_state=None, k_state=None, v_state=None,
               carry_in=False, force_sequential=False, y=None, handle=None):
    """Mamba-3 SISO SSD forward.  x [B,T,nh*hd], K/Q [B,T,nh,N] in the storage
    dtype (contiguous); dt, trap, adt [B,T,nh] and Dh [nh] f32.  State tensors
    (f32) receive the state after the window; with carry_in they are read first."""
    _require_cuda(x, K, Q, dt, trap, adt, Dh, ssm_state, k_state, v_state, y)
    Bsz, T, nh, N = K.shape
    hd = x.shape[2] // nh
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    for t, nm in ((x, "x"), (K, "K"), (Q, "Q")):
        if not t.is_contiguous() or t.dtype != x.dtype:
            raise ValueError(f"{nm} must be contiguous and share x's dtype")
    for t, nm in ((dt, "dt"), (trap, "trap"), (adt, "adt"), (Dh, "Dh"), (ssm_state, "ssm_state"),
                  (k_state, "k_state"), (v_state, "v_state")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError(f"{nm} must be contiguous float32")
    if y is None:
        y = torch.empty_like(x)
    a = ffi.M3SsdArgs()
    a.dtype = dtype_code(x.dtype)
    a.B, a.T, a.nh, a.hd, a.N = Bsz, T, nh, hd, N
    a.x, a.K, a.Q = _ptr(x), _ptr(K), _ptr(Q)
    a.dt, a.trap, a.adt, a.Dh = _ptr(dt), _ptr(trap), _ptr(adt), _ptr(Dh)
    a.y = _ptr(y)
    a.ssm_state, a.k_state, a.v_state = _ptr(ssm_state), _ptr(k_state), _ptr(v_state)
    a.carry_in, a.force_sequential = int(carry_in), int(force_sequential)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_m3_ssd_fwd(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_m3_ssd_fwd")
    return y


def m3_ssd_fwd_fused_kq(x, Bn, Cn, b_bias, c_bias, angle_vel, dt, trap, adt, Dh, *, angle_state=None,
                        ssm_state=None, k_state=None, v_state=None, y=None, handle=None):
    """Mamba-3 SISO SSD forward with the per-head K / Q built inside the kernel (bias add +
    RoPE with the running angle) from the group-level rows.  x [B,T,nh*hd], Bn / Cn
    [B,T,ng,N] in the 16-bit storage dtype; b_bias, c_bias [nh,N], angle_vel [B,T,n_angles]
    (= tanh(angles_raw) * pi; None = no rotation), dt, trap, adt [B,T,nh], Dh [nh] f32;
    angle_state [B,nh,n_angles] f32 is read and overwritten with the angle after the window."""
    _require_cuda(x, Bn, Cn, b_bias, c_bias, angle_vel, dt, trap, adt, Dh, angle_state, ssm_state, k_state,
                  v_state, y)
    Bsz, T, ng, N = Bn.shape
    nh = b_bias.shape[0]
    hd = x.shape[2] // nh
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    for t, nm in ((x, "x"), (Bn, "Bn"), (Cn, "Cn")):
        if not t.is_contiguous() or t.dtype != x.dtype:
            raise ValueError(f"{nm} must be contiguous and share x's dtype")
    for t, nm in ((b_bias, "b_bias"), (c_bias, "c_bias"), (angle_vel, "angle_vel"), (dt, "dt"), (trap, "trap"),
                  (adt, "adt"), (Dh, "Dh"), (angle_state, "angle_state"), (ssm_state, "ssm_state"),
                  (k_state, "k_state"), (v_state, "v_state")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError(f"{nm} must be contiguous float32")
    if y is None:
        y = torch.empty_like(x)
    a = ffi.M3SsdArgs()
    a.dtype = dtype_code(x.dtype)
    a.B, a.T, a.nh, a.hd, a.N = Bsz, T, nh, hd, N
    a.x = _ptr(x)
    a.dt, a.trap, a.adt, a.Dh = _ptr(dt), _ptr(trap), _ptr(adt), _ptr(Dh)
    a.y = _ptr(y)
    a.ssm_state, a.k_state, a.v_state = _ptr(ssm_state), _ptr(k_state), _ptr(v_state)
    a.Bn, a.Cn, a.b_bias, a.c_bias = _ptr(Bn), _ptr(Cn), _ptr(b_bias), _ptr(c_bias)
    a.angle_vel, a.angle_state = _ptr(angle_vel), _ptr(angle_state)
    a.ng, a.n_angles = ng, (angle_vel.shape[2] if angle_vel is not None else 0)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_m3_ssd_fwd(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_m3_ssd_fwd")
    return y


def m3_ssd_bwd(x, K, Q, dt, trap, adt, Dh, dy, *, dD=None, workspace=None, handle=None):
    """Mamba-3 SISO SSD backward for a window that started from a zero state.
    Returns dx (storage dtype), dK, dQ, d_adt, d_dt, d_trap (f32) and dD (f32,
    accumulated into the tensor passed in, or a fresh zero one).  d_dt is the
    direct path only; the caller adds A * d_adt (src/mamba3_siso/gpu/backward.rs:420-457)."""
    _require_cuda(x, K, Q, dt, trap, adt, Dh, dy, dD, workspace)
    Bsz, T, nh, N = K.shape
    hd = x.shape[2] // nh
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    for t, nm in ((x, "x"), (K, "K"), (Q, "Q"), (dy, "dy")):
        if not t.is_contiguous() or t.dtype != x.dtype:
            raise ValueError(f"{nm} must be contiguous and share x's dtype")
    for t, nm in ((dt, "dt"), (trap, "trap"), (adt, "adt"), (Dh, "Dh"), (dD, "dD")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise TypeError(f"{nm} must be contiguous float32")
    need = ffi.lib().mamba_b200_m3_ssd_bwd_workspace_bytes_for(dtype_code(x.dtype), Bsz, T, nh, hd, N)
    if workspace is None:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    dx = torch.empty_like(x)
    dK = torch.empty((Bsz, T, nh, N), **f32)
    dQ = torch.empty((Bsz, T, nh, N), **f32)
    d_adt = torch.empty((Bsz, T, nh), **f32)
    d_dt = torch.empty((Bsz, T, nh), **f32)
    d_trap = torch.empty((Bsz, T, nh), **f32)
    if dD is None:
        dD = torch.zeros(nh, **f32)
    a = ffi.M3SsdBwdArgs()
    a.dtype = dtype_code(x.dtype)
    a.B, a.T, a.nh, a.hd, a.N = Bsz, T, nh, hd, N
    a.x, a.K, a.Q, a.dy = _ptr(x), _ptr(K), _ptr(Q), _ptr(dy)
    a.dt, a.trap, a.adt, a.Dh = _ptr(dt), _ptr(trap), _ptr(adt), _ptr(Dh)
    a.dx, a.dK, a.dQ = _ptr(dx), _ptr(dK), _ptr(dQ)
    a.d_adt, a.d_dt, a.d_trap, a.dD = _ptr(d_adt), _ptr(d_dt), _ptr(d_trap), _ptr(dD)
    a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel()
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_m3_ssd_bwd(h.ptr, _stream(dev), C.byref(a))
    h.check(rc, "mamba_b200_m3_ssd_bwd")
    return dict(dx=dx, dK=dK, dQ=dQ, d_adt=d_adt, d_dt=d_dt, d_trap=d_trap, dD=dD)


def residual_rmsnorm_fwd(residual, branch, scale, *, eps=1e-5, out_dtype=None, y=None, rms_out=None, handle=None):
    """residual [rows, dim] f32 += branch (storage dtype, or None); returns
    (y = rmsnorm(residual) * scale in the storage dtype, rms [rows] f32)."""
    _require_cuda(residual, branch, scale, y, rms_out)
    rows, dim = residual.shape
    dev = residual.device
    h = handle or ffi.default_handle(dev.index or 0)
    if residual.dtype != torch.float32 or not residual.is_contiguous() or not scale.is_contiguous():
        raise TypeError("residual and scale are contiguous float32")
    dt = branch.dtype if branch is not None else (out_dtype or torch.bfloat16)
    if branch is not None and (not branch.is_contiguous() or tuple(branch.shape) != (rows, dim)):
        raise ValueError("branch must be contiguous [rows, dim]")
    if y is None:
        y = torch.empty((rows, dim), dtype=dt, device=dev)
    if rms_out is None:
        rms_out = torch.empty(rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_residual_rmsnorm_fwd(h.ptr, _stream(dev), dtype_code(dt), _ptr(residual), _ptr(branch),
                                                       _ptr(scale), _ptr(y), _ptr(rms_out), rows, dim, float(eps))
    h.check(rc, "mamba_b200_residual_rmsnorm_fwd")
    return y, rms_out


def residual_rmsnorm_bwd(dy, x, scale, rms_saved, d_residual, d_scale, *, workspace=None, handle=None):
    """d_residual [rows, dim] f32 += dx of the RMSNorm; d_scale [dim] f32 += its scale
    gradient.  x is the f32 residual the forward normalised, rms_saved its per-row rms."""
    _require_cuda(dy, x, scale, rms_saved, d_residual, d_scale, workspace)
    rows, dim = x.shape
    dev = x.device
    h = handle or ffi.default_handle(dev.index or 0)
    need = int(ffi.lib().mamba_b200_residual_rmsnorm_bwd_workspace_bytes(rows, dim))
    if workspace is None:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_residual_rmsnorm_bwd(h.ptr, _stream(dev), dtype_code(dy.dtype), _ptr(dy), _ptr(x),
                                                       _ptr(scale), _ptr(rms_saved), _ptr(d_residual), _ptr(d_scale),
                                                       rows, dim, _ptr(workspace), workspace.numel())
    h.check(rc, "mamba_b200_residual_rmsnorm_bwd")
    return d_residual, d_scale


def embedding_gather(table, ids, out=None, *, handle=None):
    """out [rows, dim] f32 = table[ids] (table [vocab, dim] in the storage dtype, ids int32)."""
    _require_cuda(table, ids, out)
    vocab, dim = table.shape
    dev = table.device
    h = handle or ffi.default_handle(dev.index or 0)
    ids = ids.reshape(-1)
    if ids.dtype != torch.int32 or not ids.is_contiguous() or not table.is_contiguous():
        raise TypeError("ids are contiguous int32, the table is contiguous")
    if out is None:
        out = torch.empty((ids.numel(), dim), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_embedding_gather(h.ptr, _stream(dev), dtype_code(table.dtype), _ptr(table), _ptr(ids),
                                                   _ptr(out), ids.numel(), dim, vocab)
    h.check(rc, "mamba_b200_embedding_gather")
    return out


def softmax_xent(logits, targets, *, grad_scale=1.0, want_grad=True, dlogits=None, handle=None):
    """Per-row cross-entropy of logits [rows, V] against int32 targets (negative = not
    counted).  Returns (loss_rows f32 [rows], d_logits in the logits' dtype or None)."""
    _require_cuda(logits, targets, dlogits)
    rows, V = logits.shape
    dev = logits.device
    h = handle or ffi.default_handle(dev.index or 0)
    if logits.stride(1) != 1 or targets.dtype != torch.int32 or not targets.is_contiguous():
        raise TypeError("logits rows are contiguous, targets are contiguous int32")
    loss = torch.empty(rows, dtype=torch.float32, device=dev)
    if want_grad and dlogits is None:
        dlogits = torch.empty_strided(logits.shape, logits.stride(), dtype=logits.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_softmax_xent(h.ptr, _stream(dev), dtype_code(logits.dtype), _ptr(logits), _ptr(targets),
                                               _ptr(loss), _ptr(dlogits if want_grad else None), float(grad_scale),
                                               rows, V, logits.stride(0))
    h.check(rc, "mamba_b200_softmax_xent")
    return loss, (dlogits if want_grad else None)


def adamw_step(param, grad, m, v, bias_factors, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
               param_lp=None, handle=None):
    """In-place AdamW on flat f32 arenas; bias_factors is a 2-float device tensor
    {1/(1-beta1^t), 1/(1-beta2^t)}; param_lp (f16 / bf16) receives the compute copy."""
    _require_cuda(param, grad, m, v, bias_factors, param_lp)
    dev = param.device
    h = handle or ffi.default_handle(dev.index or 0)
    for t in (param, grad, m, v, bias_factors):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("AdamW state is contiguous float32")
    with torch.cuda.device(dev):
        rc = ffi.lib().mamba_b200_adamw_step(h.ptr, _stream(dev), _ptr(param), _ptr(grad), _ptr(m), _ptr(v), float(lr),
                                             float(beta1), float(beta2), float(eps), float(weight_decay),
                                             _ptr(bias_factors), _ptr(param_lp),
                                             dtype_code(param_lp.dtype) if param_lp is not None else ffi.BF16,
                                             param.numel())
    h.check(rc, "mamba_b200_adamw_step")
    return param
