"""ctypes binding of ``include/mamba_b200.h`` (the same declarations a Rust
``extern "C"`` block would carry)."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# MAMBA_B200_LIB selects another build of the same ABI (tuning builds).
_LIB = os.environ.get("MAMBA_B200_LIB") or os.path.join(HERE, "libmamba_b200.so")

F32, F16, BF16 = 0, 1, 2


class LibraryMissing(RuntimeError):
    pass


def lib_path() -> str:
    return _LIB


class SscanFwdArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("B", C.c_int), ("T", C.c_int), ("D", C.c_int), ("N", C.c_int),
        ("x", C.c_void_p), ("ld_x", C.c_longlong),
        ("delta", C.c_void_p), ("ld_delta", C.c_longlong), ("delta_softplus", C.c_int),
        ("Bm", C.c_void_p), ("Cm", C.c_void_p), ("ld_bc", C.c_longlong),
        ("z", C.c_void_p), ("ld_z", C.c_longlong), ("z_mode", C.c_int),
        ("a_neg", C.c_void_p), ("Dp", C.c_void_p),
        ("conv_w", C.c_void_p), ("conv_b", C.c_void_p), ("conv_state", C.c_void_p), ("K", C.c_int),
        ("ssm_state", C.c_void_p),
        ("y", C.c_void_p), ("ld_y", C.c_longlong),
        ("u_out", C.c_void_p), ("ld_u", C.c_longlong),
        ("chunk_states", C.c_void_p), ("save_stride", C.c_int),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_longlong),
    ]


class SscanBwdArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("B", C.c_int), ("T", C.c_int), ("D", C.c_int), ("N", C.c_int),
        ("u", C.c_void_p), ("ld_u", C.c_longlong),
        ("delta", C.c_void_p), ("ld_delta", C.c_longlong), ("delta_softplus", C.c_int),
        ("Bm", C.c_void_p), ("Cm", C.c_void_p), ("ld_bc", C.c_longlong),
        ("z", C.c_void_p), ("ld_z", C.c_longlong), ("z_mode", C.c_int),
        ("a_neg", C.c_void_p), ("Dp", C.c_void_p),
        ("chunk_states", C.c_void_p), ("save_stride", C.c_int),
        ("dy", C.c_void_p), ("ld_dy", C.c_longlong),
        ("d_u", C.c_void_p), ("ld_du", C.c_longlong),
        ("d_delta", C.c_void_p), ("ld_ddelta", C.c_longlong),
        ("d_z", C.c_void_p), ("ld_dz", C.c_longlong),
        ("dBm", C.c_void_p), ("dCm", C.c_void_p), ("dA_log", C.c_void_p), ("dD", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_longlong),
    ]


class SscanStepArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("B", C.c_int), ("D", C.c_int), ("N", C.c_int),
        ("x", C.c_void_p), ("ld_x", C.c_longlong),
        ("delta", C.c_void_p), ("ld_delta", C.c_longlong), ("delta_softplus", C.c_int),
        ("Bm", C.c_void_p), ("Cm", C.c_void_p), ("ld_bc", C.c_longlong),
        ("z", C.c_void_p), ("ld_z", C.c_longlong), ("z_mode", C.c_int),
        ("a_neg", C.c_void_p), ("Dp", C.c_void_p),
        ("conv_w", C.c_void_p), ("conv_b", C.c_void_p), ("conv_state", C.c_void_p), ("K", C.c_int),
        ("ssm_state", C.c_void_p),
        ("y", C.c_void_p), ("ld_y", C.c_longlong),
        ("u_out", C.c_void_p), ("ld_u", C.c_longlong),
    ]


class Conv1dArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("B", C.c_int), ("T", C.c_int), ("D", C.c_int), ("K", C.c_int),
        ("x", C.c_void_p), ("ld_x", C.c_longlong),
        ("conv_w", C.c_void_p), ("conv_b", C.c_void_p), ("conv_state", C.c_void_p),
        ("u", C.c_void_p), ("ld_u", C.c_longlong),
        ("d_u", C.c_void_p), ("ld_du", C.c_longlong),
        ("d_x", C.c_void_p), ("ld_dx", C.c_longlong),
        ("dconv_w", C.c_void_p), ("dconv_b", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_longlong),
    ]


class M3SsdArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("B", C.c_int), ("T", C.c_int), ("nh", C.c_int), ("hd", C.c_int), ("N", C.c_int),
        ("x", C.c_void_p), ("K", C.c_void_p), ("Q", C.c_void_p),
        ("dt", C.c_void_p), ("trap", C.c_void_p), ("adt", C.c_void_p), ("Dh", C.c_void_p),
        ("y", C.c_void_p),
        ("ssm_state", C.c_void_p), ("k_state", C.c_void_p), ("v_state", C.c_void_p),
        ("carry_in", C.c_int), ("force_sequential", C.c_int),
        ("Bn", C.c_void_p), ("Cn", C.c_void_p), ("b_bias", C.c_void_p), ("c_bias", C.c_void_p),
        ("angle_vel", C.c_void_p), ("angle_state", C.c_void_p), ("ng", C.c_int), ("n_angles", C.c_int),
    ]


class M3SsdBwdArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("B", C.c_int), ("T", C.c_int), ("nh", C.c_int), ("hd", C.c_int), ("N", C.c_int),
        ("x", C.c_void_p), ("K", C.c_void_p), ("Q", C.c_void_p),
        ("dt", C.c_void_p), ("trap", C.c_void_p), ("adt", C.c_void_p), ("Dh", C.c_void_p),
        ("dy", C.c_void_p), ("dx", C.c_void_p), ("dK", C.c_void_p), ("dQ", C.c_void_p),
        ("d_adt", C.c_void_p), ("d_dt", C.c_void_p), ("d_trap", C.c_void_p), ("dD", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_longlong),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load the library; raises LibraryMissing (never falls back) if absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            raise LibraryMissing(
                f"{_LIB} not found: build it with `python -m mamba_rs_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        _lib = C.CDLL(_LIB)
        _lib.mamba_b200_last_error.restype = C.c_char_p
        _lib.mamba_b200_last_error.argtypes = [C.c_void_p]
        _lib.mamba_b200_init.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
        _lib.mamba_b200_destroy.argtypes = [C.c_void_p]
        _lib.mamba_b200_check_status.argtypes = [C.c_void_p, C.c_void_p]

        def bind(name, argtypes, restype=C.c_int):
            # a tuning build selected through MAMBA_B200_LIB may hold a subset of the
            # entry points; the shipped library exports all of them (tests/test_abi.py)
            if hasattr(_lib, name):
                fn = getattr(_lib, name)
                fn.argtypes, fn.restype = argtypes, restype
            elif not os.environ.get("MAMBA_B200_LIB"):
                raise LibraryMissing(f"{_LIB} does not export {name}: rebuild it")

        vp = C.c_void_p
        bind("mamba_b200_selftest_wait_timeout", [vp, vp, C.c_int])
        bind("mamba_b200_sscan_fwd", [vp, vp, C.POINTER(SscanFwdArgs)])
        bind("mamba_b200_sscan_fwd_workspace_bytes", [C.c_int] * 4, C.c_longlong)
        bind("mamba_b200_sscan_bwd", [vp, vp, C.POINTER(SscanBwdArgs)])
        bind("mamba_b200_ssm_scan_fwd_nosave", [vp, vp, C.c_int] + [vp] * 8 + [C.c_int] * 4)
        bind("mamba_b200_ssm_scan_fwd_save", [vp, vp, C.c_int] + [vp] * 9 + [C.c_int] * 4)
        bind("mamba_b200_ssm_scan_bwd", [vp, vp, C.c_int] + [vp] * 14 + [C.c_int] * 4 + [vp, C.c_longlong])
        bind("mamba_b200_conv1d_fwd_nosave", [vp, vp, C.c_int] + [vp] * 5 + [C.c_int] * 4)
        bind("mamba_b200_sscan_bwd_workspace_bytes", [C.c_int] * 4, C.c_longlong)
        bind("mamba_b200_sscan_step", [vp, vp, C.POINTER(SscanStepArgs)])
        bind("mamba_b200_conv1d_fwd", [vp, vp, C.POINTER(Conv1dArgs)])
        bind("mamba_b200_conv1d_bwd", [vp, vp, C.POINTER(Conv1dArgs)])
        bind("mamba_b200_conv1d_bwd_workspace_bytes", [C.c_int] * 4, C.c_longlong)
        bind("mamba_b200_conv1d_bwd_static", [vp, vp, C.POINTER(Conv1dArgs)])
        bind("mamba_b200_conv1d_bwd_static_max_bytes", [], C.c_longlong)
        ll, fl, it = C.c_longlong, C.c_float, C.c_int
        bind("mamba_b200_residual_rmsnorm_fwd", [vp, vp, it, vp, vp, vp, vp, vp, it, it, fl])
        bind("mamba_b200_residual_rmsnorm_bwd_workspace_bytes", [it, it], ll)
        bind("mamba_b200_residual_rmsnorm_bwd", [vp, vp, it, vp, vp, vp, vp, vp, vp, it, it, vp, ll])
        bind("mamba_b200_embedding_gather", [vp, vp, it, vp, vp, vp, ll, it, it])
        bind("mamba_b200_softmax_xent", [vp, vp, it, vp, vp, vp, vp, fl, ll, it, ll])
        bind("mamba_b200_adamw_step", [vp, vp, vp, vp, vp, vp, fl, fl, fl, fl, fl, vp, vp, it, ll])
        bind("mamba_b200_m3_ssd_fwd", [vp, vp, C.POINTER(M3SsdArgs)])
        bind("mamba_b200_m3_ssd_bwd", [vp, vp, C.POINTER(M3SsdBwdArgs)])
        bind("mamba_b200_m3_ssd_bwd_workspace_bytes", [C.c_int] * 5, C.c_longlong)
        bind("mamba_b200_m3_ssd_bwd_workspace_bytes_for", [C.c_int] * 6, C.c_longlong)
    return _lib


class Handle:
    """Per-device library handle (mamba_b200_init / mamba_b200_destroy)."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        self.device = device
        rc = lib().mamba_b200_init(device, C.byref(self._h))
        if rc != 0:
            msg = lib().mamba_b200_last_error(self._h).decode() if self._h else "no handle"
            if self._h:
                lib().mamba_b200_destroy(self._h)
                self._h = C.c_void_p()
            raise RuntimeError(f"mamba_b200_init({device}) failed ({rc}): {msg}")

    @property
    def ptr(self):
        return self._h

    def check(self, rc: int, what: str):
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc}): {lib().mamba_b200_last_error(self._h).decode()}")

    def check_status(self, stream=None):
        self.check(lib().mamba_b200_check_status(self._h, C.c_void_p(stream or 0)), "check_status")

    def close(self):
        if self._h:
            lib().mamba_b200_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_handles = {}


def default_handle(device: int) -> Handle:
    if device not in _handles:
        _handles[device] = Handle(device)
    return _handles[device]
