"""Launches the reference's own CUDA kernels (cubins built by build_ref.py) on
torch tensors, with the grids and shared-memory sizes of the reference's launch
sites.  Test / benchmark infrastructure: a second, independent checker of the
oracle and the "reference kernel on sm_100a" timing arm.  Uses the CUDA driver
API through cuda-python.

Grids follow src/mamba_ssm/gpu/launch.rs:57-201 (Mamba-1 scan),
src/mamba_ssm/gpu/backward_mixed.rs:205-350 (backward + reducers),
src/mamba_ssm/gpu/forward_mixed.rs:500-537 / backward_mixed.rs:586-619 (conv1d),
src/mamba3_siso/gpu/forward.rs:258-455 and backward.rs:235-337 (Mamba-3)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
MODULES = ("mamba_ssm_parallel", "mamba_ssm", "conv1d", "mamba3_ssd", "mamba3_chunked", "mamba3_ops")


def available() -> bool:
    return all(os.path.exists(os.path.join(_REF, m + ".cubin")) for m in MODULES)


def _sfx(dt: str, bare_f32: bool) -> str:
    """Kernel-name suffix: the reference's legacy f32 kernels carry no suffix,
    its macro-generated ones carry _f32 / _bf16 / _f16."""
    return "" if (dt == "f32" and bare_f32) else "_" + dt


class RefKernels:
    def __init__(self):
        import torch
        from cuda.bindings import driver
        self.drv = driver
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make the primary context current
        self.mods = {}
        self.funcs = {}

    def _func(self, module: str, name: str):
        key = (module, name)
        if key not in self.funcs:
            if module not in self.mods:
                data = open(os.path.join(_REF, module + ".cubin"), "rb").read()
                err, mod = self.drv.cuModuleLoadData(data)
                assert err == self.drv.CUresult.CUDA_SUCCESS, err
                self.mods[module] = mod
            err, fn = self.drv.cuModuleGetFunction(self.mods[module], name.encode())
            assert err == self.drv.CUresult.CUDA_SUCCESS, (name, err)
            self.funcs[key] = fn
        return self.funcs[key]

    def _launch(self, fn, grid, block, smem, args):
        import torch
        vals, types = [], []
        for a in args:
            if isinstance(a, int):
                vals.append(a)
                types.append(C.c_int)
            else:  # tensor
                vals.append(a.data_ptr())
                types.append(C.c_void_p)
        stream = torch.cuda.current_stream().cuda_stream
        if smem > 48 * 1024:  # beyond the default limit a kernel has to opt in (m3_dqkv at hd 32, N 64)
            err, = self.drv.cuFuncSetAttribute(
                fn, self.drv.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem)
            assert err == self.drv.CUresult.CUDA_SUCCESS, err
        err, = self.drv.cuLaunchKernel(fn, grid[0], grid[1], grid[2], block, 1, 1, smem, stream,
                                       (tuple(vals), tuple(types)), 0)
        assert err == self.drv.CUresult.CUDA_SUCCESS, err

    @staticmethod
    def _grid_1d(n):
        return ((n + 255) // 256, 1, 1)

    # ------------------------------------------------------------------ Mamba-1 forward
    # ssm_parallel_scan_fwd_nosave[_{bf16,f16}]  (kernels/mamba_ssm_parallel.cu:544-553, :969-980)
    def ssm_parallel_scan_fwd_nosave(self, dt, h, y, delta, u, Bm, Cm, a_neg, Dp):
        Bsz, T, D = delta.shape
        N = a_neg.shape[1]
        name = "ssm_parallel_scan_fwd_nosave" + _sfx(dt, True)
        fixed = (2 * 4 + 2 * 256 + 2 * 128) * 4
        smem = fixed + 1024 * (4 if dt == "f32" else 2)  # launch.rs:116-131, :178-201
        self._launch(self._func("mamba_ssm_parallel", name), (Bsz, D, 1), 128, smem,
                     [h, y, delta, u, Bm, Cm, a_neg, Dp, Bsz, T, D, N])

    # ssm_parallel_scan_fwd[_{bf16,f16}] with h_saved [B,(T+1),D,N] f32
    # (kernels/mamba_ssm_parallel.cu:265-276, :777-790)
    def ssm_parallel_scan_fwd(self, dt, h, y, h_saved, delta, u, Bm, Cm, a_neg, Dp):
        Bsz, T, D = delta.shape
        N = a_neg.shape[1]
        name = "ssm_parallel_scan_fwd" + _sfx(dt, True)
        fixed = (2 * 4 + 2 * 256 + 2 * 128) * 4
        smem = fixed + 1024 * (4 if dt == "f32" else 2)
        self._launch(self._func("mamba_ssm_parallel", name), (Bsz, D, 1), 128, smem,
                     [h, y, h_saved, delta, u, Bm, Cm, a_neg, Dp, Bsz, T, D, N])

    # ssm_burnin_forward_nosave[_{dt}]  (kernels/mamba_ssm.cu:304-400), 1-D grid of 256 threads
    def ssm_burnin_forward_nosave(self, dt, h, y, delta, u, Bm, Cm, a_neg, Dp):
        Bsz, T, D = delta.shape
        N = a_neg.shape[1]
        name = "ssm_burnin_forward_nosave" + _sfx(dt, True)
        self._launch(self._func("mamba_ssm", name), self._grid_1d(Bsz * D), 256, 0,
                     [h, y, delta, u, Bm, Cm, a_neg, Dp, Bsz, T, D, N])

    # ssm_burnin_forward[_{dt}] with h_saved  (kernels/mamba_ssm.cu:232-299, :404-455)
    def ssm_burnin_forward(self, dt, h, y, h_saved, delta, u, Bm, Cm, a_neg, Dp):
        Bsz, T, D = delta.shape
        N = a_neg.shape[1]
        name = "ssm_burnin_forward" + _sfx(dt, True)
        self._launch(self._func("mamba_ssm", name), self._grid_1d(Bsz * D), 256, 0,
                     [h, y, h_saved, delta, u, Bm, Cm, a_neg, Dp, Bsz, T, D, N])

    # ------------------------------------------------------------------ Mamba-1 backward
    def _reduce_bwd(self, dt, dBl, dCl, dDl, dAl, Bsz, T, D, N):
        """ssm_reduce_d_{B,C}[_{bf16,f16}], ssm_reduce_d_D, ssm_reduce_d_a_log
        (kernels/mamba_ssm.cu:667-763; backward_mixed.rs:289-348): '+=' into
        zeroed f32 outputs."""
        import torch
        f32 = dict(dtype=torch.float32, device=dBl.device)
        dB, dC = torch.zeros(Bsz, T, N, **f32), torch.zeros(Bsz, T, N, **f32)
        dD, dA = torch.zeros(D, **f32), torch.zeros(D, N, **f32)
        sfx = _sfx(dt, True)
        self._launch(self._func("mamba_ssm", "ssm_reduce_d_B" + sfx), self._grid_1d(Bsz * T * N), 256, 0,
                     [dB, dBl, Bsz, T, D, N])
        self._launch(self._func("mamba_ssm", "ssm_reduce_d_C" + sfx), self._grid_1d(Bsz * T * N), 256, 0,
                     [dC, dCl, Bsz, T, D, N])
        self._launch(self._func("mamba_ssm", "ssm_reduce_d_D"), self._grid_1d(D), 256, 0, [dD, dDl, Bsz, D])
        self._launch(self._func("mamba_ssm", "ssm_reduce_d_a_log"), self._grid_1d(D * N), 256, 0,
                     [dA, dAl, Bsz, D, N])
        return dB, dC, dD, dA

    def ssm_scan_bwd(self, kind, dt, h_saved, delta, u, Bm, Cm, a_neg, Dp, dy):
        """The reference's scan backward + its four reducers.
        kind 'parallel': ssm_parallel_scan_bwd_{dt} (kernels/mamba_ssm_parallel.cu:1182-1532,
        grid (B, D), 128 threads, 11 328 B of shared memory, launch.rs:145-165);
        kind 'sequential': ssm_backward_local[_{dt}] (kernels/mamba_ssm.cu:466-662).
        Returns d_delta, d_u (storage dtype), dB, dC [B,T,N], dD [D], dA_log [D,N] f32."""
        import torch
        Bsz, T, D = delta.shape
        N = a_neg.shape[1]
        dev = delta.device
        d_delta, d_u = torch.zeros_like(delta), torch.zeros_like(u)
        dBl = torch.zeros(Bsz, T, D, N, dtype=delta.dtype, device=dev)
        dCl = torch.zeros(Bsz, T, D, N, dtype=delta.dtype, device=dev)
        dDl = torch.zeros(Bsz, D, dtype=torch.float32, device=dev)
        dAl = torch.zeros(Bsz, D, N, dtype=torch.float32, device=dev)
        args = [h_saved, delta, u, Bm, Cm, a_neg, Dp, dy, d_delta, d_u, dBl, dCl, dDl, dAl, Bsz, T, D, N]
        if kind == "parallel":
            smem = ((2 * 4 + 2 * 256 + 2 * 128 + 1024) + (2 * 4 + 3 * 256 + 2 * 128)) * 4
            self._launch(self._func("mamba_ssm_parallel", "ssm_parallel_scan_bwd_" + dt), (Bsz, D, 1), 128,
                         smem, args)
        else:
            self._launch(self._func("mamba_ssm", "ssm_backward_local" + _sfx(dt, True)),
                         self._grid_1d(Bsz * D), 256, 0, args)
        dB, dC, dD, dA = self._reduce_bwd(dt, dBl, dCl, dDl, dAl, Bsz, T, D, N)
        return dict(d_delta=d_delta, d_u=d_u, dB=dB, dC=dC, dD=dD, dA_log=dA)

    # ------------------------------------------------------------------ conv1d
    # conv1d_burnin_forward_nosave_{dt}  (kernels/conv1d.cu:284-315)
    def conv1d_burnin_forward_nosave(self, dt, u_out, state, x, w, b):
        Bsz, T, D = x.shape
        K = w.shape[1]
        self._launch(self._func("conv1d", "conv1d_burnin_forward_nosave_" + dt), self._grid_1d(Bsz * D), 256, 0,
                     [u_out, state, x, w, b, Bsz, T, D, K])

    def conv1d_fwd_bwd(self, dt, state, x, w, b, d_u):
        """conv1d_burnin_forward_{dt} (saving post_conv and conv_states,
        kernels/conv1d.cu:326-359) followed by conv1d_burnin_backward_{dt}
        (:459-515); the per-(sample, channel) dW / db partials are summed over
        the batch here as reduce_sum_axis0 does (backward_mixed.rs:620-658)."""
        import torch
        Bsz, T, D = x.shape
        K = w.shape[1]
        dev = x.device
        u = torch.empty_like(x)
        post = torch.empty_like(x)
        cstates = torch.empty(Bsz, T, D, K, dtype=torch.float32, device=dev)
        self._launch(self._func("conv1d", "conv1d_burnin_forward_" + dt), self._grid_1d(Bsz * D), 256, 0,
                     [u, state, cstates, post, x, w, b, Bsz, T, D, K])
        d_x = torch.empty_like(x)
        dWp = torch.empty(Bsz, D, K, dtype=torch.float32, device=dev)
        dbp = torch.empty(Bsz, D, dtype=torch.float32, device=dev)
        self._launch(self._func("conv1d", "conv1d_burnin_backward_" + dt), self._grid_1d(Bsz * D), 256, 0,
                     [d_x, dWp, dbp, d_u, post, cstates, w, Bsz, T, D, K])
        return dict(u=u, d_x=d_x, dconv_w=dWp.sum(0), dconv_b=dbp.sum(0))

    # ------------------------------------------------------------------ Mamba-3 sequential
    def m3_burnin_fwd(self, dt, ssm, kst, vst, x, K, Q, alpha, beta, gamma, Dh):
        """m3_burnin_fwd[_{bf16,f16}] (kernels/mamba3_ssd.cu:229-445), grid (B, nh),
        block hd (hd <= 32, N <= 64).  States are updated in place.  Returns y and
        the saves (h_saved in the reference's transposed layout)."""
        import torch
        Bsz, T, nh, N = K.shape
        hd = x.shape[2] // nh
        dev = x.device
        f32 = dict(dtype=torch.float32, device=dev)
        y = torch.empty_like(x)
        h_saved = torch.empty(Bsz, T + 1, N, nh * hd, **f32)
        kp = torch.empty(Bsz, T, nh, N, **f32)
        vp = torch.empty(Bsz, T, nh * hd, **f32)
        self._launch(self._func("mamba3_ssd", "m3_burnin_fwd" + _sfx(dt, True)), (Bsz, nh, 1), hd, 0,
                     [ssm, kst, vst, y, h_saved, kp, vp, x, K, Q, alpha, beta, gamma, Dh, Bsz, T, nh, hd, N])
        return dict(y=y, h_saved=h_saved, k_prev=kp, v_prev=vp)

    def m3_backward_seq(self, saves, x, K, Q, alpha, beta, gamma, Dh, dy):
        """m3_backward_seq (f32 only, kernels/mamba3_ssd.cu:576-788) + m3_reduce_d_D."""
        import torch
        Bsz, T, nh, N = K.shape
        hd = x.shape[2] // nh
        f32 = dict(dtype=torch.float32, device=x.device)
        dx = torch.zeros(Bsz, T, nh * hd, **f32)
        dK, dQ = torch.zeros(Bsz, T, nh, N, **f32), torch.zeros(Bsz, T, nh, N, **f32)
        da, db, dg = (torch.zeros(Bsz, T, nh, **f32) for _ in range(3))
        dDl = torch.zeros(Bsz, nh * hd, **f32)
        self._launch(self._func("mamba3_ssd", "m3_backward_seq"), (Bsz, nh, 1), hd, 0,
                     [saves["h_saved"], saves["k_prev"], saves["v_prev"], x, K, Q, alpha, beta, gamma, Dh, dy,
                      dx, dK, dQ, da, db, dg, dDl, Bsz, T, nh, hd, N])
        dD = torch.zeros(nh, **f32)
        self._launch(self._func("mamba3_ssd", "m3_reduce_d_D"), (nh, 1, 1), 32, 0, [dD, dDl, Bsz, nh, hd])
        return dict(dx=dx, dK=dK, dQ=dQ, d_alpha=da, d_beta=db, d_gamma=dg, dD=dD)

    # ------------------------------------------------------------------ Mamba-3 chunked
    def m3_chunked_fwd(self, dt, x, K, Q, dtv, trap, adt, Dh, CS=64):
        """The reference's chunked forward chain m3_preprocess_chunks -> m3_dA_cumsum ->
        m3_chunk_state_fwd -> m3_state_passing_fwd -> m3_chunk_scan_fwd
        (kernels/mamba3_chunked.cu:57-419, :1050-1242; forward.rs:258-385).
        Returns y, the final state and the intermediates the backward consumes."""
        import torch
        Bsz, T, nh, N = K.shape
        hd = x.shape[2] // nh
        nc = (T + CS - 1) // CS
        dev = x.device
        f32 = dict(dtype=torch.float32, device=dev)
        sfx = _sfx(dt, True)
        Ks = torch.empty_like(K)
        qk, scale, gam = (torch.empty(Bsz, T, nh, **f32) for _ in range(3))
        self._launch(self._func("mamba3_chunked", "m3_preprocess_chunks" + sfx), (Bsz * nc, nh, 1), CS, 0,
                     [Ks, qk, scale, gam, K, Q, dtv, trap, Bsz, T, nh, N, CS])
        dacs = torch.zeros(Bsz, nc, nh, CS, **f32)
        bx = min(nh, 256)
        self._launch(self._func("mamba3_chunked", "m3_dA_cumsum"), (Bsz, nc, (nh + bx - 1) // bx), bx, 0,
                     [dacs, adt, Bsz, T, nh, CS])
        states = torch.empty(Bsz, nc, nh, hd, N, **f32)
        self._launch(self._func("mamba3_chunked", "m3_chunk_state_fwd" + sfx), (Bsz * nc, nh, 1), hd, 0,
                     [states, x, Ks, dacs, Bsz, T, nh, hd, N, CS])
        final = torch.empty(Bsz, nh, hd, N, **f32)
        dim = hd * N
        bx2 = min(dim, 256)
        self._launch(self._func("mamba3_chunked", "m3_state_passing_fwd"), (Bsz, nh, (dim + bx2 - 1) // bx2),
                     bx2, 0, [states, final, dacs, Bsz, nc, nh, hd, N, CS, T])
        y = torch.empty_like(x)
        self._launch(self._func("mamba3_chunked", "m3_chunk_scan_fwd" + sfx), (Bsz * nc, nh, 1), hd, 0,
                     [y, x, Q, Ks, qk, dacs, states, Dh, Bsz, T, nh, hd, N, CS])
        return dict(y=y, final_state=final, K_scaled=Ks, qk_dot=qk, scale=scale, gamma=gam, dA_cumsum=dacs,
                    chunk_states=states)

    def m3_kq_from_groups(self, Bn, Cn, b_bias, c_bias, angles_raw, dtv, angle_state):
        """The reference's per-head K / Q chain in f32: bc_bias_add (x2) -> m3_angle_dt_fwd_seq ->
        rope_fwd (kernels/mamba3_ops.cu:279-310, :400-440, :575-640; launch sites
        src/mamba3_siso/gpu/forward.rs:170-255).  Bn, Cn [B,T,ng,N], biases [nh,N], angles_raw
        [B,T,n_angles], dtv [B,T,nh], angle_state [B,nh,n_angles] (updated in place).
        Returns K, Q [B,T,nh,N] and the per-step angles [B,T,nh,n_angles]."""
        import torch
        Bsz, T, ng, N = Bn.shape
        nh = b_bias.shape[0]
        na = angles_raw.shape[2]
        f32 = dict(dtype=torch.float32, device=Bn.device)
        rows = Bsz * T
        Kb, Qb = torch.empty(Bsz, T, nh, N, **f32), torch.empty(Bsz, T, nh, N, **f32)
        fn = self._func("mamba3_ops", "bc_bias_add")
        self._launch(fn, self._grid_1d(rows * nh * N), 256, 0, [Kb, Bn, b_bias, rows, nh, ng, N])
        self._launch(fn, self._grid_1d(rows * nh * N), 256, 0, [Qb, Cn, c_bias, rows, nh, ng, N])
        cum = torch.empty(Bsz, T, nh, na, **f32)
        self._launch(self._func("mamba3_ops", "m3_angle_dt_fwd_seq"), (Bsz, (nh * na + 255) // 256, 1), 256, 0,
                     [cum, angle_state, angles_raw, dtv, Bsz, T, nh, na])
        K, Q = torch.empty_like(Kb), torch.empty_like(Qb)
        self._launch(self._func("mamba3_ops", "rope_fwd"), self._grid_1d(rows * nh * N), 256, 0,
                     [K, Q, Kb, Qb, cum, rows, nh, N, na])
        return K, Q, cum

    def m3_dqkv(self, dt, fw, x, Q, Dh, dy, CS=64):
        """m3_extract_da_cs_sum + m3_dqkv[_{bf16,f16}] (kernels/mamba3_chunked.cu:439-794,
        :1280-1527; backward.rs:266-337) on the intermediates of m3_chunked_fwd."""
        import torch
        Bsz, T, nh, N = Q.shape
        hd = x.shape[2] // nh
        nc = (T + CS - 1) // CS
        f32 = dict(dtype=torch.float32, device=x.device)
        dasum = torch.empty(Bsz, nc, nh, **f32)
        bx = min(nh, 256)
        self._launch(self._func("mamba3_chunked", "m3_extract_da_cs_sum"), (Bsz, nc, (nh + bx - 1) // bx), bx, 0,
                     [dasum, fw["dA_cumsum"], Bsz, T, nh, CS])
        dQm, dKm = torch.zeros(Bsz, T, nh, N, **f32), torch.zeros(Bsz, T, nh, N, **f32)
        dV = torch.zeros(Bsz, T, nh * hd, **f32)
        dADT, dQK = torch.zeros(Bsz, T, nh, **f32), torch.zeros(Bsz, T, nh, **f32)
        dDp = torch.zeros(Bsz, nh, **f32)
        smem = (2 * CS * N + 2 * CS * hd + 2 * CS + hd * N) * 4
        self._launch(self._func("mamba3_chunked", "m3_dqkv" + _sfx(dt, True)), (nh, Bsz, 1), hd, smem,
                     [dQm, dKm, dV, dADT, dQK, dDp, Q, fw["K_scaled"], x, fw["dA_cumsum"], dasum, fw["qk_dot"],
                      fw["chunk_states"], dy, Dh, Bsz, T, nh, hd, N, CS])
        return dict(dQ_mid=dQm, dK_mid=dKm, dV=dV, dADT=dADT, dQK_dot=dQK, dD=dDp.sum(0))

    def m3_dqk_tail(self, dt, fw, g, K, Q, dtv, trap, CS=64):
        """m3_dqktheta[_{bf16,f16}] with n_angles = 0 (RoPE is then the identity, so the
        'raw' Q / K are the scan's own inputs) followed by m3_ddt_dtrap
        (kernels/mamba3_chunked.cu:801-982, :1531-1640; backward.rs:372-443): turns the
        m3_dqkv outputs into dQ, dK, d(dt) and d(trap before its sigmoid)."""
        import torch
        Bsz, T, nh, N = Q.shape
        nc = (T + CS - 1) // CS
        f32 = dict(dtype=torch.float32, device=Q.device)
        dQ, dK = torch.zeros(Bsz, T, nh, N, **f32), torch.zeros(Bsz, T, nh, N, **f32)
        dang = torch.zeros(max(Bsz * T * nh, 1), **f32)
        dscale, dgamma = torch.zeros(Bsz, T, nh, **f32), torch.zeros(Bsz, T, nh, **f32)
        ang = torch.zeros(max(Bsz * T * nh, 1), **f32)
        self._launch(self._func("mamba3_chunked", "m3_dqktheta" + _sfx(dt, True)), (Bsz * nc, nh, 1), CS, 0,
                     [dQ, dK, dang, dscale, dgamma, Q, K, fw["scale"], fw["gamma"], ang, g["dQ_mid"], g["dK_mid"],
                      g["dQK_dot"], Bsz, T, nh, N, 0, CS])
        d_dt, d_trap_raw = torch.zeros(Bsz, T, nh, **f32), torch.zeros(Bsz, T, nh, **f32)
        self._launch(self._func("mamba3_chunked", "m3_ddt_dtrap"), self._grid_1d(Bsz * T * nh), 256, 0,
                     [d_dt, d_trap_raw, dscale, dgamma, dtv, trap, Bsz, T, nh])
        return dict(dQ=dQ, dK=dK, d_dt=d_dt, d_trap_raw=d_trap_raw)
