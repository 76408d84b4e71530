"""Launches the reference's own CUDA kernels (cubins built by build_ref.py) on
torch tensors, with the grids and shared-memory sizes of the reference's launch
helpers (src/mamba_ssm/gpu/launch.rs:57-201).  Test / benchmark infrastructure:
a second, independent checker of the oracle and the "reference kernel on
sm_100a" timing arm.  Uses the CUDA driver API through cuda-python."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
SUFFIX = {"f32": "f32", "bf16": "bf16", "f16": "f16"}


def available() -> bool:
    return os.path.exists(os.path.join(_REF, "mamba_ssm_parallel.cubin"))


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
        err, = self.drv.cuLaunchKernel(fn, grid[0], grid[1], grid[2], block, 1, 1, smem, stream,
                                       (tuple(vals), tuple(types)), 0)
        assert err == self.drv.CUresult.CUDA_SUCCESS, err

    # ssm_parallel_scan_fwd_nosave[_{bf16,f16}]  (kernels/mamba_ssm_parallel.cu:544-553, :969-980)
    def ssm_parallel_scan_fwd_nosave(self, dt, h, y, delta, u, Bm, Cm, a_neg, Dp):
        Bsz, T, D = delta.shape
        N = a_neg.shape[1]
        name = "ssm_parallel_scan_fwd_nosave" + ("" if dt == "f32" else "_" + SUFFIX[dt])
        fixed = (2 * 4 + 2 * 256 + 2 * 128) * 4
        smem = fixed + 1024 * (4 if dt == "f32" else 2)  # launch.rs:116-131, :178-201
        self._launch(self._func("mamba_ssm_parallel", name), (Bsz, D, 1), 128, smem,
                     [h, y, delta, u, Bm, Cm, a_neg, Dp, Bsz, T, D, N])

    # ssm_burnin_forward_nosave[_{dt}]  (kernels/mamba_ssm.cu:304-400), 1-D grid of 256 threads
    def ssm_burnin_forward_nosave(self, dt, h, y, delta, u, Bm, Cm, a_neg, Dp):
        Bsz, T, D = delta.shape
        N = a_neg.shape[1]
        name = "ssm_burnin_forward_nosave" + ("" if dt == "f32" else "_" + SUFFIX[dt])
        n = Bsz * D
        self._launch(self._func("mamba_ssm", name), ((n + 255) // 256, 1, 1), 256, 0,
                     [h, y, delta, u, Bm, Cm, a_neg, Dp, Bsz, T, D, N])

    # conv1d_burnin_forward_nosave_{dt}  (kernels/conv1d.cu:284-315)
    def conv1d_burnin_forward_nosave(self, dt, u_out, state, x, w, b):
        Bsz, T, D = x.shape
        K = w.shape[1]
        name = "conv1d_burnin_forward_nosave_" + SUFFIX[dt]
        n = Bsz * D
        self._launch(self._func("conv1d", name), ((n + 255) // 256, 1, 1), 256, 0,
                     [u_out, state, x, w, b, Bsz, T, D, K])
