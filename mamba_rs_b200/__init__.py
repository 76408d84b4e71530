"""mamba_rs_b200 — host-side mirror of the mamba-rs kernel-launch boundary for the
selective-scan hot path, over the C ABI of ``libmamba_b200.so``.

The product path is the sm_100a library: importing works anywhere (so the CPU
test-suite can check symbols), but every compute call raises if the library or
a CUDA device is missing — there is no CPU or eager fallback.
"""
from __future__ import annotations

from . import ffi  # noqa: F401
from .ffi import Handle, LibraryMissing, lib, lib_path  # noqa: F401
from .ops import *  # noqa: F401,F403
from .parallel import BucketedGradReducer, allreduce_grads, shard_batch  # noqa: F401,E402
from .model import GpuMambaBackbone, GpuMambaLM, MambaConfig, MambaLMTrainer, MambaWeights  # noqa: F401,E402
