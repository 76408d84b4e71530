"""Regenerates tests/golden/m1_fused_*.npz from the CPU oracle.

Run from the repository root:  python tests/golden/gen_golden.py
Inputs are seeded (mamba_rs_b200.synth) and rounded to the storage dtype; the
fixture stores the oracle's outputs for them, so a test can check both that the
oracle still produces these numbers and that the CUDA path matches them."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from helpers import GOLDEN_CASES as CASES, quantised_inputs, random_states  # noqa: E402

def main():
    out_dir = os.path.dirname(os.path.abspath(__file__))
    for name, B, T, D, N, K, dt, a_mode, seed in CASES:
        q = quantised_inputs(B, T, D, N, K, dt, seed, a_mode)
        ssm0, cst0 = random_states(B, D, N, K, seed + 100)
        fwd = oracle.m1_fused_fwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q["z"], q["a_neg"],
                                  q["Dp"], q.get("conv_w"), q.get("conv_b"), cst0, ssm0)
        rng = np.random.default_rng(seed + 200)
        dg = rng.standard_normal((B, T, D)).astype(np.float32)
        bwd = oracle.m1_fused_bwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q["z"], q["a_neg"],
                                  q["Dp"], dg, q.get("conv_w"), q.get("conv_b"), cst0, ssm0)
        arrs = dict(meta=np.array([B, T, D, N, K, seed]), y=fwd["y"], ssm_state=fwd["ssm_state"],
                    dg=dg, d_x=bwd["d_x"], d_delta=bwd["d_delta"], d_z=bwd["d_z"], dB=bwd["dB"],
                    dC=bwd["dC"], dA_log=bwd["dA_log"], dD=bwd["dD"])
        if K:
            arrs.update(conv_state=fwd["conv_state"], dconv_w=bwd["dconv_w"], dconv_b=bwd["dconv_b"])
        np.savez_compressed(os.path.join(out_dir, f"m1_fused_{name}.npz"), **arrs)
        print(name, {k: v.shape for k, v in arrs.items()})


if __name__ == "__main__":
    main()
