"""Times one operator of the library on one GPU and prints one JSON line.

    python -m mamba_rs_b200.measure --op sscan_bwd [--batch 16] [--steps 10] [--warmup 3]

Operators and their default shapes (seeded synthetic inputs, bf16 storage):
  sscan_fwd, sscan_fwd_unfused, sscan_bwd, conv1d_fwd, conv1d_bwd, sscan_step
      Mamba-1, d_inner 1536, d_state 16, L 2048, d_conv 4 (batch 16; step: batch 8)
  m3_ssd_fwd, m3_ssd_bwd
      Mamba-3 SISO, 32 heads x headdim 64, d_state 128, L 4096 (batch 8)
The line gives the mean kernel time over --steps launches (CUDA events on the
launching stream, after --warmup launches), the algorithmic bytes of one launch
and their ratio to the measured HBM copy peak.  It is the command behind the
per-operator figures and the profiler captures; the headline benchmark is
bench.py at the repository root.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def hbm_peak():
    try:
        with open(os.path.join(HERE, "..", "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True,
                    choices=["sscan_fwd", "sscan_fwd_unfused", "sscan_bwd", "conv1d_fwd", "conv1d_bwd",
                             "sscan_step", "m3_ssd_fwd", "m3_ssd_bwd"])
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--save-stride", type=int, default=32)
    ap.add_argument("--a-mode", default="s4d", choices=["s4d", "random"])
    ap.add_argument("--heads", type=int, default=32, help="Mamba-3: number of heads")
    ap.add_argument("--headdim", type=int, default=64, help="Mamba-3: head dimension")
    ap.add_argument("--dstate", type=int, default=128, help="Mamba-3: state size")
    ap.add_argument("--sequential", action="store_true", help="Mamba-3 forward: the sequential kernel")
    args = ap.parse_args()

    import torch

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import synth

    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the library has no CPU fallback")
    dev = torch.device("cuda", 0)
    bf = torch.bfloat16
    t = lambda a, d=None: torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(d or torch.float32)
    e = 2
    cfg, by, fn = {}, 0, None

    if args.op.startswith("m3_"):
        B, T, nh, hd, N = args.batch or 8, 4096, args.heads, args.headdim, args.dstate
        i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=0)
        a = [t(i[k], bf if k in ("x", "K", "Q") else None) for k in ("x", "K", "Q", "dt", "trap", "adt", "Dh")]
        cfg = dict(B=B, T=T, nh=nh, hd=hd, N=N, storage="bf16")
        if args.op == "m3_ssd_fwd":
            y = torch.empty_like(a[0])
            ssm = torch.zeros(B, nh, hd, N, device=dev)
            by = synth.m3_fwd_algorithmic_bytes(B, T, nh, hd, N, e)
            fn = lambda: mb.m3_ssd_fwd(*a, ssm_state=ssm, y=y, force_sequential=args.sequential)
        else:
            dy = torch.randn(B, T, nh * hd, device=dev).to(bf)
            ws = torch.empty(mb.ffi.lib().mamba_b200_m3_ssd_bwd_workspace_bytes_for(2, B, T, nh, hd, N),
                             dtype=torch.uint8, device=dev)
            # x, K, Q, dy read; dx written; dK, dQ f32; five [B,T,nh] f32 vectors
            by = (3 * e * B * T * nh * hd + 2 * e * B * T * nh * N + 2 * 4 * B * T * nh * N + 6 * 4 * B * T * nh)
            fn = lambda: mb.m3_ssd_bwd(*a, dy, workspace=ws)
    else:
        B, T, D, N, K = args.batch or (8 if args.op == "sscan_step" else 16), 2048, 1536, 16, 4
        inp = synth.m1_scan_inputs(B, T, D, N, K, seed=0, a_mode=args.a_mode)
        x, dl, Bm, Cm, z = [t(inp[k], bf) for k in ("x", "delta_raw", "Bm", "Cm", "z")]
        a_neg, Dp, cw, cb = t(inp["a_neg"]), t(inp["Dp"]), t(inp["conv_w"]), t(inp["conv_b"])
        cfg = dict(B=B, T=T, D=D, N=N, storage="bf16", a_neg=args.a_mode)
        if args.op == "sscan_fwd":
            y = torch.empty_like(x)
            ssm = torch.zeros(B, D, N, device=dev)
            by = synth.m1_fwd_algorithmic_bytes(B, T, D, N, e)
            fn = lambda: mb.selective_scan_fwd(x, dl, Bm, Cm, a_neg, Dp, z, ssm_state=ssm, y=y)
        elif args.op == "sscan_fwd_unfused":
            y = torch.empty_like(x)
            ssm = torch.zeros(B, D, N, device=dev)
            dsp = torch.nn.functional.softplus(dl.float()).to(bf)
            by = synth.m1_fwd_algorithmic_bytes(B, T, D, N, e, z=False)
            fn = lambda: mb.ssm_parallel_scan_fwd_nosave(ssm, y, dsp, x, Bm, Cm, a_neg, Dp)
        elif args.op == "sscan_bwd":
            S = args.save_stride
            cfg["save_stride"] = S
            cs = torch.empty(B, (T + S - 1) // S, D, N, device=dev)
            mb.selective_scan_fwd(x, dl, Bm, Cm, a_neg, Dp, z, chunk_states=cs, save_stride=S)
            dy = torch.randn(B, T, D, device=dev).to(bf)
            ws = torch.empty(mb.selective_scan_bwd_workspace_bytes(B, T, D, N), dtype=torch.uint8, device=dev)
            by = 7 * e * B * T * D + 2 * e * B * T * N + 2 * 4 * B * T * N + 4 * B * ((T + S - 1) // S) * D * N
            fn = lambda: mb.selective_scan_bwd(x, dl, Bm, Cm, a_neg, Dp, dy, cs, S, z, workspace=ws)
        elif args.op == "conv1d_fwd":
            cfg["K"] = K
            u = torch.empty_like(x)
            by = 2 * e * B * T * D
            fn = lambda: mb.conv1d_fwd(x, cw, cb, None, u)
        elif args.op == "conv1d_bwd":
            cfg["K"] = K
            dy = torch.randn(B, T, D, device=dev).to(bf)
            ws = torch.empty(int(mb.ffi.lib().mamba_b200_conv1d_bwd_workspace_bytes(B, T, D, K)),
                             dtype=torch.uint8, device=dev)
            by = 3 * e * B * T * D
            fn = lambda: mb.conv1d_bwd(x, cw, cb, dy, None, workspace=ws)
        else:  # one decode step
            cfg.pop("T")
            cfg["K"] = K
            xs, ds, zs = [torch.randn(B, D, device=dev).to(bf) for _ in range(3)]
            bs, cs2 = [torch.randn(B, N, device=dev).to(bf) for _ in range(2)]
            ssm = torch.zeros(B, D, N, device=dev)
            cst = torch.zeros(B, D, K, device=dev)
            ys = torch.empty(B, D, device=dev, dtype=bf)
            by = 2 * 4 * B * D * N + 2 * 4 * B * D * K + 4 * e * B * D
            fn = lambda: mb.selective_scan_step(xs, ds, bs, cs2, a_neg, Dp, ssm, zs, conv_w=cw, conv_b=cb,
                                                conv_state=cst, y=ys)

    for _ in range(max(args.warmup, 1)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    mb.ffi.default_handle(0).check_status()
    ms = e0.elapsed_time(e1) / args.steps
    peak, src = hbm_peak()
    gbs = by / (ms * 1e-3) / 1e9
    print(json.dumps({"op": args.op, "config": cfg, "ms": ms, "steps": args.steps, "algorithmic_bytes": by,
                      "GBps": gbs, "hbm_peak_GBps": peak, "peak_source": src, "frac": gbs / peak,
                      "note": "time per call through the Python operator, including its launch overhead"}))


if __name__ == "__main__":
    main()
