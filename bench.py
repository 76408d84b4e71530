#!/usr/bin/env python
"""Benchmark of the selective-scan hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --op NAME [--batch B] ...      one operator, one JSON line

A step is one pass of the fused Mamba-1 selective-scan forward over one batch
of synthetic input at the standalone-op configuration (batch 16 per GPU,
d_inner 1536, d_state 16, L 2048, bf16 storage / f32 compute).  Batches shard
by whole sequences, so with N ranks every rank runs the same per-GPU workload
on its own sequences (weak scaling) and there is no collective on the data
path.  Rank 0 prints one JSON line.

  value   : algorithmic GB/s of the whole job with inputs resident in HBM
  e2e     : the same metric through the public operator with host buffers:
            pinned host -> device copy of every step's inputs, kernel, device ->
            host copy of every step's result, all inside the timed region (steps
            pipelined over three streams and two device buffer sets)
  roofline: achieved algorithmic GB/s of the dominant kernel (CUDA events on
            the launching stream) against the measured HBM copy peak
  cpu_baseline: the CPU restatement of the reference's CPU path timed on the
            host cores of this box on a bounded sample of the same workload
  extra   : (1 GPU) every other operator of the path, timed after the headline
            region with CUDA events: scan forward with a trained-like a_neg,
            scan backward, conv1d forward / backward, the Mamba-3 SSD forward /
            backward, the decode loop (24 layers x 128 steps), small-batch
            prefill with time segments
            (N GPUs) the one collective of the design: the bucketed gradient
            all-reduce, alone and overlapped with the scan backward

--impl reference times the reference's CPU algorithm alone (the reference is
Rust and cannot be built without cargo; its algorithm is restated in oracle/),
on every host core, whatever thread count the launcher exported.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(B=16, T=2048, D=1536, N=16, dtype="bf16")
METRIC = "selective_scan_fwd_algorithmic_GBps"
FALLBACK_HBM_GBS = 6650.0
OPS = ["sscan_fwd", "sscan_fwd_random_a", "sscan_fwd_unfused", "sscan_fwd_small_batch", "sscan_bwd", "conv1d_fwd",
       "conv1d_bwd", "sscan_step", "decode_loop", "m3_ssd_fwd", "m3_ssd_fwd_fused_kq", "m3_ssd_bwd", "residual_rmsnorm_fwd",
       "residual_rmsnorm_bwd", "softmax_xent", "adamw_step", "embedding_gather"]


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def workload_name():
    w = WORKLOAD
    return (f"mamba1_selective_scan_fwd B={w['B']}/gpu D={w['D']} N={w['N']} L={w['T']} {w['dtype']} "
            "storage, softplus(delta) + SiLU(z) gate + D skip fused")


def config_block(world):
    """The `config` object both arms print (same keys, same values for the same launch)."""
    w = WORKLOAD
    by = algorithmic_bytes(w)
    return {"workload": workload_name(), "storage_dtype": "bf16", "accum_dtype": "f32",
            "global_batch": world * w["B"], "seq_len": w["T"],
            "parallelism": f"batch-sharded x{world}, no collective on the scan",
            "l2": (f"inputs+outputs per step ({by / 1e6:.0f} MB) exceed the 126 MB L2" if by > 126e6 else
                   f"inputs+outputs per step ({by / 1e6:.0f} MB) fit the 126 MB L2: not a valid bench size"),
            "a_neg": "S4D-real -(n+1) (the reference's init): arithmetic-progression decay path"}


def algorithmic_bytes(w):
    from mamba_rs_b200 import synth
    return synth.m1_fwd_algorithmic_bytes(w["B"], w["T"], w["D"], w["N"], 2, K=0, z=True)


def host_threads():
    """Every core this process may run on, whatever OMP_NUM_THREADS the launcher set."""
    try:
        os.sched_setaffinity(0, range(os.cpu_count() or 1))  # torchrun may have narrowed it
    except Exception:
        pass
    import oracle
    return oracle.set_num_threads()


def cpu_scan_leg(sample_B, sample_D, repeats=5):
    """Times the oracle's fused forward (the reference's CPU algorithm, OpenMP over
    samples x 8-channel blocks as PrefillMode::Parallel does) on `sample_B` sequences
    x `sample_D` channels of the workload, full length.  Returns (GB/s, seconds)."""
    import oracle
    from mamba_rs_b200 import synth
    w = WORKLOAD
    inp = synth.m1_scan_inputs(sample_B, w["T"], sample_D, w["N"], 0, seed=0, a_mode="s4d")
    q = {k: synth.round_to(v, "bf16") if k in ("x", "z", "delta_raw", "Bm", "Cm") else v
         for k, v in inp.items()}
    best = None
    for _ in range(repeats + 1):  # first pass is the warm-up
        t0 = time.perf_counter()
        oracle.m1_fused_fwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q["z"], q["a_neg"], q["Dp"])
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    by = synth.m1_fwd_algorithmic_bytes(sample_B, w["T"], sample_D, w["N"], 2, K=0, z=True)
    return by / best / 1e9, best


def cpu_prefill_leg(repeats=3):
    """The named CPU baseline: backbone forward_prefill of the reference's small model
    (d_model 128, 2 layers, d_inner 256, d_state 16, d_conv 4, dt_rank 8; batch 4 x 512,
    weights seed 42, inputs N(0,1) seed 7), restated with its scalar-order GEMM, one
    OpenMP task per sample.  Returns tokens/s and seconds per pass."""
    import oracle
    cfg = oracle.m1_config(d_model=128, n_layers=2, d_state=16, d_conv=4, expand=2, dt_rank=8, input_dim=128)
    w = oracle.m1_weights_init(cfg, 42)
    inp = np.random.default_rng(7).standard_normal((4, 512, 128)).astype(np.float32)
    best = None
    for _ in range(repeats + 1):
        t0 = time.perf_counter()
        r = oracle.m1_prefill_batch(cfg, w, inp)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return 4 * 512 / best, best, int(r["threads"])


def run_reference(args):
    """Reference arm: the reference's own CPU algorithm for the path (restated in
    oracle/, all host threads), each step the full workload of one GPU."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    cores = host_threads()
    import oracle
    from mamba_rs_b200 import synth
    w = WORKLOAD
    inp = synth.m1_scan_inputs(w["B"], w["T"], w["D"], w["N"], 0, seed=0, a_mode="s4d")
    q = {k: synth.round_to(v, "bf16") if k in ("x", "z", "delta_raw", "Bm", "Cm") else v
         for k, v in inp.items()}
    call = lambda: oracle.m1_fused_fwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q["z"], q["a_neg"], q["Dp"])
    for _ in range(args.warmup):
        call()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        call()
    dt = (time.perf_counter() - t0) / args.steps
    by = algorithmic_bytes(w)
    val = by / dt / 1e9
    sample = (f"one GPU's workload per step ({w['B']} sequences x {w['D']} channels x L={w['T']}); the CPU "
              "runs one such shard whatever the number of GPUs")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "storage_dtype": "bf16", "data": "synthetic",
        "config": config_block(world),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                         "note": "the reference's Rust build is unavailable on this box (no cargo); this is "
                                 "its CPU algorithm restated in C"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------------
# one operator at a time (also the `extra` block of the headline line)
# --------------------------------------------------------------------------------------

def time_call(fn, steps, warmup):
    import torch
    for _ in range(max(warmup, 1)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def op_case(name, dev, batch=0, save_stride=32, heads=32, headdim=64, dstate=128, sequential=False):
    """Builds one operator's seeded inputs on `dev`.  Returns (callable, algorithmic bytes of
    one call, config dict)."""
    import torch

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import synth
    bf = torch.bfloat16
    t = lambda a, d=None: torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(d or torch.float32)
    e = 2
    if name.startswith("m3_"):
        B, T, nh, hd, N = batch or 8, 4096, heads, headdim, dstate
        i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=0)
        a = [t(i[k], bf if k in ("x", "K", "Q") else None) for k in ("x", "K", "Q", "dt", "trap", "adt", "Dh")]
        cfg = dict(B=B, T=T, nh=nh, hd=hd, N=N, storage="bf16")
        if name == "m3_ssd_fwd_fused_kq":
            ng, na = 1, N // 4  # one group, rope_fraction 0.5 (the reference's default)
            g = synth.m3_group_inputs(B, T, nh, ng, N, na, i["dt"], seed=0)
            y = torch.empty_like(a[0])
            ssm = torch.zeros(B, nh, hd, N, device=dev)
            ang = t(g["angle_state"])
            ga = [t(g["Bn"], bf), t(g["Cn"], bf), t(g["b_bias"]), t(g["c_bias"]), t(g["angle_vel"])]
            cfg.update(ngroups=ng, n_angles=na)
            by = synth.m3_fused_kq_algorithmic_bytes(B, T, nh, ng, hd, N, na, e)
            return (lambda: mb.m3_ssd_fwd_fused_kq(a[0], *ga, a[3], a[4], a[5], a[6], angle_state=ang,
                                                   ssm_state=ssm, y=y)), by, cfg
        if name == "m3_ssd_fwd":
            y = torch.empty_like(a[0])
            ssm = torch.zeros(B, nh, hd, N, device=dev)
            by = synth.m3_fwd_algorithmic_bytes(B, T, nh, hd, N, e)
            return (lambda: mb.m3_ssd_fwd(*a, ssm_state=ssm, y=y, force_sequential=sequential)), by, cfg
        dy = torch.randn(B, T, nh * hd, device=dev).to(bf)
        ws = torch.empty(mb.ffi.lib().mamba_b200_m3_ssd_bwd_workspace_bytes_for(2, B, T, nh, hd, N),
                         dtype=torch.uint8, device=dev)
        # x, K, Q, dy read; dx written; dK, dQ f32; five [B,T,nh] f32 vectors
        by = (3 * e * B * T * nh * hd + 2 * e * B * T * nh * N + 2 * 4 * B * T * nh * N + 6 * 4 * B * T * nh)
        return (lambda: mb.m3_ssd_bwd(*a, dy, workspace=ws)), by, cfg

    if name in ("residual_rmsnorm_fwd", "residual_rmsnorm_bwd", "embedding_gather"):
        rows, dim = (batch or 8) * 8192, 2560  # the 2.8b layer shape: one GPU's shard of tokens
        cfg = dict(rows=rows, dim=dim, storage="bf16")
        scale = torch.ones(dim, device=dev)
        res = torch.randn(rows, dim, device=dev)
        if name == "embedding_gather":
            V = 50280
            table = torch.randn(V, dim, device=dev).to(bf)
            ids = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
            cfg["vocab"] = V
            return (lambda: mb.embedding_gather(table, ids, res)), rows * dim * (e + 4) + 4 * rows, cfg
        if name == "residual_rmsnorm_fwd":
            br = torch.randn(rows, dim, device=dev).to(bf)
            y, rms = torch.empty_like(br), torch.empty(rows, device=dev)
            return (lambda: mb.residual_rmsnorm_fwd(res, br, scale, y=y, rms_out=rms)), rows * dim * 2 * (4 + e), cfg
        dy = torch.randn(rows, dim, device=dev).to(bf)
        rms = res.pow(2).mean(1).add(1e-5).sqrt()
        dres, dsc = torch.zeros(rows, dim, device=dev), torch.zeros(dim, device=dev)
        ws = torch.empty(int(mb.ffi.lib().mamba_b200_residual_rmsnorm_bwd_workspace_bytes(rows, dim)), dtype=torch.uint8,
                         device=dev)
        return (lambda: mb.residual_rmsnorm_bwd(dy, res, scale, rms, dres, dsc, workspace=ws)), rows * dim * (e + 12), cfg
    if name == "softmax_xent":
        rows, V = (batch or 1) * 8192, 50280
        lg = (3.0 * torch.randn(rows, V, device=dev)).to(bf)
        tg = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
        dlg = torch.empty_like(lg)
        cfg = dict(rows=rows, vocab=V, storage="bf16")
        return (lambda: mb.softmax_xent(lg, tg, dlogits=dlg)), rows * V * 2 * e + 8 * rows, cfg
    if name == "adamw_step":
        n = 100_000_000
        pa, g, m, v = (torch.randn(n, device=dev) for _ in range(4))
        v.abs_()
        lp = torch.empty(n, device=dev, dtype=bf)
        bcf = torch.tensor([1.1, 1.2], device=dev)
        cfg = dict(params=n, compute_copy="bf16")
        return (lambda: mb.adamw_step(pa, g, m, v, bcf, lr=1e-4, weight_decay=0.1, param_lp=lp)), n * (16 + 12 + e), cfg

    small = name == "sscan_fwd_small_batch"
    B = batch or (8 if name in ("sscan_step", "decode_loop") else (1 if small else 16))
    T, D, N, K = (8192 if small else 2048), 1536, 16, 4
    a_mode = "random" if name == "sscan_fwd_random_a" else "s4d"
    inp = synth.m1_scan_inputs(B, 2 if name in ("sscan_step", "decode_loop") else T, D, N, K, seed=0, a_mode=a_mode)
    a_neg, Dp, cw, cb = t(inp["a_neg"]), t(inp["Dp"]), t(inp["conv_w"]), t(inp["conv_b"])
    cfg = dict(B=B, T=T, D=D, N=N, storage="bf16", a_neg=a_mode)
    if name in ("sscan_step", "decode_loop"):
        cfg.pop("T")
        cfg["K"] = K
        L = 24 if name == "decode_loop" else 1
        STEPS = 128 if name == "decode_loop" else 1
        cfg.update(layers=L, steps=STEPS)
        xs, ds, zs = [torch.randn(B, D, device=dev).to(bf) for _ in range(3)]
        bs, cs2 = [torch.randn(B, N, device=dev).to(bf) for _ in range(2)]
        ssm = [torch.zeros(B, D, N, device=dev) for _ in range(L)]
        cst = [torch.zeros(B, D, K, device=dev) for _ in range(L)]
        ys = torch.empty(B, D, device=dev, dtype=bf)
        by = L * STEPS * (2 * 4 * B * D * N + 2 * 4 * B * D * K + 4 * e * B * D)

        def loop():
            for _ in range(STEPS):
                for l in range(L):
                    mb.selective_scan_step(xs, ds, bs, cs2, a_neg, Dp, ssm[l], zs, conv_w=cw, conv_b=cb,
                                           conv_state=cst[l], y=ys)
        if name == "sscan_step":
            return loop, by, cfg
        # the decode loop is launch-bound: capture the 24 x 128 launches once, replay the graph
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            loop()  # every first call (handle set-up) happens before the capture
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loop()
        cfg["cuda_graph"] = True
        cfg["tokens"] = B * STEPS
        return graph.replay, by, cfg

    x, dl, Bm, Cm, z = [t(inp[k], bf) for k in ("x", "delta_raw", "Bm", "Cm", "z")]
    if name in ("sscan_fwd", "sscan_fwd_random_a", "sscan_fwd_small_batch"):
        y = torch.empty_like(x)
        ssm = torch.zeros(B, D, N, device=dev)
        ws = None
        if small:
            ws = torch.empty(mb.selective_scan_fwd_workspace_bytes(B, T, D, N), dtype=torch.uint8, device=dev)
            cfg["time_segments"] = "exact carry, workspace lent"
        by = synth.m1_fwd_algorithmic_bytes(B, T, D, N, e)
        return (lambda: mb.selective_scan_fwd(x, dl, Bm, Cm, a_neg, Dp, z, ssm_state=ssm, y=y, workspace=ws)), by, cfg
    if name == "sscan_fwd_unfused":
        y = torch.empty_like(x)
        ssm = torch.zeros(B, D, N, device=dev)
        dsp = torch.nn.functional.softplus(dl.float()).to(bf)
        by = synth.m1_fwd_algorithmic_bytes(B, T, D, N, e, z=False)
        return (lambda: mb.ssm_parallel_scan_fwd_nosave(ssm, y, dsp, x, Bm, Cm, a_neg, Dp)), by, cfg
    if name == "sscan_bwd":
        S = save_stride
        cfg["save_stride"] = S
        cs = torch.empty(B, (T + S - 1) // S, D, N, device=dev)
        mb.selective_scan_fwd(x, dl, Bm, Cm, a_neg, Dp, z, chunk_states=cs, save_stride=S)
        dy = torch.randn(B, T, D, device=dev).to(bf)
        ws = torch.empty(mb.selective_scan_bwd_workspace_bytes(B, T, D, N), dtype=torch.uint8, device=dev)
        by = 7 * e * B * T * D + 2 * e * B * T * N + 2 * 4 * B * T * N + 4 * B * ((T + S - 1) // S) * D * N
        return (lambda: mb.selective_scan_bwd(x, dl, Bm, Cm, a_neg, Dp, dy, cs, S, z, workspace=ws)), by, cfg
    cfg["K"] = K
    if name == "conv1d_fwd":
        u = torch.empty_like(x)
        return (lambda: mb.conv1d_fwd(x, cw, cb, None, u)), 2 * e * B * T * D, cfg
    if name == "conv1d_bwd":
        dy = torch.randn(B, T, D, device=dev).to(bf)
        ws = torch.empty(int(mb.ffi.lib().mamba_b200_conv1d_bwd_workspace_bytes(B, T, D, K)), dtype=torch.uint8,
                         device=dev)
        return (lambda: mb.conv1d_bwd(x, cw, cb, dy, None, workspace=ws)), 3 * e * B * T * D, cfg
    raise ValueError(name)


def measure_op(name, dev, steps=10, warmup=3, **kw):
    import torch

    import mamba_rs_b200 as mb
    fn, by, cfg = op_case(name, dev, **kw)
    ms = time_call(fn, steps, warmup)
    mb.ffi.default_handle(dev.index or 0).check_status()
    peak, src = measured_peaks()
    gbs = by / (ms * 1e-3) / 1e9
    out = {"op": name, "config": cfg, "ms": ms, "steps": steps, "algorithmic_bytes": by, "GBps": gbs,
           "frac_of_hbm_peak": gbs / peak, "peak_source": src}
    if "tokens" in cfg:
        out["tokens_per_s"] = cfg["tokens"] / (ms * 1e-3)
    del fn
    torch.cuda.empty_cache()
    return out


def run_op(args):
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the library has no CPU fallback")
    dev = torch.device("cuda", 0)
    out = measure_op(args.op, dev, steps=args.steps if args.steps != 100 else 10, warmup=max(args.warmup, 3),
                     batch=args.batch, save_stride=args.save_stride, heads=args.heads, headdim=args.headdim,
                     dstate=args.dstate, sequential=args.sequential)
    out["note"] = "time per call through the Python operator, including its launch overhead"
    print(json.dumps(out))


def lm_extra(dev, world, rank):
    """Model-level figures through the host-side engines (library GEMMs between this
    library's kernels), per rank on its own sequences, max over ranks:
      * 130m architecture (d_model 768, 24 layers, vocab 50280, tied head), random init,
        bf16: prefill of 8 x 2048 token ids, then 128 greedy decode steps (CUDA graph);
      * 2.8b layer shape (d_model 2560, d_inner 5120, dt_rank 160, vocab 50280), bf16
        compute / f32 master, 4 of its 64 layers, 2 x 8192 tokens per micro-batch: one
        training step (forward, cross-entropy, backward, bucketed all-reduce under the
        backward when N > 1, AdamW)."""
    import torch
    import torch.distributed as dist

    import mamba_rs_b200 as mb

    def tmax(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    out = {}
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    # ---- 130m: prefill + decode ----
    cfg = mb.MambaConfig(d_model=768, n_layers=24)
    V, B, T, steps = 50280, 8, 2048, 128
    w = mb.MambaWeights(cfg, dev, dtype=torch.bfloat16, vocab=V).init_random(0)
    ids = torch.randint(0, V, (B, T), device=dev, dtype=torch.int32, generator=g)
    lm = mb.GpuMambaLM(w, B)

    def prefill():
        lm.backbone.reset()
        lm.prefill(ids)
    ms_prefill = tmax(time_call(prefill, 5, 2))
    lm.generate_greedy(2)  # builds the graph
    ms_decode = tmax(time_call(lambda: lm.generate_greedy(steps), 3, 1))
    out["lm_130m"] = {"config": "d_model 768, 24 layers, d_state 16, vocab 50280, tied head, bf16, random init seed 0",
                      "prefill": {"batch": B, "seq_len": T, "ms": ms_prefill,
                                  "tokens_per_s": world * B * T / (ms_prefill * 1e-3)},
                      "decode": {"batch": B, "steps": steps, "ms": ms_decode, "cuda_graph": True,
                                 "tokens_per_s": world * B * steps / (ms_decode * 1e-3),
                                 "ms_per_step": ms_decode / steps}}
    del lm, w
    torch.cuda.empty_cache()
    # ---- 2.8b layer shape: training step ----
    L = 4
    cfg = mb.MambaConfig(d_model=2560, n_layers=L)
    Bm, Tm = 2, 8192
    w = mb.MambaWeights(cfg, dev, dtype=torch.bfloat16, vocab=V).init_random(3)
    tr = mb.MambaLMTrainer(w)
    tok = torch.randint(0, V, (Bm, Tm + 1), device=dev, dtype=torch.int32, generator=g)
    ms_train = tmax(time_call(lambda: tr.step(tok), 3, 1))
    out["lm_2p8b_train_step"] = {
        "config": f"d_model 2560, d_inner 5120, dt_rank 160, d_state 16, vocab 50280, {L} of 64 layers, bf16 compute / "
                  "f32 master, random init seed 3",
        "micro_batch": Bm, "seq_len": Tm, "ms": ms_train, "tokens_per_s": world * Bm * Tm / (ms_train * 1e-3),
        "parameters": int(w.n), "allreduce": "bucketed per layer under the backward" if world > 1 else "single rank"}
    del tr, w
    torch.cuda.empty_cache()
    return out


def collective_extra(dev, world, rank):
    """The one collective of the design, measured: all-reduce (sum) of a flat f32
    gradient arena, bucketed per layer, alone and issued on a side stream while the scan
    backward of the following layers runs (what a trainer does between backward and
    optimiser).  8 layers of the 2.8b shape (d_inner 5120: 43.3 M parameters per layer
    -> 173 MB per bucket) stand for its 64; the per-GPU shard is batch 2 x 8192."""
    import torch
    import torch.distributed as dist

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import parallel, synth
    L, per_layer = 8, 43_300_000
    B, T, D, N, S = 2, 8192, 5120, 16, 32
    bf = torch.bfloat16
    arena = torch.zeros(L * per_layer, device=dev)
    bounds = [(l * per_layer, (l + 1) * per_layer) for l in range(L)]
    par = synth.m1_scan_inputs(1, 1, D, N, 0, seed=rank, a_mode="random")
    a_neg = torch.from_numpy(par["a_neg"]).to(dev)
    Dp = torch.from_numpy(par["Dp"]).to(dev)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    x, z, dy = rn(B, T, D).to(bf), rn(B, T, D).to(bf), rn(B, T, D).to(bf)
    dl = (0.5 * rn(B, T, D) - 4.0).to(bf)
    Bm, Cm = rn(B, T, N).to(bf), rn(B, T, N).to(bf)
    cs = torch.empty(B, T // S, D, N, device=dev)
    ws = torch.empty(mb.selective_scan_bwd_workspace_bytes(B, T, D, N), dtype=torch.uint8, device=dev)
    mb.selective_scan_fwd(x, dl, Bm, Cm, a_neg, Dp, z, chunk_states=cs, save_stride=S)
    dA, dD = torch.zeros(D, N, device=dev), torch.zeros(D, device=dev)
    bwd = lambda: mb.selective_scan_bwd(x, dl, Bm, Cm, a_neg, Dp, dy, cs, S, z, dA_log=dA, dD=dD, workspace=ws)

    def step(overlap, compute=True, reduce=True):
        red = parallel.BucketedGradReducer(arena, bounds)
        for l in reversed(range(L)):
            if compute:
                bwd()
            if reduce and overlap:
                red.bucket_ready(l)
        if reduce and not overlap:
            for l in reversed(range(L)):
                red.bucket_ready(l)
        red.finish()

    def timed(**kw):
        for _ in range(2):
            step(**kw)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            step(**kw)
        e1.record()
        torch.cuda.synchronize()
        tt = torch.tensor([e0.elapsed_time(e1) / 3], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt)

    ms_bwd = timed(overlap=False, reduce=False)
    ms_red = timed(overlap=False, compute=False)
    ms_serial = timed(overlap=False)
    ms_overlap = timed(overlap=True)
    bytes_ = arena.numel() * 4
    return {"collective": "all-reduce (sum) of the flat f32 gradient arena, one bucket per layer",
            "layers": L, "bucket_bytes": per_layer * 4, "arena_bytes": bytes_,
            "shard": f"B={B} T={T} D={D} N={N} bf16 per GPU", "ms_backward_only": ms_bwd, "ms_allreduce_only": ms_red,
            "ms_backward_then_allreduce": ms_serial, "ms_overlapped": ms_overlap,
            "bus_GBps_per_gpu": 2 * (world - 1) / world * bytes_ / (ms_red * 1e-3) / 1e9,
            "nvlink_peer_copy_GBps_reference": 770.0,
            "hidden_fraction": max(0.0, min(1.0, (ms_serial - ms_overlap) / max(ms_red, 1e-9)))}


def bind_to_gpu_numa_node(local):
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, so that the
    pinned staging buffers allocated afterwards are local to that node."""
    try:
        import torch
        p = torch.cuda.get_device_properties(local)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        os.sched_setaffinity(0, cpus)
        return node
    except Exception:
        return None


def ncu_traffic_bytes():
    """dram read+write bytes of one launch of the dominant kernel from the ncu capture
    summarised under profiles/: None when the kernel source has changed since."""
    p = os.path.join(ROOT, "profiles", "sscan_fwd_traffic.txt")
    try:
        kv = dict(line.strip().split("=", 1) for line in open(p) if "=" in line)
        src = open(os.path.join(ROOT, "mamba_rs_b200", "csrc", "m1_fwd_kernel.cuh"), "rb").read()
        if kv.get("kernel_source_sha1") != hashlib.sha1(src).hexdigest():
            return None
        return int(kv["dram_bytes_per_launch_full_workload"])
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="skip the per-operator block")
    ap.add_argument("--batch", type=int, default=0,
                    help="sequences per GPU (default: the benchmark workload's 16); smaller values are for "
                         "profiler captures only and are reported in config.workload")
    ap.add_argument("--op", choices=OPS, help="time one operator on one GPU and print one JSON line")
    ap.add_argument("--save-stride", type=int, default=32)
    ap.add_argument("--heads", type=int, default=32, help="Mamba-3: number of heads")
    ap.add_argument("--headdim", type=int, default=64, help="Mamba-3: head dimension")
    ap.add_argument("--dstate", type=int, default=128, help="Mamba-3: state size")
    ap.add_argument("--sequential", action="store_true", help="Mamba-3 forward: the sequential kernel")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.op:
        return run_op(args)

    import torch
    import torch.distributed as dist

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)

    w = dict(WORKLOAD)
    if args.batch > 0:
        w["B"] = args.batch
        WORKLOAD["B"] = args.batch
    B, T, D, N = w["B"], w["T"], w["D"], w["N"]
    td = torch.bfloat16
    inp = synth.m1_scan_inputs(B, T, D, N, 0, seed=rank, a_mode="s4d")
    host = {k: torch.from_numpy(inp[k]).to(td).pin_memory() for k in ("x", "delta_raw", "Bm", "Cm", "z")}
    devt = {k: v.to(dev) for k, v in host.items()}
    a_neg = torch.from_numpy(inp["a_neg"]).to(dev)
    Dp = torch.from_numpy(inp["Dp"]).to(dev)
    ssm = torch.zeros(B, D, N, device=dev)
    y = torch.empty(B, T, D, device=dev, dtype=td)
    y_host = torch.empty(B, T, D, dtype=td).pin_memory()
    # inputs + output of one step are 4 x 100 MB: larger than the 126 MB L2,
    # so consecutive steps cannot be served from cache.
    handle = mb.ffi.default_handle(local)

    def step():
        ssm.zero_()
        mb.selective_scan_fwd(devt["x"], devt["delta_raw"], devt["Bm"], devt["Cm"], a_neg, Dp, devt["z"],
                              ssm_state=ssm, y=y, handle=handle)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the product path is checked against the oracle before anything is timed ----
    checked = None
    if rank == 0:
        import oracle
        step()
        torch.cuda.synchronize()
        bs, ds = min(3, B - 1), [5, D - 7]
        f = lambda t_: t_[bs:bs + 1].float().cpu().numpy()
        ref = oracle.m1_fused_fwd(f(devt["x"])[..., ds], f(devt["delta_raw"])[..., ds], f(devt["Bm"]), f(devt["Cm"]),
                                  f(devt["z"])[..., ds], inp["a_neg"][ds], inp["Dp"][ds])
        err = float(np.abs(f(y)[..., ds] - ref["y"]).max() / np.abs(ref["y"]).max())
        if not err <= 2e-2:
            raise SystemExit(f"bench.py: the scan output differs from the oracle (rel err {err:.3g}): not timing it")
        checked = {"against": "oracle.m1_fused_fwd, 1 sequence x 2 channels", "rel_err": err, "tol": 2e-2}

    # ---- device-resident throughput (value) + per-kernel time (roofline) ----
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for a, b in ev:
        ssm.zero_()
        a.record()  # brackets the scan kernel alone, on the launching stream
        mb.selective_scan_fwd(devt["x"], devt["delta_raw"], devt["Bm"], devt["Cm"], a_neg, Dp, devt["z"],
                              ssm_state=ssm, y=y, handle=handle)
        b.record()
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in ev]))
    handle.check_status()

    # ---- end to end through the operator with host buffers ----
    # Every step uploads its inputs from pinned host memory, runs the operator and
    # downloads y.  Steps are pipelined over three streams and two sets of device
    # buffers (upload of step i+1 and download of step i-1 overlap the kernel of
    # step i), as a serving loop would run them; the time is the whole loop's.
    e2e_ms = float("nan")
    if not args.no_e2e:
        dev2 = [devt, {k: torch.empty_like(v) for k, v in devt.items()}]
        y2 = [y, torch.empty_like(y)]
        yh2 = [y_host, torch.empty_like(y_host).pin_memory()]
        s_up, s_run, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

        def e2e_loop(n):
            up, run, down = [], [], []
            for i in range(n):
                k = i & 1
                with torch.cuda.stream(s_up):
                    if i >= 2:
                        s_up.wait_event(run[i - 2])  # the kernel that read this buffer set is done
                    for name in host:
                        dev2[k][name].copy_(host[name], non_blocking=True)
                    up.append(torch.cuda.Event())
                    up[-1].record()
                with torch.cuda.stream(s_run):
                    s_run.wait_event(up[i])
                    if i >= 2:
                        s_run.wait_event(down[i - 2])  # y of this set has been downloaded
                    ssm.zero_()
                    mb.selective_scan_fwd(dev2[k]["x"], dev2[k]["delta_raw"], dev2[k]["Bm"], dev2[k]["Cm"], a_neg,
                                          Dp, dev2[k]["z"], ssm_state=ssm, y=y2[k], handle=handle)
                    run.append(torch.cuda.Event())
                    run[-1].record()
                with torch.cuda.stream(s_down):
                    s_down.wait_event(run[i])
                    yh2[k].copy_(y2[k], non_blocking=True)
                    down.append(torch.cuda.Event())
                    down[-1].record()

        for st_ in (s_up, s_run, s_down):
            st_.wait_stream(torch.cuda.current_stream())
        e2e_loop(2)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(4, min(args.steps, 12))
        f0.record()
        for st_ in (s_up, s_run, s_down):
            st_.wait_event(f0)
        e2e_loop(n_e2e)
        for st_ in (s_up, s_run, s_down):
            torch.cuda.current_stream().wait_stream(st_)
        f1.record()
        barrier()
        e2e_ms = f0.elapsed_time(f1) / n_e2e
        del dev2, y2, yh2
    clocks = sampler.stop() if rank == 0 else None  # sampled over both timed regions

    times = torch.tensor([total_ms, 0.0 if args.no_e2e else e2e_ms, kern_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, kern_ms = [float(v) for v in times.cpu()]

    # ---- everything else on the path, after the headline region ----
    extra = None
    if not args.no_extra and not args.no_e2e:
        del devt, y
        torch.cuda.empty_cache()
        if world == 1:
            extra = {}
            for name in ("sscan_fwd_random_a", "sscan_bwd", "conv1d_fwd", "conv1d_bwd", "sscan_fwd_small_batch",
                         "decode_loop", "m3_ssd_fwd", "m3_ssd_fwd_fused_kq", "m3_ssd_bwd", "residual_rmsnorm_fwd",
                         "residual_rmsnorm_bwd", "softmax_xent", "adamw_step", "embedding_gather"):
                try:  # a failing extra must not take the headline line with it
                    r = measure_op(name, dev)
                    r.pop("op")
                    extra[name] = r
                except Exception as exc:
                    extra[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
                    torch.cuda.empty_cache()
        else:
            try:
                extra = {"gradient_allreduce": collective_extra(dev, world, rank)}
            except Exception as exc:
                extra = {"gradient_allreduce": {"error": f"{type(exc).__name__}: {exc}"[:300]}}
        try:
            extra.update(lm_extra(dev, world, rank))
        except Exception as exc:
            extra["lm"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    if rank == 0:
        by = algorithmic_bytes(w)
        ms_per_step = total_ms / args.steps
        peak, peak_src = measured_peaks()
        achieved = by / (kern_ms * 1e-3) / 1e9
        h2d = sum(v.numel() * v.element_size() for v in host.values())
        d2h = y_host.numel() * y_host.element_size()
        cfgb = config_block(world)
        cfgb["tokens_per_s"] = world * B * T / (ms_per_step * 1e-3)
        out = {
            "metric": METRIC, "value": world * by / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "storage_dtype": "bf16", "data": "synthetic", "config": cfgb,
            "clocks": clocks, "gpu_launches": args.steps, "checked_before_timing": checked,
            "e2e": (None if args.no_e2e else
                    {"value": world * by / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                     "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                     "staging_numa_node": numa,
                     "note": "PCIe-bound: every rank uploads 304 MB and downloads 101 MB per step through the "
                             "host's root complexes, which the GPUs of one box share"}),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": ncu_traffic_bytes(), "peak_source": peak_src,
                         "kernel": "sscan_fwd_kernel", "kernel_ms": kern_ms,
                         "algorithmic_bytes": by},
        }
        if extra is not None:
            if "sscan_fwd_random_a" in extra:
                out["roofline"]["general_path_frac"] = extra["sscan_fwd_random_a"]["frac_of_hbm_peak"]
                out["roofline"]["general_path_note"] = ("trained weights leave the arithmetic progression: one "
                                                        "exp2 per state and step")
            if "sscan_bwd" in extra:
                out["backward"] = {"ms": extra["sscan_bwd"]["ms"],
                                   "algorithmic_bytes": extra["sscan_bwd"]["algorithmic_bytes"],
                                   "GBps": extra["sscan_bwd"]["GBps"], "save_stride": 32,
                                   "frac_of_hbm_peak": extra["sscan_bwd"]["frac_of_hbm_peak"]}
            out["extra"] = extra
        if world == 1 and not args.no_cpu_baseline:
            cores = host_threads()
            val, secs = cpu_scan_leg(sample_B=B, sample_D=D)
            out["cpu_baseline"] = {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                                   "sample": f"the full workload ({B} sequences x {D} channels x L={T}), "
                                             f"best of 5 passes after one warm-up, {secs:.2f} s per pass",
                                   "note": "the reference's Rust build is unavailable on this box (no cargo)"}
            tps, psecs, pthreads = cpu_prefill_leg()
            out["cpu_baseline"]["forward_prefill"] = {
                "tokens_per_s": tps, "seconds_per_pass": psecs, "threads": pthreads,
                "workload": "backbone prefill d_model 128, 2 layers, d_inner 256, d_state 16, batch 4 x 512 f32 "
                            "(weights seed 42, inputs seed 7), one task per sample"}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
