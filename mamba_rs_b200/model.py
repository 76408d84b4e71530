"""Host-side mirror of the reference's Mamba-1 engines on top of the C ABI.

The reference's engines are per-layer launch sequences around the scan
(``GpuMambaBackbone::prefill_sequence_mixed`` / ``step``,
src/mamba_ssm/gpu/inference.rs:1515-1855, prefill.rs:676-961; ``MambaTrainer``,
src/mamba_ssm/gpu/trainer.rs:437-481, forward_mixed.rs:433-758,
backward_mixed.rs:83-782).  This module keeps their method names and argument
meaning and issues the same sequence with this library's fused entry points:

    residual+RMSNorm | GEMM in_proj | conv1d+SiLU | GEMM x_proj | GEMM dt_proj |
    scan (softplus, D skip, SiLU(z) gate fused) | GEMM out_proj | (residual add fused
    into the next layer's norm)

The dense projections stay library GEMMs (``torch.matmul`` -> cuBLAS), as they are
cuBLAS calls in the reference: they are not part of the scan path.  Parameters and
their gradients live in flat f32 arenas (the reference's ``GpuMambaGrads.flat``,
src/mamba_ssm/gpu/weights.rs:487-560) with a compute-dtype copy beside the master,
so the data-parallel all-reduce and AdamW are one call each over the arena.
torch supplies device memory, streams and the process group, nothing else.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import ops
from .parallel import BucketedGradReducer

__all__ = ["MambaConfig", "MambaWeights", "GpuMambaBackbone", "GpuMambaLM", "MambaLMTrainer"]


@dataclass
class MambaConfig:
    """src/config.rs:57-101."""
    d_model: int
    n_layers: int
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    rms_norm_eps: float = 1e-5
    dt_rank: int | None = None

    def __post_init__(self):
        if self.dt_rank is None:
            self.dt_rank = (self.d_model + 15) // 16
        if not (1 <= self.d_conv <= 8):
            raise ValueError("d_conv must be 1..8")
        if not (1 <= self.d_state <= 256):
            raise ValueError("d_state must be 1..256")

    @property
    def d_inner(self):
        return self.expand * self.d_model

    @property
    def xdbl_dim(self):
        return self.dt_rank + 2 * self.d_state


_LAYER_FIELDS = ("norm_w", "in_proj_w", "conv_w", "conv_b", "x_proj_w", "dt_proj_w", "dt_proj_b", "a_log", "d_param",
                 "out_proj_w")


class MambaWeights:
    """Flat f32 master arena + compute-dtype copy, with named views per layer
    (src/weights.rs:8-65).  GEMM weights are [in, out] row-major, as in the reference."""

    def __init__(self, cfg: MambaConfig, device, dtype=torch.bfloat16, vocab: int | None = None):
        self.cfg, self.device, self.dtype, self.vocab = cfg, device, dtype, vocab
        dm, di, N, K, dr, xd = cfg.d_model, cfg.d_inner, cfg.d_state, cfg.d_conv, cfg.dt_rank, cfg.xdbl_dim
        self.shapes = dict(norm_w=(dm,), in_proj_w=(dm, 2 * di), conv_w=(di, K), conv_b=(di,), x_proj_w=(di, xd),
                           dt_proj_w=(dr, di), dt_proj_b=(di,), a_log=(di, N), d_param=(di,), out_proj_w=(di, dm))
        per_layer = sum(math.prod(s) for s in self.shapes.values())
        self.layer_size = (per_layer + 63) // 64 * 64  # buckets start on 256-byte boundaries
        extra = dm + (vocab * dm if vocab else 0)
        self.n = cfg.n_layers * self.layer_size + extra
        self.master = torch.zeros(self.n, device=device)
        self.grad = torch.zeros(self.n, device=device)
        self.lp = torch.zeros(self.n, device=device, dtype=dtype) if dtype != torch.float32 else self.master
        self.a_neg = [torch.empty(di, N, device=device) for _ in range(cfg.n_layers)]

    # ---- views ----
    def _views(self, flat, l):
        o = l * self.layer_size
        out = {}
        for k in _LAYER_FIELDS:
            n = math.prod(self.shapes[k])
            out[k] = flat[o:o + n].view(self.shapes[k])
            o += n
        return out

    def layer(self, l, which="lp"):
        return self._views(getattr(self, which), l)

    def tail(self, which="lp"):
        flat = getattr(self, which)
        o = self.cfg.n_layers * self.layer_size
        dm = self.cfg.d_model
        out = dict(norm_f=flat[o:o + dm])
        if self.vocab:
            out["embedding"] = flat[o + dm:o + dm + self.vocab * dm].view(self.vocab, dm)
        return out

    def bucket_bounds(self):
        """One gradient bucket per layer, then the tail (final norm, embedding)."""
        b = [(l * self.layer_size, (l + 1) * self.layer_size) for l in range(self.cfg.n_layers)]
        b.append((self.cfg.n_layers * self.layer_size, self.n))
        return b

    def refresh(self):
        """master -> compute copy, and a_neg = -exp(a_log) (trainer.rs:78-111)."""
        if self.lp is not self.master:
            self.lp.copy_(self.master)
        for l in range(self.cfg.n_layers):
            torch.exp(self.layer(l, "master")["a_log"], out=self.a_neg[l]).neg_()

    def init_random(self, seed: int):
        """MambaWeights::init (src/weights.rs:107-160): Kaiming-uniform projections,
        A_log = ln(1..N), dt bias = inverse softplus of log-uniform dt in [1e-3, 1e-1], D = 1,
        norm weights 1 (the distributions; this generator is torch's, not the reference's LCG)."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        cfg = self.cfg

        def kaiming(t, fan_in):
            bound = math.sqrt(3.0 / fan_in)
            t.copy_((torch.rand(t.shape, device=self.device, generator=g) * 2 - 1) * bound)

        for l in range(cfg.n_layers):
            v = self.layer(l, "master")
            v["norm_w"].fill_(1.0)
            kaiming(v["in_proj_w"], cfg.d_model)
            kaiming(v["conv_w"], cfg.d_conv)
            v["conv_b"].zero_()
            kaiming(v["x_proj_w"], cfg.d_inner)
            kaiming(v["dt_proj_w"], cfg.dt_rank)
            dt = torch.exp(torch.rand(cfg.d_inner, device=self.device, generator=g) *
                           (math.log(1e-1) - math.log(1e-3)) + math.log(1e-3))
            v["dt_proj_b"].copy_(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
            v["a_log"].copy_(torch.log(torch.arange(1, cfg.d_state + 1, device=self.device).float()).expand_as(v["a_log"]))
            v["d_param"].fill_(1.0)
            kaiming(v["out_proj_w"], cfg.d_inner)
        t = self.tail("master")
        t["norm_f"].fill_(1.0)
        if self.vocab:
            t["embedding"].copy_(torch.randn(t["embedding"].shape, device=self.device, generator=g) * 0.02)
        self.refresh()
        return self

    def load_layers(self, layers, norm_f):
        """Copies named numpy / tensor arrays (same field names) into the master arena."""
        for l, src in enumerate(layers):
            v = self.layer(l, "master")
            for k in _LAYER_FIELDS:
                v[k].copy_(torch.as_tensor(src[k], dtype=torch.float32).reshape(self.shapes[k]))
        self.tail("master")["norm_f"].copy_(torch.as_tensor(norm_f, dtype=torch.float32))
        self.refresh()
        return self


class GpuMambaBackbone:
    """Prefill + decode over a residual stream [B, T, d_model] f32
    (``GpuMambaBackbone``, src/mamba_ssm/gpu/inference.rs:1515-1855): ``prefill_sequence``
    walks whole sequences, ``step`` one token; both update the recurrent state
    (``conv[L][B,D,K]``, ``ssm[L][B,D,N]`` f32) in place; ``reset`` zeroes it."""

    def __init__(self, weights: MambaWeights, batch: int):
        self.w, self.cfg, self.batch = weights, weights.cfg, batch
        dev, c = weights.device, weights.cfg
        self.conv = torch.zeros(c.n_layers, batch, c.d_inner, c.d_conv, device=dev)
        self.ssm = torch.zeros(c.n_layers, batch, c.d_inner, c.d_state, device=dev)
        self._ws = {}

    def reset(self):
        self.conv.zero_()
        self.ssm.zero_()

    def _fwd_ws(self, B, T):
        key = (B, T)
        if key not in self._ws:
            c = self.cfg
            self._ws[key] = torch.empty(ops.selective_scan_fwd_workspace_bytes(B, T, c.d_inner, c.d_state),
                                        dtype=torch.uint8, device=self.w.device)
        return self._ws[key]

    def prefill_sequence(self, temporal: torch.Tensor) -> torch.Tensor:
        """temporal [B, T, d_model] f32 (embedded inputs) -> norm_f(residual) [B, T, d_model]
        in the compute dtype.  The input tensor is used as the residual stream (updated in place)."""
        c, w = self.cfg, self.w
        B, T, dm = temporal.shape
        di, N, dr = c.d_inner, c.d_state, c.dt_rank
        res = temporal.view(B * T, dm)
        branch = None
        for l in range(c.n_layers):
            p = w.layer(l)
            post, _ = ops.residual_rmsnorm_fwd(res, branch, w.layer(l, "master")["norm_w"], eps=c.rms_norm_eps,
                                               out_dtype=w.dtype)
            proj = post @ p["in_proj_w"]                                   # [BT, 2 di]: x | z in place
            pv = proj.view(B, T, 2 * di)
            u = ops.conv1d_fwd(pv[..., :di], w.layer(l, "master")["conv_w"], w.layer(l, "master")["conv_b"], self.conv[l])
            xdbl = u.view(B * T, di) @ p["x_proj_w"]                       # [BT, dr + 2N]: dt | B | C in place
            delta = torch.addmm(p["dt_proj_b"], xdbl[:, :dr], p["dt_proj_w"])
            xv = xdbl.view(B, T, c.xdbl_dim)
            y = ops.selective_scan_fwd(u, delta.view(B, T, di), xv[..., dr:dr + N], xv[..., dr + N:], w.a_neg[l],
                                       w.layer(l, "master")["d_param"], pv[..., di:], ssm_state=self.ssm[l],
                                       workspace=self._fwd_ws(B, T))
            branch = y.view(B * T, di) @ p["out_proj_w"]
        out, _ = ops.residual_rmsnorm_fwd(res, branch, w.tail("master")["norm_f"], eps=c.rms_norm_eps, out_dtype=w.dtype)
        return out.view(B, T, dm)

    def step(self, temporal: torch.Tensor) -> torch.Tensor:
        """One token per sequence: temporal [B, d_model] f32 -> [B, d_model] (compute dtype)."""
        c, w = self.cfg, self.w
        B, dm = temporal.shape
        di, N, dr = c.d_inner, c.d_state, c.dt_rank
        res = temporal
        branch = None
        for l in range(c.n_layers):
            p, pm = w.layer(l), w.layer(l, "master")
            post, _ = ops.residual_rmsnorm_fwd(res, branch, pm["norm_w"], eps=c.rms_norm_eps, out_dtype=w.dtype)
            proj = post @ p["in_proj_w"]
            u = torch.empty(B, di, device=res.device, dtype=w.dtype)
            # x_proj needs u before the scan step can run: conv step first (u_out), then the
            # fused softplus + SSM step + gate on the ready u
            ops.conv1d_fwd(torch.as_strided(proj, (B, 1, di), (2 * di, 2 * di, 1)), pm["conv_w"], pm["conv_b"],
                           self.conv[l], u.view(B, 1, di))
            xdbl = u @ p["x_proj_w"]
            delta = torch.addmm(p["dt_proj_b"], xdbl[:, :dr], p["dt_proj_w"])
            y = ops.selective_scan_step(u, delta, xdbl[:, dr:dr + N], xdbl[:, dr + N:], w.a_neg[l], pm["d_param"],
                                        self.ssm[l], proj[:, di:])
            branch = y @ p["out_proj_w"]
        out, _ = ops.residual_rmsnorm_fwd(res, branch, w.tail("master")["norm_f"], eps=c.rms_norm_eps, out_dtype=w.dtype)
        return out


class GpuMambaLM:
    """Token-level wrapper with a tied head (``GpuMambaLM``, src/module/gpu_lm.rs:136-679):
    ``prefill`` runs whole prompts through the backbone and returns the logits of the last
    position, ``generate_greedy`` decodes token by token.  One decode step (embedding row,
    24-layer step, head GEMM, argmax) is captured in a CUDA graph on first use and replayed,
    as the reference captures its step (src/mamba_ssm/gpu/inference.rs:1608-1630)."""

    def __init__(self, weights: MambaWeights, batch: int):
        if not weights.vocab:
            raise ValueError("the LM needs weights with a vocabulary")
        self.w, self.batch = weights, batch
        self.backbone = GpuMambaBackbone(weights, batch)
        dev = weights.device
        self.next_ids = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.logits = torch.empty(batch, weights.vocab, device=dev, dtype=weights.dtype)
        self._graph = None

    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, T] int32 -> logits of the last position [B, vocab]; leaves the greedy
        next token in ``next_ids``."""
        B, T = ids.shape
        emb = self.w.tail()["embedding"]
        temporal = ops.embedding_gather(emb, ids.contiguous()).view(B, T, -1)
        hidden = self.backbone.prefill_sequence(temporal)
        torch.matmul(hidden[:, -1], emb.t(), out=self.logits)
        self.next_ids.copy_(self.logits.argmax(dim=1))
        return self.logits

    def _decode_once(self):
        emb = self.w.tail()["embedding"]
        temporal = ops.embedding_gather(emb, self.next_ids)
        hidden = self.backbone.step(temporal)
        torch.matmul(hidden, emb.t(), out=self.logits)
        self.next_ids.copy_(self.logits.argmax(dim=1))

    def generate_greedy(self, n: int, use_graph: bool = True) -> torch.Tensor:
        """n greedy tokens after a prefill; returns them as [B, n] int32."""
        out = torch.empty(self.batch, n, dtype=torch.int32, device=self.w.device)
        if use_graph and self._graph is None:
            dev = self.w.device
            keep = (self.backbone.conv.clone(), self.backbone.ssm.clone(), self.next_ids.clone())
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                self._decode_once()  # warm-up outside the capture (first-call set-up, cuBLAS workspaces)
            torch.cuda.current_stream(dev).wait_stream(side)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._decode_once()
            self.backbone.conv.copy_(keep[0])
            self.backbone.ssm.copy_(keep[1])
            self.next_ids.copy_(keep[2])
        for i in range(n):
            out[:, i] = self.next_ids
            if use_graph:
                self._graph.replay()
            else:
                self._decode_once()
        return out


class MambaLMTrainer:
    """A next-token training step on the device: embedding gather, the backbone forward
    with block-boundary state saves, tied-head logits, softmax cross-entropy, the manual
    backward (scan / conv / norm backward kernels of this library, GEMM gradients through
    cuBLAS), a bucketed gradient all-reduce that overlaps the rest of the backward, and
    fused AdamW.  ``forward`` / ``backward_step`` / ``step`` follow ``MambaTrainer``
    (src/mamba_ssm/gpu/trainer.rs:437-481); ``accumulate_only`` is its
    ``BackwardOpts::accumulate_only`` (trainer.rs:176-206) for micro-batching."""

    SAVE = 32  # steps between saved scan states

    def __init__(self, weights: MambaWeights, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, group=None):
        if not weights.vocab:
            raise ValueError("the LM trainer needs weights with a vocabulary")
        self.w, self.cfg, self.group = weights, weights.cfg, group
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.m = torch.zeros_like(weights.master)
        self.v = torch.zeros_like(weights.master)
        self.t = 0
        self.bias = torch.ones(2, device=weights.device)
        self._acts = None
        self._pending = 0

    # ---- forward ----
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, T+1] int32: predicts token t+1 from tokens <= t.  Returns the mean loss
        (a device scalar) and keeps what the backward needs."""
        c, w = self.cfg, self.w
        B, T1 = ids.shape
        T = T1 - 1
        di, N, dr, dm = c.d_inner, c.d_state, c.dt_rank, c.d_model
        S = self.SAVE
        emb = w.tail()["embedding"]
        inp = ids[:, :-1].contiguous()
        res = ops.embedding_gather(emb, inp)                      # [BT, dm] f32 residual stream
        acts, branch = [], None
        for l in range(c.n_layers):
            p, pm = w.layer(l), w.layer(l, "master")
            post, rms = ops.residual_rmsnorm_fwd(res, branch, pm["norm_w"], eps=c.rms_norm_eps, out_dtype=w.dtype)
            x_res = res.clone()                                    # the stream this norm saw
            proj = post @ p["in_proj_w"]
            pv = proj.view(B, T, 2 * di)
            u = ops.conv1d_fwd(pv[..., :di], pm["conv_w"], pm["conv_b"])
            xdbl = u.view(B * T, di) @ p["x_proj_w"]
            delta = torch.addmm(p["dt_proj_b"], xdbl[:, :dr], p["dt_proj_w"])
            xv = xdbl.view(B, T, c.xdbl_dim)
            cs = torch.empty(B, (T + S - 1) // S, di, N, device=res.device)
            y = ops.selective_scan_fwd(u, delta.view(B, T, di), xv[..., dr:dr + N], xv[..., dr + N:], w.a_neg[l],
                                       pm["d_param"], pv[..., di:], chunk_states=cs, save_stride=S)
            branch = y.view(B * T, di) @ p["out_proj_w"]
            acts.append(dict(x_res=x_res, rms=rms, post=post, proj=proj, u=u, xdbl=xdbl, delta=delta, cs=cs, y=y))
        hidden, rms_f = ops.residual_rmsnorm_fwd(res, branch, w.tail("master")["norm_f"], eps=c.rms_norm_eps,
                                                 out_dtype=w.dtype)
        logits = hidden @ emb.t()                                  # tied head, [BT, V]
        tgt = ids[:, 1:].contiguous().view(-1)
        loss_rows, dlogits = ops.softmax_xent(logits, tgt, grad_scale=1.0 / (B * T))
        self._acts = dict(layers=acts, res_f=res, rms_f=rms_f, hidden=hidden, dlogits=dlogits, inp=inp, B=B, T=T)
        return loss_rows.sum() / (B * T)

    # ---- backward + optimiser ----
    def backward_step(self, accumulate_only: bool = False):
        c, w, a = self.cfg, self.w, self._acts
        if a is None:
            raise RuntimeError("backward_step needs a forward first")
        B, T = a["B"], a["T"]
        di, N, dr, dm = c.d_inner, c.d_state, c.dt_rank, c.d_model
        S = self.SAVE
        L = c.n_layers
        red = None if accumulate_only else BucketedGradReducer(w.grad, w.bucket_bounds(), group=self.group, average=True)
        emb = w.tail()["embedding"]
        gt = w.tail("grad")
        dl = a["dlogits"]
        gt["embedding"].add_((dl.t() @ a["hidden"]).float())       # head weight gradient
        d_hidden = dl @ emb                                         # [BT, dm]
        d_res = torch.zeros(B * T, dm, device=w.device)
        ops.residual_rmsnorm_bwd(d_hidden, a["res_f"], w.tail("master")["norm_f"], a["rms_f"], d_res, gt["norm_f"])
        for l in reversed(range(L)):
            p, pm, g, s = w.layer(l), w.layer(l, "master"), w.layer(l, "grad"), a["layers"][l]
            pv = s["proj"].view(B, T, 2 * di)
            xv = s["xdbl"].view(B, T, c.xdbl_dim)
            d_out = d_res.to(w.dtype)                               # gradient of this layer's branch output
            g["out_proj_w"].add_((s["y"].view(B * T, di).t() @ d_out).float())
            d_y = (d_out @ p["out_proj_w"].t()).view(B, T, di)
            sb = ops.selective_scan_bwd(s["u"], s["delta"].view(B, T, di), xv[..., dr:dr + N], xv[..., dr + N:],
                                        w.a_neg[l], pm["d_param"], d_y, s["cs"], S, pv[..., di:],
                                        dA_log=g["a_log"], dD=g["d_param"])
            d_delta = sb["d_delta"].view(B * T, di)
            g["dt_proj_b"].add_(d_delta.float().sum(0))
            g["dt_proj_w"].add_((s["xdbl"][:, :dr].t() @ d_delta).float())
            d_xdbl = torch.empty(B * T, c.xdbl_dim, device=w.device, dtype=w.dtype)
            d_xdbl[:, :dr] = d_delta @ p["dt_proj_w"].t()
            d_xdbl[:, dr:dr + N] = sb["dB"].view(B * T, N)
            d_xdbl[:, dr + N:] = sb["dC"].view(B * T, N)
            g["x_proj_w"].add_((s["u"].view(B * T, di).t() @ d_xdbl).float())
            d_u = sb["d_u"].view(B * T, di) + d_xdbl @ p["x_proj_w"].t()   # backward_mixed.rs:350-580
            cg = ops.conv1d_bwd(pv[..., :di], pm["conv_w"], pm["conv_b"], d_u.view(B, T, di), None, dconv_w=g["conv_w"],
                                dconv_b=g["conv_b"])
            d_proj = torch.cat([cg["d_x"].view(B * T, di), sb["d_z"].view(B * T, di)], dim=1)
            g["in_proj_w"].add_((s["post"].t() @ d_proj).float())
            d_post = d_proj @ p["in_proj_w"].t()
            ops.residual_rmsnorm_bwd(d_post, s["x_res"], pm["norm_w"], s["rms"], d_res, g["norm_w"])
            if red is not None:
                red.bucket_ready(l)                                  # its all-reduce runs under layers l-1 .. 0
        # embedding rows: the residual gradient flows into the gathered rows
        gt["embedding"].index_add_(0, a["inp"].view(-1).long(), d_res)
        self._acts = None
        self._pending += 1
        if accumulate_only:
            return
        red.bucket_ready(L)
        red.finish()
        if self._pending > 1:
            w.grad.div_(self._pending)
        self._pending = 0
        self.t += 1
        b1, b2 = self.betas
        self.bias.copy_(torch.tensor([1.0 / (1.0 - b1 ** self.t), 1.0 / (1.0 - b2 ** self.t)]))
        ops.adamw_step(w.master, w.grad, self.m, self.v, self.bias, lr=self.lr, beta1=b1, beta2=b2, eps=self.eps,
                       weight_decay=self.wd, param_lp=None if w.lp is w.master else w.lp)
        for l in range(L):
            torch.exp(w.layer(l, "master")["a_log"], out=w.a_neg[l]).neg_()
        w.grad.zero_()

    def step(self, ids: torch.Tensor) -> torch.Tensor:
        loss = self.forward(ids)
        self.backward_step()
        return loss
