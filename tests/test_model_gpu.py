"""The host-side engines (mamba_rs_b200.model) against the CPU oracle's backbone prefill
(d_model 128, 2 layers, f32: every layer's GEMMs, conv, scan, gate, norm chained) and
against a float64 torch restatement with autograd for the training step's gradients."""
import numpy as np
import pytest

import oracle
from helpers import rel_err

pytestmark = pytest.mark.gpu


def host(t):
    return t.float().cpu().numpy()


def reference_weights(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    ocfg = oracle.m1_config(d_model=128, n_layers=2, d_state=16, d_conv=4, expand=2, dt_rank=8, input_dim=128)
    flat = oracle.m1_weights_init(ocfg, 42)
    lv = oracle.m1_layer_views(ocfg, flat)
    cfg = mb.MambaConfig(d_model=128, n_layers=2, d_state=16, d_conv=4, expand=2, dt_rank=8)
    w = mb.MambaWeights(cfg, cuda_dev, dtype=torch.float32)
    w.load_layers(lv["layers"], lv["norm_f"])
    return ocfg, flat, lv, cfg, w


def test_backbone_prefill_matches_the_cpu_backbone_end_to_end(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    ocfg, flat, lv, cfg, w = reference_weights(cuda_dev)
    B, T = 4, 512
    inp = np.random.default_rng(7).standard_normal((B, T, 128)).astype(np.float32)
    refs = [oracle.m1_prefill(ocfg, flat, inp[b]) for b in range(B)]
    # input projection (a GEMM outside the path) on the host, as the oracle does it
    temporal = (inp.astype(np.float64) @ lv["input_proj_w"].astype(np.float64) + lv["input_proj_b"]).astype(np.float32)
    bb = mb.GpuMambaBackbone(w, B)
    out = bb.prefill_sequence(torch.from_numpy(temporal).to(cuda_dev))
    torch.cuda.synchronize()
    ref_out = np.stack([r["out"] for r in refs])
    assert rel_err(host(out), ref_out) <= 1e-4
    assert rel_err(host(bb.ssm), np.stack([r["ssm_state"] for r in refs], axis=1)) <= 1e-4
    np.testing.assert_allclose(host(bb.conv), np.stack([r["conv_state"] for r in refs], axis=1), rtol=0, atol=2e-5)
    mb.ffi.default_handle(0).check_status()


def test_decode_steps_continue_the_prefill(cuda_dev):
    """prefill(T) followed by step() on the next tokens == prefill(T + k) (tests/prefill.rs:174-232)."""
    import torch

    import mamba_rs_b200 as mb
    _, _, _, cfg, w = reference_weights(cuda_dev)
    B, T, k = 3, 100, 5
    g = torch.Generator(device=cuda_dev).manual_seed(3)
    x = torch.randn(B, T + k, 128, device=cuda_dev, generator=g)
    whole = mb.GpuMambaBackbone(w, B)
    ref = whole.prefill_sequence(x.clone())
    bb = mb.GpuMambaBackbone(w, B)
    head = bb.prefill_sequence(x[:, :T].clone().contiguous())
    steps = [bb.step(x[:, T + i].clone().contiguous()) for i in range(k)]
    torch.cuda.synchronize()
    got = torch.cat([head, torch.stack(steps, dim=1)], dim=1)
    assert rel_err(host(got), host(ref)) <= 1e-4
    assert rel_err(host(bb.ssm), host(whole.ssm)) <= 1e-4
    bb.reset()
    assert float(bb.ssm.abs().max()) == 0.0 and float(bb.conv.abs().max()) == 0.0


def torch_reference_loss(w, cfg, ids):
    """float64 restatement of the training forward with autograd (sequential scan)."""
    import torch
    import torch.nn.functional as F
    P = [{k: v.detach().double().requires_grad_(True) for k, v in w.layer(l, "master").items()} for l in range(cfg.n_layers)]
    tail = {k: v.detach().double().requires_grad_(True) for k, v in w.tail("master").items()}
    B, T1 = ids.shape
    T, di, N, dr, K = T1 - 1, cfg.d_inner, cfg.d_state, cfg.dt_rank, cfg.d_conv
    s = tail["embedding"][ids[:, :-1].long()]

    def norm(x, wt):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + cfg.rms_norm_eps) * wt

    for p in P:
        post = norm(s, p["norm_w"])
        proj = post @ p["in_proj_w"]
        x, z = proj[..., :di], proj[..., di:]
        xp = F.pad(x.transpose(1, 2), (K - 1, 0))
        u = F.silu(F.conv1d(xp, p["conv_w"][:, None, :], p["conv_b"], groups=di)).transpose(1, 2)
        xdbl = u @ p["x_proj_w"]
        delta = F.softplus(xdbl[..., :dr] @ p["dt_proj_w"] + p["dt_proj_b"])
        Bm, Cm = xdbl[..., dr:dr + N], xdbl[..., dr + N:]
        a = -torch.exp(p["a_log"])
        h = torch.zeros(B, di, N, dtype=torch.float64, device=s.device)
        ys = []
        for t in range(T):
            h = torch.exp(delta[:, t, :, None] * a) * h + (delta[:, t] * u[:, t])[..., None] * Bm[:, t, None, :]
            ys.append((h * Cm[:, t, None, :]).sum(-1) + p["d_param"] * u[:, t])
        y = torch.stack(ys, 1) * F.silu(z)
        s = s + y @ p["out_proj_w"]
    logits = norm(s, tail["norm_f"]) @ tail["embedding"].t()
    loss = F.cross_entropy(logits.view(B * T, -1), ids[:, 1:].reshape(-1).long())
    loss.backward()
    return loss.item(), P, tail


def test_training_step_gradients_match_autograd_and_adamw_reduces_the_loss(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    cfg = mb.MambaConfig(d_model=32, n_layers=2, d_state=16, d_conv=4, expand=2)
    V, B, T = 50, 2, 70
    w = mb.MambaWeights(cfg, cuda_dev, dtype=torch.float32, vocab=V).init_random(5)
    ids = torch.randint(0, V, (B, T + 1), device=cuda_dev, dtype=torch.int32,
                        generator=torch.Generator(device=cuda_dev).manual_seed(1))
    tr = mb.MambaLMTrainer(w, lr=3e-3, weight_decay=0.0)
    loss = tr.forward(ids)
    tr.backward_step(accumulate_only=True)
    torch.cuda.synchronize()
    ref_loss, P, tail = torch_reference_loss(w, cfg, ids)
    assert abs(float(loss) - ref_loss) <= 1e-4 * abs(ref_loss)
    for l in range(cfg.n_layers):
        g = w.layer(l, "grad")
        for k, v in P[l].items():
            assert rel_err(host(g[k]), v.grad.cpu().numpy()) <= 2e-3, (l, k)
    gt = w.tail("grad")
    for k, v in tail.items():
        assert rel_err(host(gt[k]), v.grad.cpu().numpy()) <= 2e-3, k
    # a few optimiser steps on the same batch: the loss goes down
    w.grad.zero_()
    tr._pending = 0
    first = float(tr.step(ids))
    for _ in range(5):
        last = float(tr.step(ids))
    assert last < first
    mb.ffi.default_handle(0).check_status()


def test_bf16_training_step_runs_at_a_model_layer_shape(cuda_dev):
    """130m layer shape (d_model 768, d_inner 1536, dt_rank 48), 2 layers, bf16: finite loss
    close to ln(vocab) at initialisation, finite gradients."""
    import torch

    import mamba_rs_b200 as mb
    cfg = mb.MambaConfig(d_model=768, n_layers=2)
    V, B, T = 5000, 2, 256
    w = mb.MambaWeights(cfg, cuda_dev, dtype=torch.bfloat16, vocab=V).init_random(0)
    ids = torch.randint(0, V, (B, T + 1), device=cuda_dev, dtype=torch.int32)
    tr = mb.MambaLMTrainer(w)
    loss = tr.forward(ids)
    tr.backward_step(accumulate_only=True)
    torch.cuda.synchronize()
    assert abs(float(loss) - np.log(V)) < 0.5
    assert bool(torch.isfinite(w.grad).all()) and float(w.grad.abs().max()) > 0


def test_greedy_decode_from_a_captured_graph_equals_eager_decode(cuda_dev):
    import torch

    import mamba_rs_b200 as mb
    cfg = mb.MambaConfig(d_model=128, n_layers=3)
    V, B, T, n = 997, 4, 60, 12
    w = mb.MambaWeights(cfg, cuda_dev, dtype=torch.bfloat16, vocab=V).init_random(11)
    ids = torch.randint(0, V, (B, T), device=cuda_dev, dtype=torch.int32,
                        generator=torch.Generator(device=cuda_dev).manual_seed(2))
    outs = []
    for use_graph in (False, True):
        lm = mb.GpuMambaLM(w, B)
        lm.prefill(ids)
        outs.append(lm.generate_greedy(n, use_graph=use_graph).cpu().numpy())
    np.testing.assert_array_equal(outs[0], outs[1])
    assert outs[0].min() >= 0 and outs[0].max() < V
