"""The entry points launch asynchronously, allocate nothing and never synchronise, so a
layer's worth of them can be captured in a CUDA graph and replayed (the reference
captures its step and training loops the same way, src/mamba_ssm/gpu/graph_capture.rs:32,
inference.rs:1608-1630): the replay must reproduce the eager launches bit for bit."""
import numpy as np
import pytest

from helpers import quantised_inputs, to_dev, torch_dtype

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_forward_backward_conv_and_step_replay_bit_identically_from_a_graph(cuda_dev, dt):
    import torch

    import mamba_rs_b200 as mb
    B, T, D, N, K, S = 2, 600, 96, 16, 4, 32
    q = quantised_inputs(B, T, D, N, K, dt, seed=21, a_mode="random")
    td = torch_dtype(dt)
    d = lambda a, t_=None: to_dev(a, cuda_dev, t_)
    x, dl, Bm, Cm, z = (d(q[k], td) for k in ("x", "delta_raw", "Bm", "Cm", "z"))
    a_neg, Dp, cw, cb = d(q["a_neg"]), d(q["Dp"]), d(q["conv_w"]), d(q["conv_b"])
    dy = d(np.random.default_rng(3).standard_normal((B, T, D)).astype(np.float32), td)
    # every buffer exists before the capture: pointers must be stable across replays
    u, y = torch.empty_like(x), torch.empty_like(x)
    cst, ssm = torch.zeros(B, D, K, device=cuda_dev), torch.zeros(B, D, N, device=cuda_dev)
    cs = torch.empty(B, (T + S - 1) // S, D, N, device=cuda_dev)
    ws = torch.empty(mb.selective_scan_bwd_workspace_bytes(B, T, D, N), dtype=torch.uint8, device=cuda_dev)
    wsc = torch.empty(int(mb.ffi.lib().mamba_b200_conv1d_bwd_workspace_bytes(B, T, D, K)), dtype=torch.uint8,
                      device=cuda_dev)
    wsf = torch.empty(mb.selective_scan_fwd_workspace_bytes(B, T, D, N), dtype=torch.uint8, device=cuda_dev)
    dA, dD = torch.zeros(D, N, device=cuda_dev), torch.zeros(D, device=cuda_dev)
    dW, db = torch.zeros(D, K, device=cuda_dev), torch.zeros(D, device=cuda_dev)
    ys = torch.empty(B, D, device=cuda_dev, dtype=td)
    out = {}

    def layer():
        cst.zero_(); ssm.zero_(); dA.zero_(); dD.zero_(); dW.zero_(); db.zero_()
        mb.conv1d_fwd(x, cw, cb, cst, u)
        mb.selective_scan_fwd(u, dl, Bm, Cm, a_neg, Dp, z, ssm_state=ssm, y=y, chunk_states=cs, save_stride=S,
                              workspace=wsf)  # small batch: the time-segment path (three launches)
        g = mb.selective_scan_bwd(u, dl, Bm, Cm, a_neg, Dp, dy, cs, S, z, dA_log=dA, dD=dD, workspace=ws)
        gc = mb.conv1d_bwd(x, cw, cb, g["d_u"], None, dconv_w=dW, dconv_b=db, workspace=wsc)
        mb.selective_scan_step(x[:, 0], dl[:, 0], Bm[:, 0], Cm[:, 0], a_neg, Dp, ssm, z[:, 0], conv_w=cw, conv_b=cb,
                               conv_state=cst, y=ys)
        out.update(g, d_x=gc["d_x"])

    def snapshot():
        torch.cuda.synchronize()
        keep = dict(out)
        keep.update(y=y, u=u, ssm=ssm, cst=cst, ys=ys, dA=dA, dD=dD, dW=dW, db=db)
        return {k: v.float().cpu().numpy().copy() for k, v in keep.items() if v is not None}

    layer()  # eager (also makes every first-call set-up happen outside the capture)
    eager = snapshot()
    side = torch.cuda.Stream(device=cuda_dev)
    side.wait_stream(torch.cuda.current_stream(cuda_dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        layer()
    for _ in range(2):
        for t_ in (y, u, ys):
            t_.zero_()
        graph.replay()
        replayed = snapshot()
        for k, v in eager.items():
            np.testing.assert_array_equal(replayed[k], v, err_msg=k)
    mb.ffi.default_handle(0).check_status()


def test_mamba3_tensor_core_kernels_replay_bit_identically_from_a_graph(cuda_dev):
    """The Mamba-3 kernels take their TMA tensor maps as kernel parameters, built on the host
    at launch: a captured launch keeps them, so a replay on the same buffers must reproduce the
    eager results (forward, forward with K / Q built in the kernel, backward)."""
    import torch

    import mamba_rs_b200 as mb
    from mamba_rs_b200 import synth
    B, T, nh, ng, hd, N, na = 2, 300, 4, 1, 64, 128, 32
    i = synth.m3_ssd_inputs(B, T, nh, hd, N, seed=4)
    g = synth.m3_group_inputs(B, T, nh, ng, N, na, i["dt"], seed=4)
    bf = torch.bfloat16
    t = lambda a, d=None: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_dev).to(d or torch.float32)
    x, K, Q = t(i["x"], bf), t(i["K"], bf), t(i["Q"], bf)
    dt, trap, adt, Dh = t(i["dt"]), t(i["trap"]), t(i["adt"]), t(i["Dh"])
    Bn, Cn, bb, cbias, vel = t(g["Bn"], bf), t(g["Cn"], bf), t(g["b_bias"]), t(g["c_bias"]), t(g["angle_vel"])
    ang0 = t(g["angle_state"])
    dy = torch.randn(B, T, nh * hd, device=cuda_dev, generator=torch.Generator(device=cuda_dev).manual_seed(5)).to(bf)
    y, y2 = torch.empty_like(x), torch.empty_like(x)
    ssm = torch.zeros(B, nh, hd, N, device=cuda_dev)
    ang = torch.empty_like(ang0)
    dD = torch.zeros(nh, device=cuda_dev)
    ws = torch.empty(mb.ffi.lib().mamba_b200_m3_ssd_bwd_workspace_bytes_for(2, B, T, nh, hd, N), dtype=torch.uint8,
                     device=cuda_dev)
    out = {}

    def work():
        ang.copy_(ang0)
        dD.zero_()
        mb.m3_ssd_fwd(x, K, Q, dt, trap, adt, Dh, ssm_state=ssm, y=y)
        mb.ops.m3_ssd_fwd_fused_kq(x, Bn, Cn, bb, cbias, vel, dt, trap, adt, Dh, angle_state=ang, y=y2)
        out.update(mb.m3_ssd_bwd(x, K, Q, dt, trap, adt, Dh, dy, dD=dD, workspace=ws))

    def snapshot():
        torch.cuda.synchronize()
        keep = dict(out)
        keep.update(y=y, y2=y2, ssm=ssm, ang=ang)
        return {k: v.float().cpu().numpy().copy() for k, v in keep.items() if v is not None}

    work()
    eager = snapshot()
    side = torch.cuda.Stream(device=cuda_dev)
    side.wait_stream(torch.cuda.current_stream(cuda_dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        work()
    for _ in range(2):
        y.zero_(); y2.zero_()
        graph.replay()
        replayed = snapshot()
        for k, v in eager.items():
            np.testing.assert_array_equal(replayed[k], v, err_msg=k)
    mb.ffi.default_handle(0).check_status()
