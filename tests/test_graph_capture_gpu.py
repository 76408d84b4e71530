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
