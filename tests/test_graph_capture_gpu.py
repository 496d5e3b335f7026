"""A forward + backward call chain captured into a CUDA graph replays to the same bits.

The C-ABI calls only enqueue work on the stream they are given (kernels launched as a
programmatic chain, one 256-byte memset): a host that captures its step into a CUDA graph,
as a trainer that wants no launch overhead does, can capture them.  The prepared calls of
``wkv56`` are used so that nothing but the C ABI runs inside the capture.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant,B,T,H", [("wkv6", 2, 640, 3), ("wkv5", 1, 512, 4), ("wkv6", 1, 1024, 2)])
def test_prepared_calls_capture_and_replay(variant, B, T, H):
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import wkv56
    C = H * 64
    g = torch.Generator().manual_seed(7)
    bf = torch.bfloat16
    mk = lambda: torch.randn((B, T, C), generator=g).to(bf).cuda()
    r, k, v, gy = mk(), mk(), mk(), mk()
    if variant == "wkv6":
        w = (torch.randn((B, T, C), generator=g) * 0.5 - 0.6).to(bf).cuda()
    else:
        w = (torch.rand((H, 64), generator=g) * 5 - 6).float().cuda()
    u = torch.rand((H, 64), generator=g).to(bf).cuda()
    s0 = (torch.randn((B, H, 64, 64), generator=g) * 0.1).cuda()
    gs = (torch.randn((B, H, 64, 64), generator=g) * 0.1).cuda()
    f = wkv56.prepare_forward(variant, r, k, v, w, u, s0, w_kind=W.WKV_W_RAW)
    b = wkv56.prepare_backward(variant, r, k, v, w, u, s0, gy, gs, w_kind=W.WKV_W_RAW, ckpt=f.ckpt)
    outs = lambda: [f.y, f.state_out, b.gr, b.gk, b.gv, b.gw, b.gu, b.gstate_in]

    f.run(); b.run()                      # plain launches: the reference bits (and the one-time kernel set-up)
    torch.cuda.synchronize()
    want = [t.clone() for t in outs()]
    assert f.status() == 0 and b.status() == 0

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            f.run(); b.run()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        for t in outs():
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for name, a, e in zip(("y", "state_out", "gr", "gk", "gv", "gw", "gu", "gstate_in"), outs(), want):
            assert torch.equal(a, e), name
    assert f.status() == 0 and b.status() == 0
