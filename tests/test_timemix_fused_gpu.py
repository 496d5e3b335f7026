"""The fused neighbours of the WKV op against the PyTorch expressions the trainer uses
(RWKV-v6/src/module/TimeMix.py:262-273 and 296-298), evaluated in fp32 on the same bf16
inputs.  Tolerance: max|ours-ref| / max|ref| <= 2e-2 on bf16 tensors (forward and gradients),
1e-3 on the fp32 parameter gradients' relative error against the fp32 evaluation."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def rel(a, b):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("B,T,H", [(1, 1, 1), (2, 37, 2), (3, 300, 5), (4, 1024, 64)])
def test_lnx_gate_matches_groupnorm_times_gate(B, T, H):
    import rwkv_infctx_trainer_b200 as W
    C = H * 64
    eps = 1e-5 * 8 ** 2      # RWKV-v6/src/module/TimeMix.py: ln_x eps = 1e-5 * head_size_divisor^2
    g0 = torch.Generator(device="cuda").manual_seed(B * 1000 + T)
    y = (torch.randn((B, T, C), generator=g0, device="cuda") * 3 + 0.5).to(BF).requires_grad_(True)
    g = torch.randn((B, T, C), generator=g0, device="cuda").to(BF).requires_grad_(True)
    wt = (torch.rand(C, generator=g0, device="cuda") + 0.5).requires_grad_(True)
    bs = (torch.randn(C, generator=g0, device="cuda") * 0.2).requires_grad_(True)
    gout = torch.randn((B, T, C), generator=g0, device="cuda").to(BF)
    out = W.lnx_gate(y, g, wt, bs, eps, H)
    out.backward(gout)
    got = [out, y.grad, g.grad, wt.grad, bs.grad]
    y2, g2, w2, b2 = (t.detach().float().requires_grad_(True) for t in (y, g, wt, bs))
    ref = F.group_norm(y2.view(-1, C), H, w2, b2, eps).view(B, T, C) * g2
    ref.backward(gout.float())
    want = [ref, y2.grad, g2.grad, w2.grad, b2.grad]
    for n, a, b, tol in zip(("out", "gy", "gg", "gweight", "gbias"), got, want, (2e-2, 2e-2, 2e-2, 1e-3, 1e-3)):
        assert torch.isfinite(a.float()).all(), n
        assert rel(a.float(), b) <= tol, (n, rel(a.float(), b))
    # repeatable bit for bit (fixed-order reductions)
    y.grad = g.grad = wt.grad = bs.grad = None
    out2 = W.lnx_gate(y, g, wt, bs, eps, H)
    out2.backward(gout)
    for a, b in zip(got, [out2, y.grad, g.grad, wt.grad, bs.grad]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("B,T,C,n", [(1, 1, 64, 5), (2, 65, 128, 5), (2, 300, 320, 1), (4, 1024, 4096, 5), (1, 129, 64, 1), (2, 200, 128, 4), (1, 70, 192, 3)])
def test_ddlerp_matches_token_shift_mix(B, T, C, n):
    import rwkv_infctx_trainer_b200 as W
    g0 = torch.Generator(device="cuda").manual_seed(C + T)
    x = torch.randn((B, T, C), generator=g0, device="cuda").to(BF).requires_grad_(True)
    shift = torch.randn((B, C), generator=g0, device="cuda").to(BF).requires_grad_(True)
    maa = torch.rand((n, C), generator=g0, device="cuda").requires_grad_(True)
    m = None if n == 1 else (torch.randn((n, B, T, C), generator=g0, device="cuda") * 0.3).to(BF).requires_grad_(True)
    gout = torch.randn((n, B, T, C), generator=g0, device="cuda").to(BF)
    out = W.ddlerp(x, shift, maa, m)
    out.backward(gout)
    got = [out, x.grad, shift.grad, maa.grad] + ([m.grad] if m is not None else [])
    x2, s2, a2 = (t.detach().float().requires_grad_(True) for t in (x, shift, maa))
    m2 = None if m is None else m.detach().float().requires_grad_(True)
    dx = torch.cat((s2.unsqueeze(1), x2[:, :-1]), 1) - x2
    ref = x2.unsqueeze(0) + dx.unsqueeze(0) * (a2.view(n, 1, 1, C) + (m2 if m2 is not None else 0.0))
    ref.backward(gout.float())
    want = [ref, x2.grad, s2.grad, a2.grad] + ([m2.grad] if m2 is not None else [])
    tols = [2e-2, 2e-2, 2e-2, 2e-3, 2e-2]
    for nme, a, b, tol in zip(("out", "gx", "gshift", "gmaa", "gm"), got, want, tols):
        assert torch.isfinite(a.float()).all(), nme
        assert rel(a.float(), b) <= tol, (nme, rel(a.float(), b))


def test_ddlerp_gradient_crosses_segment_boundaries():
    """two segments chained through `shift` (the previous segment's last token) give the
    gradients of the unsplit sequence: the C ABI's gshift_in / gshift_out do the carrying"""
    import ctypes
    from rwkv_infctx_trainer_b200 import _lib as L
    lib = L.load()
    B, T, C, n = 2, 128, 128, 5
    g0 = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((B, T, C), generator=g0, device="cuda").to(BF)
    shift = torch.randn((B, C), generator=g0, device="cuda").to(BF)
    maa = torch.rand((n, C), generator=g0, device="cuda")
    m = (torch.randn((n, B, T, C), generator=g0, device="cuda") * 0.3).to(BF)
    gout = torch.randn((n, B, T, C), generator=g0, device="cuda").to(BF)
    st = torch.cuda.current_stream().cuda_stream

    def bwd(xs, sh, ms, gs, gshift_in):
        Bq, Tq, _ = xs.shape
        gx, gm, gsh = torch.empty_like(xs), torch.empty_like(ms), torch.empty_like(sh)
        gma = torch.empty((n, C), device="cuda")
        nb = lib.wkv_ddlerp_backward_workspace(Bq, Tq, C, n)
        ws = torch.empty(nb, dtype=torch.uint8, device="cuda")
        L.check(lib.wkv_ddlerp_backward(Bq, Tq, C, n, xs.data_ptr(), sh.data_ptr(), maa.data_ptr(), ms.data_ptr(),
                                        gs.data_ptr(), None if gshift_in is None else gshift_in.data_ptr(),
                                        gx.data_ptr(), gm.data_ptr(), gsh.data_ptr(), gma.data_ptr(), ws.data_ptr(),
                                        nb, st), "bwd")
        return gx, gm, gsh, gma

    one = bwd(x, shift, m, gout, None)
    h = T // 2
    x0, x1 = x[:, :h].contiguous(), x[:, h:].contiguous()
    m0, m1 = m[:, :, :h].contiguous(), m[:, :, h:].contiguous()
    g0_, g1_ = gout[:, :, :h].contiguous(), gout[:, :, h:].contiguous()
    b = bwd(x1, x0[:, -1].contiguous(), m1, g1_, None)
    a = bwd(x0, shift, m0, g0_, b[2])
    torch.cuda.synchronize()
    assert rel(torch.cat((a[0], b[0]), 1).float(), one[0].float()) <= 1e-2
    assert rel(torch.cat((a[1], b[1]), 2).float(), one[1].float()) <= 1e-2
    assert rel(a[2].float(), one[2].float()) <= 1e-2
    assert rel(a[3] + b[3], one[3]) <= 1e-3
