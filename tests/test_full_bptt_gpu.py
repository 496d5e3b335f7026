"""Trainer-side check that the op's state gradient makes full (un-truncated) BPTT right.

RWKV-infctx-trainer forces ``bptt_truncated_learning = True`` for v6 because its CUDA kernel
returns no usable state gradient (RWKV-v6/src/model.py:291-299).  With WKV6 the gradient of a
later segment flows back through ``state_out -> state_in``.  This test builds a small time-mix
block of the v6 shape (token shift with a data-dependent mix, r/k/v/g projections, a low-rank
data-dependent decay, the WKV op, per-head GroupNorm, SiLU gate, output projection -- the
structure of RWKV-v6/src/module/TimeMix.py:255-300, written out here for the test) and trains
it one step three ways:

  whole      one call over all T tokens
  segmented  T cut into BPTT segments, the (shift, wkv) state carried WITH its gradient
  truncated  the same with the state detached between segments (what the trainer does today)

``segmented`` must reproduce the parameter gradients of ``whole``; ``truncated`` must not
(otherwise the test would not show anything).
"""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


class TinyTimeMix(nn.Module):
    def __init__(self, C, H, lora=16):
        super().__init__()
        g = torch.Generator().manual_seed(3)
        rnd = lambda *s, scale=1.0: nn.Parameter(torch.randn(*s, generator=g) * scale)
        self.H, self.C = H, C
        self.maa = rnd(6, C, scale=0.3)                   # x, w, k, v, r, g
        self.maa_w1, self.maa_w2 = rnd(C, 5 * lora, scale=0.05), rnd(5, lora, C, scale=0.05)
        self.decay = nn.Parameter(torch.linspace(-5, -0.5, C))
        self.decay_w1, self.decay_w2 = rnd(C, lora, scale=0.05), rnd(lora, C, scale=0.05)
        self.u = rnd(H, C // H, scale=0.3)
        self.wr, self.wk, self.wv, self.wg, self.wo = (rnd(C, C, scale=C ** -0.5) for _ in range(5))
        self.ln_x = nn.GroupNorm(H, C)

    def forward(self, x, state):
        import rwkv_infctx_trainer_b200 as W
        shift, wkv = state
        B, T, C = x.shape
        dx = torch.cat((shift.unsqueeze(1), x[:, :-1]), 1) - x
        xxx = torch.tanh((x + dx * self.maa[0]) @ self.maa_w1).view(B * T, 5, -1).transpose(0, 1)
        m = torch.bmm(xxx, self.maa_w2).view(5, B, T, C)
        xw, xk, xv, xr, xg = (x + dx * (self.maa[i + 1] + m[i]) for i in range(5))
        r, k, v, g = xr @ self.wr, xk @ self.wk, xv @ self.wv, F.silu(xg @ self.wg)
        w = self.decay + torch.tanh(xw @ self.decay_w1) @ self.decay_w2
        bf = torch.bfloat16
        y, wkv = W.WKV6.apply(B, T, C, self.H, r.to(bf), k.to(bf), v.to(bf), w.to(bf), self.u.to(bf), wkv)
        y = self.ln_x(y.float().view(-1, C)).view(B, T, C)
        return (y * g) @ self.wo, (x[:, -1], wkv)


def _grads(model, x, target, cuts, detach):
    model.zero_grad(set_to_none=True)
    B, _, C = x.shape
    state = (torch.zeros((B, C), device=x.device), torch.zeros((B, model.H, 64, 64), device=x.device))
    loss = 0.0
    for t0, t1 in cuts:
        out, state = model(x[:, t0:t1], state)
        loss = loss + ((out - target[:, t0:t1]) ** 2).sum()
        if detach:
            state = tuple(s.detach() for s in state)
    loss.backward()
    return {n: p.grad.detach().clone() for n, p in model.named_parameters()}, float(loss.detach())


def test_segmented_full_bptt_equals_one_long_segment():
    torch.manual_seed(0)
    B, T, C, H, seg = 2, 512, 128, 2, 128
    model = TinyTimeMix(C, H).cuda()
    x = torch.randn((B, T, C), device="cuda") * 0.5
    target = torch.randn((B, T, C), device="cuda")
    whole, l0 = _grads(model, x, target, [(0, T)], detach=False)
    cuts = [(t0, t0 + seg) for t0 in range(0, T, seg)]
    full, l1 = _grads(model, x, target, cuts, detach=False)
    trunc, l2 = _grads(model, x, target, cuts, detach=True)
    assert abs(l0 - l1) <= 2e-3 * abs(l0) and abs(l0 - l2) <= 2e-3 * abs(l0)   # the forward is the same
    rel = lambda a, b: float((a - b).abs().max() / b.abs().max().clamp_min(1e-20))
    worst_full = max(rel(full[n], whole[n]) for n in whole)
    worst_trunc = max(rel(trunc[n], whole[n]) for n in whole)
    # bf16 op outputs differ by rounding between the two chunkings; truncation is a different gradient
    assert worst_full <= 2e-2, {n: rel(full[n], whole[n]) for n in whole}
    assert worst_trunc >= 5 * max(worst_full, 1e-3), (worst_trunc, worst_full)
