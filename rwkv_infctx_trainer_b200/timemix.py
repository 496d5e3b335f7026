"""The elementwise neighbours of the WKV op in the time-mix block, each one fused CUDA pass.

``lnx_gate(y, g, weight, bias, eps, n_head)``
    ``ln_x(y.view(-1,C)).view(B,T,C) * g`` of RWKV-v6/src/module/TimeMix.py:296-298
    (``ln_x = nn.GroupNorm(n_head, C, eps=...)``), differentiable w.r.t. y, g, weight, bias.

``ddlerp(x, shift, maa, m=None)``
    the token-shift mixes of RWKV-v6/src/module/TimeMix.py:262-273:
    ``x + (x_prev - x) * (maa[i] + m[i])`` for every i, with ``x_prev`` the previous token
    (``shift`` [B,C] before a row's first token).  ``maa`` [n,C], ``m`` [n,B,T,C] or None,
    n = 1, 3, 4 or 5; returns [n,B,T,C].  Differentiable w.r.t. x, shift, maa, m.

bf16 tensors only (the dtype the trainer runs these in); parameters may have any float dtype.
"""
from __future__ import annotations

import torch

from . import _lib as L

HEAD_SIZE = 64


def _bf16_contig(name, t):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16")
    return t.contiguous()


class _LnxGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, g, weight, bias, eps, n_head):
        dev = L.require_cuda(y, g, weight, bias)
        C = y.shape[-1]
        if C != n_head * HEAD_SIZE or g.shape != y.shape or weight.numel() != C or bias.numel() != C:
            raise ValueError("y, g must be [..., n_head*64]; weight, bias [n_head*64]")
        y2, g2 = _bf16_contig("y", y), _bf16_contig("g", g)
        ga, be = weight.detach().float().contiguous(), bias.detach().float().contiguous()
        out = torch.empty_like(y2)
        tokens = y2.numel() // C
        with torch.cuda.device(dev):
            L.check(L.load().wkv_lnx_gate_forward(tokens, n_head, L.ptr(y2), L.ptr(g2), L.ptr(ga), L.ptr(be),
                                                  float(eps), L.ptr(out), L.stream_handle(dev)),
                    "wkv_lnx_gate_forward")
        ctx.save_for_backward(y2, g2, ga, be)
        ctx.meta = (float(eps), n_head, weight.dtype, bias.dtype, weight.shape, bias.shape)
        return out

    @staticmethod
    def backward(ctx, gout):
        y2, g2, ga, be = ctx.saved_tensors
        eps, n_head, wdt, bdt, wsh, bsh = ctx.meta
        dev, C = y2.device, y2.shape[-1]
        tokens = y2.numel() // C
        gout = _bf16_contig("grad", gout.to(torch.bfloat16))
        gy, gg = torch.empty_like(y2), torch.empty_like(y2)
        gga, gbe = torch.empty(C, device=dev), torch.empty(C, device=dev)
        lib = L.load()
        with torch.cuda.device(dev):
            n = lib.wkv_lnx_gate_backward_workspace(tokens, n_head)
            ws = torch.empty(max(n, 16), dtype=torch.uint8, device=dev)
            L.check(lib.wkv_lnx_gate_backward(tokens, n_head, L.ptr(y2), L.ptr(g2), L.ptr(ga), L.ptr(be), eps,
                                              L.ptr(gout), L.ptr(gy), L.ptr(gg), L.ptr(gga), L.ptr(gbe),
                                              L.ptr(ws), n, L.stream_handle(dev)), "wkv_lnx_gate_backward")
        return gy, gg, gga.view(wsh).to(wdt), gbe.view(bsh).to(bdt), None, None


def lnx_gate(y, g, weight, bias, eps, n_head):
    return _LnxGate.apply(y, g, weight, bias, eps, n_head)


class _DDLerp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shift, maa, m):
        dev = L.require_cuda(x, shift, maa, m)
        B, T, C = x.shape
        n = maa.shape[0]
        if maa.shape != (n, C) or shift.shape != (B, C) or (m is not None and m.shape != (n, B, T, C)):
            raise ValueError("x [B,T,C], shift [B,C], maa [n,C], m [n,B,T,C]")
        x2, sh = _bf16_contig("x", x), _bf16_contig("shift", shift)
        m2 = None if m is None else _bf16_contig("m", m)
        ma = maa.detach().float().contiguous()
        out = torch.empty((n, B, T, C), device=dev, dtype=torch.bfloat16)
        with torch.cuda.device(dev):
            L.check(L.load().wkv_ddlerp_forward(B, T, C, n, L.ptr(x2), L.ptr(sh), L.ptr(ma), L.ptr(m2), L.ptr(out),
                                                L.stream_handle(dev)), "wkv_ddlerp_forward")
        ctx.save_for_backward(x2, sh, ma) if m2 is None else ctx.save_for_backward(x2, sh, ma, m2)
        ctx.meta = (maa.dtype, m is not None)
        return out

    @staticmethod
    def backward(ctx, gout):
        st = ctx.saved_tensors
        x2, sh, ma = st[:3]
        m2 = st[3] if ctx.meta[1] else None
        B, T, C = x2.shape
        n, dev = ma.shape[0], x2.device
        gout = _bf16_contig("grad", gout.to(torch.bfloat16))
        gx = torch.empty_like(x2)
        gm = None if m2 is None else torch.empty_like(m2)
        gsh = torch.empty_like(sh)
        gma = torch.empty((n, C), device=dev)
        lib = L.load()
        with torch.cuda.device(dev):
            nb = lib.wkv_ddlerp_backward_workspace(B, T, C, n)
            ws = torch.empty(max(nb, 16), dtype=torch.uint8, device=dev)
            L.check(lib.wkv_ddlerp_backward(B, T, C, n, L.ptr(x2), L.ptr(sh), L.ptr(ma), L.ptr(m2), L.ptr(gout), None,
                                            L.ptr(gx), L.ptr(gm), L.ptr(gsh), L.ptr(gma), L.ptr(ws), nb,
                                            L.stream_handle(dev)), "wkv_ddlerp_backward")
        return gx, gsh, gma.to(ctx.meta[0]), gm


def ddlerp(x, shift, maa, m=None):
    return _DDLerp.apply(x, shift, maa, m)
