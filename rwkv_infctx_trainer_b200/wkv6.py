"""v6 WKV op (per-head 64x64 fp32 state, data-dependent per-token decay).

``WKV6.apply(B,T,C,H,r,k,v,w,u,state_in) -> (y, state_out)``
    the full contract: differentiable w.r.t. r,k,v,w,u and state_in, accepts a
    gradient on state_out.  ``w`` is the raw decay activation x ``[B,T,C]``
    (decay = exp(-exp(x)), RWKV-v6/src/module/TimeMix.py:280-281); state is fp32
    ``[B,H,N,N]`` indexed [key,value] (RWKV-v6/src/module/rwkv_inner.py:22).

``WKV6STATE_CUDA`` / ``RUN_WKV6STATE_CUDA`` / ``wkv6state_cuda_kernel``
    name-for-name mirrors of RWKV-v6/src/module/TimeMix.py:19-118.  The module
    object exports the functions that file actually calls
    (``forward_bf16`` ... ``backward_fp32``, TimeMix.py:59-64, 95-100) and the
    ``forward`` / ``backward`` names the project's extension defines
    (RWKV-v6/src/module/cuda/wkv6state_op.cpp:14-22).  ``s`` is updated in place
    in the kernels' [value,key] layout and, unlike the project's kernel, is
    indexed per batch row and kept in fp32 while computing.
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import wkv56

N = wkv56.HEAD_SIZE


class WKV6(torch.autograd.Function):
    @staticmethod
    def forward(ctx, B, T, C, H, r, k, v, w, u, state_in, path=L.WKV_PATH_AUTO, saved=None):
        if C != H * N:
            raise ValueError(f"C must equal H*{N}")
        for name, t in (("r", r), ("k", k), ("v", v), ("w", w)):
            if tuple(t.shape) != (B, T, C):
                raise ValueError(f"{name} must be [B,T,C]")
        if u.numel() != C or state_in.numel() != B * H * N * N:
            raise ValueError("u must be [H,N] and state [B,H,N,N]")
        dt = r.dtype
        r, k, v = r.contiguous(), k.to(dt).contiguous(), v.to(dt).contiguous()
        wx = w.to(dt).contiguous()
        uf = u.to(dt).contiguous()
        s_in = state_in.float().contiguous()
        # the hand-over to backward is only built when something asks for a gradient (not in the
        # first, autograd-free run of a checkpointed block)
        y, s_out, ckpt = wkv56.forward("wkv6", r, k, v, wx, uf, s_in, w_kind=L.WKV_W_RAW, path=path,
                                       save_ckpt=any(ctx.needs_input_grad), saved=saved)
        ctx.has_ckpt = ckpt is not None
        ctx.save_for_backward(*((r, k, v, wx, uf, s_in) + ((ckpt,) if ckpt is not None else ())))
        ctx.meta = (B, T, C, H, path, w.dtype, u.dtype, u.shape, state_in.dtype)
        return y, s_out.view(B, H, N, N)

    @staticmethod
    def backward(ctx, gy, gstate_out):
        st = ctx.saved_tensors          # (one access: saved-tensor hooks unpack once)
        r, k, v, wx, uf, s_in = st[:6]
        ckpt = st[6] if ctx.has_ckpt else None
        B, T, C, H, path, wdt, udt, ushape, sdt = ctx.meta
        gy = gy.to(r.dtype).contiguous()
        gso = None if gstate_out is None else gstate_out.float().contiguous()
        gr, gk, gv, gw, gu, gsi = wkv56.backward("wkv6", r, k, v, wx, uf, s_in, gy, gso,
                                                 w_kind=L.WKV_W_RAW, path=path, ckpt=ckpt)
        return (None, None, None, None, gr, gk, gv, gw.to(wdt), gu.sum(0).view(ushape).to(udt),
                gsi.to(sdt), None, None)


def wkv6(r, k, v, w, u, state_in, path=L.WKV_PATH_AUTO, saved=None):
    """Convenience form of ``WKV6.apply`` taking the sizes from ``r``.  ``saved``: a
    ``wkv56.SavedStates`` shared by the two forward runs of an activation-checkpointed block."""
    B, T, C = r.shape
    return WKV6.apply(B, T, C, C // N, r, k, v, w, u, state_in, path, saved)


# ----------------------------------------------------------------------------
# literal drop-ins


class _Wkv6StateKernel:
    """Stand-in for the extension module RWKV-v6/src/module/TimeMix.py loads."""

    @staticmethod
    def _fwd(dt, B, T, C, H, r, k, v, ew, u, s, y):
        if dt is not None:
            for t in (r, k, v, u, y):
                if t.dtype != dt:
                    raise TypeError(f"expected {dt} tensors")
        if ew.dtype != torch.float32:
            raise TypeError("ew must be float32")
        s32 = s.float().contiguous()
        y_new, _ = wkv56.forward("wkv6", r, k, v, ew.contiguous(), u, s32, w_kind=L.WKV_W_NEGEXP,
                                 layout=L.WKV_STATE_VK, state_out=s32)
        y.copy_(y_new)
        if s32.data_ptr() != s.data_ptr():
            s.copy_(s32.view_as(s))

    @staticmethod
    def _bwd(dt, B, T, C, H, r, k, v, ew, u, s, gy, gr, gk, gv, gw, gu, gs):
        if dt is not None:
            for t in (r, k, v, u, gy):
                if t.dtype != dt:
                    raise TypeError(f"expected {dt} tensors")
        a, b, c, d, e, f = wkv56.backward("wkv6", r, k, v, ew.float().contiguous(), u,
                                          s.float().contiguous(), gy, None,
                                          w_kind=L.WKV_W_NEGEXP, layout=L.WKV_STATE_VK)
        gr.copy_(a); gk.copy_(b); gv.copy_(c); gw.copy_(d); gu.copy_(e.view_as(gu))
        gs.copy_(f.view_as(gs))

    def forward_bf16(self, *a): self._fwd(torch.bfloat16, *a)
    def forward_fp16(self, *a): self._fwd(torch.float16, *a)
    def forward_fp32(self, *a): self._fwd(torch.float32, *a)
    def backward_bf16(self, *a): self._bwd(torch.bfloat16, *a)
    def backward_fp16(self, *a): self._bwd(torch.float16, *a)
    def backward_fp32(self, *a): self._bwd(torch.float32, *a)
    def forward(self, *a): self._fwd(None, *a)      # wkv6state_op.cpp:15
    def backward(self, *a): self._bwd(None, *a)     # wkv6state_op.cpp:16


wkv6state_cuda_kernel = _Wkv6StateKernel()


class _Wkv6Kernel:
    """Stand-in for the stateless extension module ``wkv6``
    (RWKV-v6/src/module/cuda/wkv6_op.cpp:8-22): ``forward(B,T,C,H,r,k,v,w,u,y)`` and
    ``backward(B,T,C,H,r,k,v,w,u,gy,gr,gk,gv,gw,gu)`` with ``w`` the fp32 ``ew = -exp(x)``; the
    state starts from zero, is not returned, and takes no gradient."""

    @staticmethod
    def forward(B, T, C, H, r, k, v, w, u, y):
        if w.dtype != torch.float32:
            raise TypeError("w must be float32 (ew = -exp(x))")
        y_new, _ = wkv56.forward("wkv6", r, k, v, w.contiguous(), u, None, w_kind=L.WKV_W_NEGEXP,
                                 layout=L.WKV_STATE_VK)
        y.copy_(y_new)

    @staticmethod
    def backward(B, T, C, H, r, k, v, w, u, gy, gr, gk, gv, gw, gu):
        a, b, c, d, e, _ = wkv56.backward("wkv6", r, k, v, w.float().contiguous(), u, None, gy, None,
                                          w_kind=L.WKV_W_NEGEXP, layout=L.WKV_STATE_VK, want_gstate=False)
        gr.copy_(a); gk.copy_(b); gv.copy_(c); gw.copy_(d); gu.copy_(e.view_as(gu))


wkv6_cuda_kernel = _Wkv6Kernel()


class WKV6STATE_CUDA(torch.autograd.Function):
    """RWKV-v6/src/module/TimeMix.py:19-109: ``apply(B,T,C,H,r,k,v,w,u,s) -> y`` with
    ``s`` updated in place ([value,key] layout, any float dtype, indexed per batch row);
    backward returns (gr,gk,gv,gw,gu,gs).  The raw decay activation ``w`` goes to the
    kernels as it is (they apply exp(-exp(w)) themselves), so bf16 calls run on the
    chunked tensor-core path; ``wkv6state_cuda_kernel`` keeps the project's lower-level
    signature with the precomputed ``ew`` for callers that use it directly."""

    @staticmethod
    def forward(ctx, B, T, C, H, r, k, v, w, u, s):
        with torch.no_grad():
            dtype = r.dtype
            ctx.B, ctx.T, ctx.C, ctx.H, ctx.dtype = B, T, C, H, dtype
            for t in (s, w, r, k, v, u):
                if not t.is_contiguous():
                    raise ValueError("inputs must be contiguous")
            if not (dtype == k.dtype == v.dtype == u.dtype):
                raise TypeError("r,k,v,u must share one dtype")
            if dtype not in L.DTYPE_CODE:
                raise ValueError(f"Unsupported dtype {dtype} for WKV6_CUDA")
            wx = w.to(dtype).contiguous()
            s32 = s.float().contiguous()
            s_in = s32.clone()
            y, _, ckpt = wkv56.forward("wkv6", r, k, v, wx, u, s32, w_kind=L.WKV_W_RAW,
                                       layout=L.WKV_STATE_VK, state_out=s32, save_ckpt=True)
            if s32.data_ptr() != s.data_ptr():
                s.copy_(s32.view_as(s))
            ctx.has_ckpt = ckpt is not None
            ctx.save_for_backward(*((r, k, v, wx, u, s_in) + ((ckpt,) if ckpt is not None else ())))
            ctx.s_dtype, ctx.w_dtype = s.dtype, w.dtype
            return y

    @staticmethod
    def backward(ctx, gy):
        with torch.no_grad():
            B, T, C, H, dtype = ctx.B, ctx.T, ctx.C, ctx.H, ctx.dtype
            gy = gy.to(dtype).contiguous()
            st = ctx.saved_tensors          # (one access: saved-tensor hooks unpack once)
            r, k, v, wx, u, s_in = st[:6]
            ckpt = st[6] if ctx.has_ckpt else None
            gr, gk, gv, gw, gu, gs = wkv56.backward("wkv6", r, k, v, wx, u, s_in, gy, None,
                                                    w_kind=L.WKV_W_RAW, layout=L.WKV_STATE_VK,
                                                    ckpt=ckpt)
            gu = torch.sum(gu, 0).view(H, C // H).to(dtype)
            return (None, None, None, None, gr, gk, gv, gw.to(ctx.w_dtype), gu,
                    gs.view(B, H, C // H, C // H).to(ctx.s_dtype))


def RUN_WKV6STATE_CUDA(B, T, C, H, r, k, v, w, u, s):
    """RWKV-v6/src/module/TimeMix.py:111-118."""
    return WKV6STATE_CUDA.apply(B, T, C, H, r, k, v, w, u, s)
