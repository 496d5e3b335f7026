"""v5 WKV op (per-head 64x64 fp32 state, static per-channel decay).

Two interfaces over the same kernels:

``WKV5.apply(B,T,C,H,r,k,v,w,u,state_in) -> (y, state_out)``
    the full contract: differentiable w.r.t. r,k,v,w,u and state_in, accepts a
    gradient on state_out.  ``w`` is the raw ``time_decay`` (decay =
    exp(-exp(w))), state is fp32 ``[B,H,N,N]`` indexed [key,value] like
    rwkv_inner's kv_state (RWKV-v5/src/module/rwkv_inner.py:22).

``WKV5_CUDA`` / ``RUN_WKV5_CUDA`` / ``wkv5_cuda_kernel``
    name-for-name mirrors of RWKV-v5/src/module/TimeMix.py:20-154 and of the
    extension module bound in RWKV-v5/src/module/cuda/wkv5_op.cpp:124-142:
    same argument order, outputs pre-allocated by the caller, ``state`` mutated
    in place in the project kernels' [value,key] layout, no state gradient.
    Unlike the project's kernel the state is indexed per batch row.
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import wkv56

N = wkv56.HEAD_SIZE


def _check_shapes(B, T, C, H, r, k, v, u, state):
    if C != H * N:
        raise ValueError(f"C must equal H*{N}")
    for name, t in (("r", r), ("k", k), ("v", v)):
        if tuple(t.shape) != (B, T, C):
            raise ValueError(f"{name} must be [B,T,C]")
    if u.numel() != C:
        raise ValueError("u must have H*N elements")
    if state is not None and state.numel() != B * H * N * N:
        raise ValueError("state must be [B,H,N,N]")


class WKV5(torch.autograd.Function):
    @staticmethod
    def forward(ctx, B, T, C, H, r, k, v, w, u, state_in, path=L.WKV_PATH_AUTO, saved=None):
        _check_shapes(B, T, C, H, r, k, v, u, state_in)
        dt = r.dtype
        r, k, v = r.contiguous(), k.to(dt).contiguous(), v.to(dt).contiguous()
        wf = w.float().contiguous()
        uf = u.to(dt).contiguous()
        s_in = state_in.float().contiguous()
        y, s_out, ckpt = wkv56.forward("wkv5", r, k, v, wf, uf, s_in, w_kind=L.WKV_W_RAW, path=path,
                                       save_ckpt=any(ctx.needs_input_grad), saved=saved)
        ctx.has_ckpt = ckpt is not None
        ctx.save_for_backward(*((r, k, v, wf, uf, s_in) + ((ckpt,) if ckpt is not None else ())))
        ctx.meta = (B, T, C, H, path, w.dtype, u.dtype, w.shape, u.shape, state_in.dtype)
        return y, s_out.view(B, H, N, N)

    @staticmethod
    def backward(ctx, gy, gstate_out):
        st = ctx.saved_tensors          # (one access: saved-tensor hooks unpack once)
        r, k, v, wf, uf, s_in = st[:6]
        ckpt = st[6] if ctx.has_ckpt else None
        B, T, C, H, path, wdt, udt, wshape, ushape, sdt = ctx.meta
        gy = gy.to(r.dtype).contiguous()
        gso = None if gstate_out is None else gstate_out.float().contiguous()
        gr, gk, gv, gw, gu, gsi = wkv56.backward("wkv5", r, k, v, wf, uf, s_in, gy, gso,
                                                 w_kind=L.WKV_W_RAW, path=path, ckpt=ckpt)
        return (None, None, None, None, gr, gk, gv, gw.sum(0).view(wshape).to(wdt),
                gu.sum(0).view(ushape).to(udt), gsi.to(sdt), None, None)


def wkv5(r, k, v, w, u, state_in, path=L.WKV_PATH_AUTO):
    """Convenience form of ``WKV5.apply`` taking the sizes from ``r`` and ``u``."""
    B, T, C = r.shape
    return WKV5.apply(B, T, C, C // N, r, k, v, w, u, state_in, path)


# ----------------------------------------------------------------------------
# literal drop-ins


class _Wkv5Kernel:
    """Stand-in for the project's ``wkv5`` extension module (wkv5_op.cpp:124-142)."""

    @staticmethod
    def _fwd(dt, B, T, C, H, state, r, k, v, eew, u, y):
        for t in (r, k, v, u, y):
            if t.dtype != dt:
                raise TypeError(f"expected {dt} tensors")
        if state.dtype != torch.float32 or eew.dtype != torch.float32:
            raise TypeError("state and w must be float32")
        ew = torch.log(eew.float()).contiguous()
        y_new, _ = wkv56.forward("wkv5", r, k, v, ew, u, state, w_kind=L.WKV_W_NEGEXP,
                                 layout=L.WKV_STATE_VK, state_out=state)
        y.copy_(y_new)

    @staticmethod
    def _bwd(dt, B, T, C, H, state, r, k, v, eew, ew, u, gy, gr, gk, gv, gw, gu):
        for t in (r, k, v, u, gy):
            if t.dtype != dt:
                raise TypeError(f"expected {dt} tensors")
        a, b, c, d, e, _ = wkv56.backward("wkv5", r, k, v, ew.float().contiguous(), u, state, gy,
                                          None, w_kind=L.WKV_W_NEGEXP, layout=L.WKV_STATE_VK,
                                          want_gstate=False)
        gr.copy_(a); gk.copy_(b); gv.copy_(c); gw.copy_(d.view_as(gw)); gu.copy_(e.view_as(gu))

    def forward_bf16(self, *a): self._fwd(torch.bfloat16, *a)
    def forward_fp16(self, *a): self._fwd(torch.float16, *a)
    def forward_fp32(self, *a): self._fwd(torch.float32, *a)
    def backward_bf16(self, *a): self._bwd(torch.bfloat16, *a)
    def backward_fp16(self, *a): self._bwd(torch.float16, *a)
    def backward_fp32(self, *a): self._bwd(torch.float32, *a)


wkv5_cuda_kernel = _Wkv5Kernel()


class WKV5_CUDA(torch.autograd.Function):
    """RWKV-v5/src/module/TimeMix.py:20-143: ``apply(B,T,C,H,state,r,k,v,w,u) -> y``;
    ``state`` (fp32, [B,H,value,key]) is updated in place; no gradient flows to it."""

    @staticmethod
    def forward(ctx, B, T, C, H, state, r, k, v, w, u):
        with torch.no_grad():
            dtype = r.dtype
            ctx.B, ctx.T, ctx.C, ctx.H, ctx.dtype = B, T, C, H, dtype
            if state.dtype != torch.float32 or w.dtype != torch.float32:
                raise TypeError("state and w must be float32")
            for t in (state, w, r, k, v, u):
                if not t.is_contiguous():
                    raise ValueError("inputs must be contiguous")
            if not (dtype == k.dtype == v.dtype == u.dtype):
                raise TypeError("r,k,v,u must share one dtype")
            if dtype not in L.DTYPE_CODE:
                raise ValueError(f"Unsupported dtype {dtype} for WKV5_CUDA")
            ew = (-torch.exp(w.float())).contiguous()
            eew = torch.exp(ew).contiguous()
            ctx.save_for_backward(r, k, v, eew, ew, u, state.clone())
            y = torch.empty(B, T, C, device=r.device, dtype=dtype)
            name = {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32"}[dtype]
            getattr(wkv5_cuda_kernel, "forward_" + name)(B, T, C, H, state, r, k, v, eew, u, y)
            return y

    @staticmethod
    def backward(ctx, gy):
        with torch.no_grad():
            B, T, C, H, dtype = ctx.B, ctx.T, ctx.C, ctx.H, ctx.dtype
            gy = gy.to(dtype).contiguous()
            r, k, v, eew, ew, u, in_state = ctx.saved_tensors
            mk = lambda *s: torch.empty(s, device=gy.device, dtype=dtype)
            gr, gk, gv, gw, gu = mk(B, T, C), mk(B, T, C), mk(B, T, C), mk(B, C), mk(B, C)
            name = {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32"}[dtype]
            getattr(wkv5_cuda_kernel, "backward_" + name)(B, T, C, H, in_state, r, k, v, eew, ew,
                                                          u, gy, gr, gk, gv, gw, gu)
            gw = torch.sum(gw, 0).view(H, C // H)
            gu = torch.sum(gu, 0).view(H, C // H)
            return (None, None, None, None, None, gr, gk, gv, gw, gu)


def RUN_WKV5_CUDA(B, T, C, H, state, r, k, v, w, u):
    """RWKV-v5/src/module/TimeMix.py:145-154."""
    return WKV5_CUDA.apply(B, T, C, H, state, r, k, v, w, u)
