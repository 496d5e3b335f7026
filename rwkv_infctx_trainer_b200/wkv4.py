"""v4 WKV op: drop-in for RWKV-v4neo's ``torch.ops.rwkv.wkv``.

Mirrors, name for name, the host interface of RWKV-infctx-trainer's v4 path:
  * ``WKVFunction`` / ``wkv``  -- RWKV-v4neo/cuda/wkv_op_bf16.cpp:13-92
  * op registration ``rwkv::wkv(Tensor w, Tensor u, Tensor k, Tensor v,
    Tensor last_state) -> Tensor[]`` -- wkv_op_bf16.cpp:98
  * ``wkv_op(time_decay, time_first, k, v, wkv_state)`` -- RWKV-v4neo/src/model.py:130-132
Beyond the project's kernel: u,k,v may be fp32 or fp16 as well as bf16, and T has
no compile-time limit.
"""
from __future__ import annotations

import torch

from . import _lib as L


def _ws(nbytes: int, device) -> torch.Tensor | None:
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


class WKVFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, raw_w, raw_u, raw_k, raw_v, raw_last_state):
        if raw_k.dim() != 3:
            raise ValueError("k must be [B,T,C]")
        B, T, C = raw_k.shape
        if raw_w.shape != (C,) or raw_u.shape != (C,):
            raise ValueError("time_decay and time_first must be [C]")
        if raw_v.shape != (B, T, C):
            raise ValueError("v must match k")
        if raw_last_state.shape != (B, C, 3):
            raise ValueError("last_state must be [B,C,3]")
        dev = L.require_cuda(raw_w, raw_u, raw_k, raw_v, raw_last_state)
        dt = raw_k.dtype
        if dt not in L.DTYPE_CODE:
            raise ValueError(f"unsupported dtype {dt}")
        w = -torch.exp(raw_w.float().contiguous())
        u = raw_u.to(dt).contiguous()
        k = raw_k.contiguous()
        v = raw_v.to(dt).contiguous()
        last_state = raw_last_state.float().contiguous()
        y = torch.empty_like(k)
        new_state = torch.empty_like(last_state)
        lib = L.load()
        with torch.cuda.device(dev):
            nbytes = lib.wkv4_forward_workspace(B, T, C)
            ws = _ws(nbytes, dev)
            # the states at the start of every 64-token piece go to backward (when there will be one)
            nck = lib.wkv4_state_ckpt_bytes(B, T, C) if any(ctx.needs_input_grad) else 0
            ckpt = _ws(nck, dev)
            L.check(lib.wkv4_forward_ckpt(B, T, C, L.DTYPE_CODE[dt], L.ptr(w), L.ptr(u), L.ptr(k),
                                          L.ptr(v), L.ptr(last_state), L.ptr(y), L.ptr(new_state),
                                          L.ptr(ws), nbytes, L.ptr(ckpt), nck, L.stream_handle(dev)),
                    "wkv4_forward")
        ctx.has_ckpt = ckpt is not None
        ctx.save_for_backward(*((w, u, k, v, last_state) + ((ckpt,) if ckpt is not None else ())))
        ctx.u_dtype = raw_u.dtype
        return y, new_state

    @staticmethod
    def backward(ctx, gy, gnew_state):
        st = ctx.saved_tensors
        w, u, k, v, last_state = st[:5]
        ckpt = st[5] if ctx.has_ckpt else None
        B, T, C = k.shape
        dev = k.device
        dt = k.dtype
        gy = gy.to(dt).contiguous()
        gns = None if gnew_state is None else gnew_state.float().contiguous()
        gw = torch.empty((B, C), device=dev, dtype=torch.float32)
        gu = torch.empty((B, C), device=dev, dtype=torch.float32)
        gk = torch.empty_like(k)
        gv = torch.empty_like(v)
        glast = torch.empty_like(last_state)
        lib = L.load()
        with torch.cuda.device(dev):
            nbytes = lib.wkv4_backward_workspace(B, T, C)
            ws = _ws(nbytes, dev)
            L.check(lib.wkv4_backward_ckpt(B, T, C, L.DTYPE_CODE[dt], L.ptr(w), L.ptr(u), L.ptr(k),
                                           L.ptr(v), L.ptr(last_state), L.ptr(gy), L.ptr(gns),
                                           L.ptr(gw), L.ptr(gu), L.ptr(gk), L.ptr(gv), L.ptr(glast),
                                           L.ptr(ws), nbytes, L.ptr(ckpt), 0 if ckpt is None else ckpt.numel(),
                                           L.stream_handle(dev)), "wkv4_backward")
        return gw.sum(0), gu.sum(0).to(ctx.u_dtype), gk, gv, glast


def wkv(w, u, k, v, last_state):
    """Same as the project's C++ ``wkv``: returns [y, new_state]."""
    return list(WKVFunction.apply(w, u, k, v, last_state))


def wkv_op(time_decay, time_first, k, v, wkv_state):
    """RWKV-v4neo/src/model.py:130-132."""
    return torch.ops.rwkv.wkv(time_decay, time_first, k, v, wkv_state)


_registered = False


def register_torch_op() -> None:
    """Register ``rwkv::wkv`` with the schema of wkv_op_bf16.cpp:98 so that
    ``torch.ops.rwkv.wkv`` resolves to this implementation."""
    global _registered, _libdef
    if _registered:
        return
    _libdef = torch.library.Library("rwkv", "DEF")
    _libdef.define("wkv(Tensor w, Tensor u, Tensor k, Tensor v, Tensor last_state) -> Tensor[]")
    _libdef.impl("wkv", wkv, "CompositeImplicitAutograd")
    _registered = True
