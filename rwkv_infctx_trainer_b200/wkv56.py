"""Shared host code of the v5 and v6 ops: fills the C-ABI argument block."""
from __future__ import annotations

import ctypes

import torch

from . import _lib as L

HEAD_SIZE = 64

# Debug aid: when True every call synchronises and checks the status word the chunked
# kernels keep at the start of their workspace (non-zero = a bounded device-side wait ran
# out and the kernel gave up).  Off by default: the ops never synchronise on their own.
CHECK_STATUS = False


def _check_status(lib, a, variant, ws, what):
    if (CHECK_STATUS and ws is not None and ws.numel() >= 4
            and lib.wkv56_uses_chunked(ctypes.byref(a), int(variant == "wkv6"))):
        torch.cuda.synchronize(ws.device)
        code = int(ws[:4].view(torch.int32).item())
        if code != 0:
            raise RuntimeError(f"{what}: device-side wait timed out (status {code})")


def _args(variant, B, T, H, dtype, w_kind, layout, path, **t) -> L.WkvArgs:
    a = L.WkvArgs()
    a.B, a.T, a.H, a.N = B, T, H, HEAD_SIZE
    a.dtype, a.w_kind, a.state_layout, a.path = L.DTYPE_CODE[dtype], w_kind, layout, path
    for name, tensor in t.items():
        setattr(a, name, L.ptr(tensor))
    return a


def _with_workspace(lib, variant, direction, a, dev):
    nbytes = getattr(lib, f"{variant}_{direction}_workspace")(ctypes.byref(a))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
    a.workspace, a.workspace_bytes = L.ptr(ws), nbytes
    return ws


def forward(variant: str, r, k, v, w, u, state_in, *, w_kind, layout=L.WKV_STATE_KV,
            path=L.WKV_PATH_AUTO, state_out=None, save_ckpt=False):
    """Launch wkv5_forward / wkv6_forward.  All tensors contiguous, on one device.
    Returns (y, state_out); ``state_out`` may be given (it may be ``state_in`` itself).
    With ``save_ckpt`` a third value is returned: the chunk-start states to hand to
    ``backward(..., ckpt=...)`` (None when the call did not run on the chunked kernels)."""
    B, T, C = r.shape
    H = C // HEAD_SIZE
    dev = L.require_cuda(r, k, v, w, u, state_in)
    y = torch.empty_like(r)
    if state_out is None:
        state_out = torch.empty((B, H, HEAD_SIZE, HEAD_SIZE), device=dev, dtype=torch.float32)
    lib = L.load()
    with torch.cuda.device(dev):
        a = _args(variant, B, T, H, r.dtype, w_kind, layout, path, r=r, k=k, v=v, w=w, u=u,
                  state_in=state_in, y=y, state_out=state_out)
        ckpt = None
        if save_ckpt:
            nck = lib.wkv56_state_ckpt_bytes(ctypes.byref(a), int(variant == "wkv6"))
            if nck:
                ckpt = torch.empty(nck, dtype=torch.uint8, device=dev)
                a.state_ckpt, a.state_ckpt_bytes = L.ptr(ckpt), nck
        ws = _with_workspace(lib, variant, "forward", a, dev)
        L.check(getattr(lib, f"{variant}_forward")(ctypes.byref(a), L.stream_handle(dev)),
                f"{variant}_forward")
        _check_status(lib, a, variant, ws, f"{variant}_forward")
        del ws
    if save_ckpt:
        return y, state_out, ckpt
    return y, state_out


def backward(variant: str, r, k, v, w, u, state_in, gy, gstate_out, *, w_kind,
             layout=L.WKV_STATE_KV, path=L.WKV_PATH_AUTO, want_gstate=True, ckpt=None):
    """Launch wkv5_backward / wkv6_backward.  Returns gr, gk, gv, gw, gu, gstate_in with
    gw = [B,T,C] (v6, activation dtype) or [B,C] fp32 per-batch partials (v5); gu [B,C] fp32."""
    B, T, C = r.shape
    H = C // HEAD_SIZE
    dev = L.require_cuda(r, k, v, w, u, state_in, gy, gstate_out)
    gr, gk, gv = torch.empty_like(r), torch.empty_like(r), torch.empty_like(r)
    if variant == "wkv6":
        gw = torch.empty_like(r)
    else:
        gw = torch.empty((B, C), device=dev, dtype=torch.float32)
    gu = torch.empty((B, C), device=dev, dtype=torch.float32)
    gsi = (torch.empty((B, H, HEAD_SIZE, HEAD_SIZE), device=dev, dtype=torch.float32)
           if want_gstate else None)
    lib = L.load()
    with torch.cuda.device(dev):
        a = _args(variant, B, T, H, r.dtype, w_kind, layout, path, r=r, k=k, v=v, w=w, u=u,
                  state_in=state_in, gy=gy, gstate_out=gstate_out, gr=gr, gk=gk, gv=gv, gw=gw,
                  gu=gu, gstate_in=gsi)
        if ckpt is not None:
            a.state_ckpt, a.state_ckpt_bytes = L.ptr(ckpt), ckpt.numel()
        ws = _with_workspace(lib, variant, "backward", a, dev)
        L.check(getattr(lib, f"{variant}_backward")(ctypes.byref(a), L.stream_handle(dev)),
                f"{variant}_backward")
        _check_status(lib, a, variant, ws, f"{variant}_backward")
        del ws
    return gr, gk, gv, gw, gu, gsi
