"""TEST INFRASTRUCTURE ONLY -- numpy front end of the fp64 CPU oracle.

Wraps ``wkv_naive.c`` (same directory; see its header for the reference lines
it restates).  Only ``tests/``, the smoke check and the CPU-baseline leg of
``bench.py`` may import this module; the shipped package never does.

All functions take and return float64 numpy arrays.  Layouts: ``r,k,v,gy`` are
``[B,T,C]``; v5/v6 state is ``[B,H,N,N]`` indexed ``[key, value]``; v4 state is
``[B,C,3] = (p,q,o)``.

Decay parametrisations (``x`` is what the trainer's modules hold):
  v4  ``w = -exp(time_decay)``                    (wkv_op_bf16.cpp:34)
  v5  ``wdec = exp(-exp(time_decay[h,n]))``      (RWKV-v5/src/module/TimeMix.py:57-60)
  v6  ``wdec = exp(-exp(x[b,t,c]))``             (RWKV-v6/src/module/TimeMix.py:49-51)
The ``*_x`` helpers return gradients w.r.t. ``x``, which is what the
project's kernels return as ``gw``.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

_lib = None
_dp = ctypes.POINTER(ctypes.c_double)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build_naive())
    return _lib


def _a(x):
    if x is None:
        return None
    if hasattr(x, "detach"):
        x = x.detach().cpu().double().numpy()
    return np.ascontiguousarray(x, dtype=np.float64)


def _p(x):
    return None if x is None else x.ctypes.data_as(_dp)


# ---------------------------------------------------------------- v4 ----

def wkv4_fwd(w, u, k, v, state_in=None):
    w, u, k, v, state_in = map(_a, (w, u, k, v, state_in))
    B, T, C = k.shape
    y = np.empty_like(k)
    so = np.empty((B, C, 3))
    lib().wkv4_naive_fwd(B, T, C, _p(w), _p(u), _p(k), _p(v), _p(state_in), _p(y), _p(so))
    return y, so


def wkv4_bwd(w, u, k, v, state_in, gy, gstate_out=None):
    w, u, k, v, state_in, gy, gstate_out = map(_a, (w, u, k, v, state_in, gy, gstate_out))
    B, T, C = k.shape
    gw = np.empty((B, C)); gu = np.empty((B, C))
    gk = np.empty_like(k); gv = np.empty_like(k); gsi = np.empty((B, C, 3))
    lib().wkv4_naive_bwd(B, T, C, _p(w), _p(u), _p(k), _p(v), _p(state_in), _p(gy),
                         _p(gstate_out), _p(gw), _p(gu), _p(gk), _p(gv), _p(gsi))
    return dict(gw=gw, gu=gu, gk=gk, gv=gv, gstate_in=gsi)


# ------------------------------------------------------------ v5 / v6 ----

def _fwd56(r, k, v, wdec, wsb, wst, u, state_in, H):
    B, T, C = r.shape
    N = C // H
    y = np.empty_like(r)
    so = np.empty((B, H, N, N))
    lib().wkv56_naive_fwd(B, T, H, N, _p(r), _p(k), _p(v), _p(wdec), ctypes.c_long(wsb),
                          ctypes.c_long(wst), _p(u), _p(state_in), _p(y), _p(so))
    return y, so


def _bwd56(r, k, v, wdec, wsb, wst, u, state_in, gy, gstate_out, H):
    B, T, C = r.shape
    N = C // H
    gr = np.empty_like(r); gk = np.empty_like(r); gv = np.empty_like(r)
    gwd = np.zeros_like(r); gu = np.empty((B, C)); gsi = np.empty((B, H, N, N))
    lib().wkv56_naive_bwd(B, T, H, N, _p(r), _p(k), _p(v), _p(wdec), ctypes.c_long(wsb),
                          ctypes.c_long(wst), _p(u), _p(state_in), _p(gy), _p(gstate_out),
                          _p(gr), _p(gk), _p(gv), _p(gwd), _p(gu), _p(gsi))
    return gr, gk, gv, gwd, gu, gsi


def wkv6_fwd(r, k, v, wdec, u, state_in=None):
    """wdec [B,T,C] in (0,1]; u [H,N]."""
    r, k, v, wdec, u, state_in = map(_a, (r, k, v, wdec, u, state_in))
    B, T, C = r.shape
    return _fwd56(r, k, v, wdec, T * C, C, u, state_in, u.shape[0])


def wkv6_bwd(r, k, v, wdec, u, state_in, gy, gstate_out=None):
    """Returns dict with gr,gk,gv,gwdec [B,T,C] (dL/dwdec), gu [B,C], gstate_in."""
    r, k, v, wdec, u, state_in, gy, gstate_out = map(
        _a, (r, k, v, wdec, u, state_in, gy, gstate_out))
    B, T, C = r.shape
    gr, gk, gv, gwd, gu, gsi = _bwd56(r, k, v, wdec, T * C, C, u, state_in, gy, gstate_out,
                                      u.shape[0])
    return dict(gr=gr, gk=gk, gv=gv, gwdec=gwd, gu=gu, gstate_in=gsi)


def wkv6_fwd_x(r, k, v, x, u, state_in=None):
    x = _a(x)
    return wkv6_fwd(r, k, v, np.exp(-np.exp(x)), u, state_in)


def wkv6_bwd_x(r, k, v, x, u, state_in, gy, gstate_out=None):
    """As wkv6_bwd but 'gw' is the gradient w.r.t. x where wdec = exp(-exp(x))."""
    x = _a(x)
    lw = -np.exp(x)
    wdec = np.exp(lw)
    out = wkv6_bwd(r, k, v, wdec, u, state_in, gy, gstate_out)
    out["gw"] = out.pop("gwdec") * wdec * lw
    return out


def wkv5_fwd(r, k, v, wdec, u, state_in=None):
    """wdec [H,N] in (0,1] shared by every token; u [H,N]."""
    r, k, v, wdec, u, state_in = map(_a, (r, k, v, wdec, u, state_in))
    return _fwd56(r, k, v, wdec.reshape(-1), 0, 0, u, state_in, u.shape[0])


def wkv5_bwd(r, k, v, wdec, u, state_in, gy, gstate_out=None):
    """gwdec is [B,C]: dL/dwdec per batch row (summed over tokens)."""
    r, k, v, wdec, u, state_in, gy, gstate_out = map(
        _a, (r, k, v, wdec, u, state_in, gy, gstate_out))
    gr, gk, gv, gwd, gu, gsi = _bwd56(r, k, v, wdec.reshape(-1), 0, 0, u, state_in, gy,
                                      gstate_out, u.shape[0])
    return dict(gr=gr, gk=gk, gv=gv, gwdec=gwd.sum(axis=1), gu=gu, gstate_in=gsi)


def wkv5_fwd_x(r, k, v, td, u, state_in=None):
    td = _a(td)
    return wkv5_fwd(r, k, v, np.exp(-np.exp(td)), u, state_in)


def wkv5_bwd_x(r, k, v, td, u, state_in, gy, gstate_out=None):
    """'gw' [B,C] is the per-batch gradient w.r.t. time_decay (wdec = exp(-exp(td)))."""
    td = _a(td)
    lw = -np.exp(td)
    wdec = np.exp(lw)
    out = wkv5_bwd(r, k, v, wdec, u, state_in, gy, gstate_out)
    out["gw"] = out.pop("gwdec") * (wdec * lw).reshape(1, -1)
    return out


def max_rel_err(a, b) -> float:
    """max|a-b| / max|b| -- the error metric every parity test uses."""
    a = _a(a); b = _a(b)
    d = float(np.max(np.abs(a - b))) if a.size else 0.0
    s = float(np.max(np.abs(b))) if b.size else 0.0
    return d / s if s > 0 else d
