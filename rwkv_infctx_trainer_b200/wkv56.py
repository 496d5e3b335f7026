"""Shared host code of the v5 and v6 ops: fills the C-ABI argument block."""
from __future__ import annotations

import ctypes

import torch

from . import _lib as L

HEAD_SIZE = 64

# The chunked kernels keep a status word at the start of their workspace: non-zero means that a
# bounded device-side wait ran out, the kernel gave up, and its outputs are invalid.  Every call
# copies that word to pinned host memory (on a side stream, without synchronising); the copies
# that have completed are looked at when the next v5/v6 call (forward or backward) on that device
# starts, and ``poll_status()`` looks at them on demand.  A non-zero word raises there.
# With CHECK_STATUS = True every call synchronises and checks its own word before returning
# (tests do that).
CHECK_STATUS = False

_pending = {}      # device index -> list of (event, pinned int32 tensor, description)
_side_streams = {}  # device index -> stream the status words are copied on


def poll_status(device=None, wait=False):
    """Raise if a chunked-kernel call on ``device`` (default: all devices) reported a device-side
    wait that ran out.  ``wait=True`` first waits for the calls issued so far."""
    keys = list(_pending) if device is None else [torch.device(device).index or 0]
    for key in keys:
        still = []
        for ev, word, what in _pending.get(key, []):
            if wait:
                ev.synchronize()
            if ev.query():
                code = int(word.item())
                if code != 0:
                    _pending[key] = []
                    raise RuntimeError(f"{what}: a device-side wait ran out (status {code}); "
                                       "the outputs of that call are invalid")
            else:
                still.append((ev, word, what))
        _pending[key] = still


def _watch_status(lib, a, variant, ws, what):
    if ws is None or ws.numel() < 4 or not lib.wkv56_uses_chunked(ctypes.byref(a), int(variant == "wkv6")):
        return
    if CHECK_STATUS:
        torch.cuda.synchronize(ws.device)
        code = int(ws[:4].view(torch.int32).item())
        if code != 0:
            raise RuntimeError(f"{what}: a device-side wait ran out (status {code})")
        return
    key = ws.device.index or 0
    side = _side_streams.get(key)
    if side is None:
        side = _side_streams[key] = torch.cuda.Stream(ws.device)
    # the copy runs on a side stream so that it never sits between two kernels of the caller's stream
    done = torch.cuda.Event()
    done.record(torch.cuda.current_stream(ws.device))
    word = torch.empty(1, dtype=torch.int32, pin_memory=True)
    with torch.cuda.stream(side):
        side.wait_event(done)
        word.copy_(ws[:4].view(torch.int32), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(side)
    ws.record_stream(side)
    _pending.setdefault(key, []).append((ev, word, what))


def _check_layout(B, T, C, **tensors):
    """the kernels take raw pointers: every [B,T,C] tensor must be exactly that, contiguous"""
    for name, t in tensors.items():
        if t is None:
            continue
        if tuple(t.shape) != (B, T, C):
            raise ValueError(f"{name} must have shape {(B, T, C)}, got {tuple(t.shape)}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous (a [:, t0:t1] view of a longer tensor is not)")


def _args(variant, B, T, H, dtype, w_kind, layout, path, time_groups=0, **t) -> L.WkvArgs:
    a = L.WkvArgs()
    a.B, a.T, a.H, a.N = B, T, H, HEAD_SIZE
    a.dtype, a.w_kind, a.state_layout, a.path = L.DTYPE_CODE[dtype], w_kind, layout, path
    a.time_groups = time_groups
    for name, tensor in t.items():
        setattr(a, name, L.ptr(tensor))
    return a


def _with_workspace(lib, variant, direction, a, dev):
    nbytes = getattr(lib, f"{variant}_{direction}_workspace")(ctypes.byref(a))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
    a.workspace, a.workspace_bytes = L.ptr(ws), nbytes
    return ws


def forward(variant: str, r, k, v, w, u, state_in, *, w_kind, layout=L.WKV_STATE_KV,
            path=L.WKV_PATH_AUTO, state_out=None, save_ckpt=False, time_groups=0, saved=None):
    """Launch wkv5_forward / wkv6_forward.  All tensors contiguous, on one device.
    Returns (y, state_out); ``state_out`` may be given (it may be ``state_in`` itself).
    With ``save_ckpt`` a third value is returned: the chunk-start states to hand to
    ``backward(..., ckpt=...)`` (None when the call did not run on the chunked kernels).
    ``time_groups``: see ``wkv_args_t.time_groups`` (0 = the library decides).
    ``saved``: a ``SavedStates``; empty, the call fills it; filled (by a call with the same
    inputs), the call restarts from it instead of scanning over T."""
    B, T, C = r.shape
    H = C // HEAD_SIZE
    dev = L.require_cuda(r, k, v, w, u, state_in)
    _check_layout(B, T, C, r=r, k=k, v=v, w=w if variant == "wkv6" else None)
    for name, t in (("u", u), ("state_in", state_in), ("state_out", state_out)):
        if t is not None and not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    poll_status(dev)
    y = torch.empty_like(r)
    if state_out is None:
        state_out = torch.empty((B, H, HEAD_SIZE, HEAD_SIZE), device=dev, dtype=torch.float32)
    lib = L.load()
    with torch.cuda.device(dev):
        a = _args(variant, B, T, H, r.dtype, w_kind, layout, path, time_groups, r=r, k=k, v=v, w=w,
                  u=u, state_in=state_in, y=y, state_out=state_out)
        ckpt = None
        if save_ckpt:
            nck = lib.wkv56_state_ckpt_bytes(ctypes.byref(a), int(variant == "wkv6"))
            if nck:
                ckpt = torch.empty(nck, dtype=torch.uint8, device=dev)
                a.state_ckpt, a.state_ckpt_bytes = L.ptr(ckpt), nck
        if saved is not None and lib.wkv56_uses_chunked(ctypes.byref(a), int(variant == "wkv6")):
            saved._attach(lib, a, (variant, B, T, H, r.dtype, w_kind, layout), dev)
        ws = _with_workspace(lib, variant, "forward", a, dev)
        L.check(getattr(lib, f"{variant}_forward")(ctypes.byref(a), L.stream_handle(dev)),
                f"{variant}_forward")
        if saved is not None:
            saved._done(a, state_out)
        _watch_status(lib, a, variant, ws, f"{variant}_forward")
        del ws
    if save_ckpt:
        return y, state_out, ckpt
    return y, state_out


def backward(variant: str, r, k, v, w, u, state_in, gy, gstate_out, *, w_kind,
             layout=L.WKV_STATE_KV, path=L.WKV_PATH_AUTO, want_gstate=True, ckpt=None,
             time_groups=0):
    """Launch wkv5_backward / wkv6_backward.  Returns gr, gk, gv, gw, gu, gstate_in with
    gw = [B,T,C] (v6, activation dtype) or [B,C] fp32 per-batch partials (v5); gu [B,C] fp32."""
    B, T, C = r.shape
    H = C // HEAD_SIZE
    dev = L.require_cuda(r, k, v, w, u, state_in, gy, gstate_out)
    _check_layout(B, T, C, r=r, k=k, v=v, gy=gy, w=w if variant == "wkv6" else None)
    for name, t in (("u", u), ("state_in", state_in), ("gstate_out", gstate_out)):
        if t is not None and not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    poll_status(dev)
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
        a = _args(variant, B, T, H, r.dtype, w_kind, layout, path, time_groups, r=r, k=k, v=v, w=w,
                  u=u, state_in=state_in, gy=gy, gstate_out=gstate_out, gr=gr, gk=gk, gv=gv, gw=gw,
                  gu=gu, gstate_in=gsi)
        if ckpt is not None:
            a.state_ckpt, a.state_ckpt_bytes = L.ptr(ckpt), ckpt.numel()
        ws = _with_workspace(lib, variant, "backward", a, dev)
        L.check(getattr(lib, f"{variant}_backward")(ctypes.byref(a), L.stream_handle(dev)),
                f"{variant}_backward")
        _watch_status(lib, a, variant, ws, f"{variant}_backward")
        del ws
    return gr, gk, gv, gw, gu, gsi


class Prepared:
    """One v5/v6 forward or backward call with every buffer (outputs, workspace, hand-over)
    allocated up front.  ``run()`` only crosses the C ABI -- for a loop that calls the op with the
    same buffers every step and wants no allocation and no Python bookkeeping on the way.
    The tensors are attributes (``y``, ``state_out``, ``ckpt`` / ``gr`` ... ``gstate_in``).
    ``status()`` synchronises and returns the call's status word (0 = ok)."""

    def __init__(self, fn, what, args, dev, **tensors):
        self._fn, self._what, self._a, self._dev = fn, what, args, dev
        self.__dict__.update(tensors)

    def run(self):
        L.check(self._fn(ctypes.byref(self._a), L.stream_handle(self._dev)), self._what)

    def status(self) -> int:
        torch.cuda.synchronize(self._dev)
        ws = self.workspace
        return 0 if ws is None or ws.numel() < 4 else int(ws[:4].view(torch.int32).item())


def prepare_forward(variant, r, k, v, w, u, state_in, *, w_kind, layout=L.WKV_STATE_KV,
                    path=L.WKV_PATH_AUTO, state_out=None, save_ckpt=True, time_groups=0) -> Prepared:
    B, T, C = r.shape
    H = C // HEAD_SIZE
    dev = L.require_cuda(r, k, v, w, u, state_in)
    _check_layout(B, T, C, r=r, k=k, v=v, w=w if variant == "wkv6" else None)
    lib = L.load()
    y = torch.empty_like(r)
    if state_out is None:
        state_out = torch.empty((B, H, HEAD_SIZE, HEAD_SIZE), device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        a = _args(variant, B, T, H, r.dtype, w_kind, layout, path, time_groups, r=r, k=k, v=v, w=w,
                  u=u, state_in=state_in, y=y, state_out=state_out)
        ckpt = None
        if save_ckpt:
            nck = lib.wkv56_state_ckpt_bytes(ctypes.byref(a), int(variant == "wkv6"))
            if nck:
                ckpt = torch.empty(nck, dtype=torch.uint8, device=dev)
                a.state_ckpt, a.state_ckpt_bytes = L.ptr(ckpt), nck
        ws = _with_workspace(lib, variant, "forward", a, dev)
    keep = (r, k, v, w, u, state_in)
    return Prepared(getattr(lib, f"{variant}_forward"), f"{variant}_forward", a, dev, y=y,
                    state_out=state_out, ckpt=ckpt, workspace=ws, _keep=keep)


def prepare_backward(variant, r, k, v, w, u, state_in, gy, gstate_out, *, w_kind,
                     layout=L.WKV_STATE_KV, path=L.WKV_PATH_AUTO, ckpt=None, gstate_in=None,
                     want_gstate=True, time_groups=0) -> Prepared:
    B, T, C = r.shape
    H = C // HEAD_SIZE
    dev = L.require_cuda(r, k, v, w, u, state_in, gy, gstate_out)
    _check_layout(B, T, C, r=r, k=k, v=v, gy=gy, w=w if variant == "wkv6" else None)
    lib = L.load()
    gr, gk, gv = torch.empty_like(r), torch.empty_like(r), torch.empty_like(r)
    gw = torch.empty_like(r) if variant == "wkv6" else torch.empty((B, C), device=dev, dtype=torch.float32)
    gu = torch.empty((B, C), device=dev, dtype=torch.float32)
    if gstate_in is None and want_gstate:
        gstate_in = torch.empty((B, H, HEAD_SIZE, HEAD_SIZE), device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        a = _args(variant, B, T, H, r.dtype, w_kind, layout, path, time_groups, r=r, k=k, v=v, w=w,
                  u=u, state_in=state_in, gy=gy, gstate_out=gstate_out, gr=gr, gk=gk, gv=gv, gw=gw,
                  gu=gu, gstate_in=gstate_in)
        if ckpt is not None:
            a.state_ckpt, a.state_ckpt_bytes = L.ptr(ckpt), ckpt.numel()
        ws = _with_workspace(lib, variant, "backward", a, dev)
    keep = (r, k, v, w, u, state_in, gy, gstate_out, ckpt)
    return Prepared(getattr(lib, f"{variant}_backward"), f"{variant}_backward", a, dev, gr=gr, gk=gk,
                    gv=gv, gw=gw, gu=gu, gstate_in=gstate_in, workspace=ws, _keep=keep)


class SavedStates:
    """What a forward call leaves for a later re-run of the SAME call (same inputs): the fp32
    state at the start of every 8th chunk (512 tokens) -- 16 KB per (batch, head) per 512 tokens.

    Made for activation checkpointing (RWKV-v6/src/model.py:657-665 wraps every block in
    ``deepspeed.checkpointing.checkpoint``): the block's forward runs once without autograd and
    once more, inside backward, to rebuild what autograd needs.  Keep one ``SavedStates`` per
    (layer, segment) outside the checkpointed function and pass it to the op in both runs: the
    first run fills it; the second finds it filled and starts every 8-chunk group from its stored
    state, all groups in parallel, with no serial pass over T -- and gives bit-identical y,
    state_out and hand-over.  ``clear()`` it when the inputs change (next training step)."""

    def __init__(self):
        self.clear()

    def clear(self):
        self.buf, self.key, self.filled, self.restarts = None, None, False, 0

    def _attach(self, lib, a, key, dev):
        n = lib.wkv56_group_states_bytes(ctypes.byref(a))
        if self.filled and self.key == key and self.buf is not None and self.buf.device == dev:
            a.group_states, a.group_states_bytes = L.ptr(self.buf), n
            a.group_states_mode = L.WKV_GROUP_STATES_USE
            self.restarts += 1
        else:
            self.buf = torch.empty(n, dtype=torch.uint8, device=dev)
            self.key, self.filled = key, False
            a.group_states, a.group_states_bytes = L.ptr(self.buf), n
            a.group_states_mode = L.WKV_GROUP_STATES_SAVE

    def _done(self, a, state_out):
        if a.group_states_mode == L.WKV_GROUP_STATES_SAVE:
            self.filled = True
