"""TEST INFRASTRUCTURE ONLY -- CPU port of the project's pure-PyTorch WKV path.

A restatement, in our own code, of the chunked algorithm that
RWKV-infctx-trainer runs when its CUDA kernels are off (``RWKV_NO_CUDA=1``, the
project default): ``rwkv_inner`` in RWKV-v5/src/module/rwkv_inner.py:10-117 and
RWKV-v6/src/module/rwkv_inner.py:10-115 (the two files hold the same algorithm).
It is the CPU baseline that ``bench.py`` times beside the GPU numbers, and a
second checker in the tests.  The shipped package never imports it.

Steps followed (v6 file's line numbers):
  * decay clamp ``w >= 0.005`` and fp32 ``log``                        (:40-48)
  * per-chunk inclusive cumulative log-decay and its one-step shift    (:51-55)
  * whole-chunk decay, decay-to-chunk-end, decay-from-chunk-start      (:69-75)
  * intra-chunk scores with factors re-centred on the mid-chunk value,
    evaluated in fp64, strictly-lower-triangular, bonus ``u`` on the
    diagonal                                                            (:88-94)
  * per-chunk key/value outer products and the serial state scan       (:99-110)
  * contribution of the carried state to every token                   (:113)
  * single-token branch                                                 (:25-29)
Gradients come from autograd, exactly as in the project.

Parity pin: compared with the project's own ``rwkv_inner`` through the fixtures
in tests/golden/ (see tests/golden/make_golden.py).
"""
from __future__ import annotations

import torch

CHUNK_LEN = 128
W_FLOOR = 0.005


def wkv_chunked(r, k, v, w, u, state, chunk_len: int = CHUNK_LEN):
    """r,k,v: (B,H,L,N); w: (B|1,H,L,N) decay in (0,1]; u: (1,H,1,N);
    state: (B,H,N,N) [key,value].  Returns (out (B,H,L,N), new_state)."""
    B, H, L, N = k.shape
    if L == 1:
        outer = k.transpose(-1, -2) * v                  # (B,H,N,N)
        out = r @ (state + u.transpose(-1, -2) * outer)
        return out, w.transpose(-1, -2) * state + outer
    if L % chunk_len:
        raise ValueError("sequence length must be 1 or a multiple of chunk_len")
    G = L // chunk_len
    dt = r.dtype
    logw = w.clamp(min=W_FLOOR).float().log().reshape(w.shape[0], H, G, chunk_len, N)
    cum = logw.cumsum(3)                                  # inclusive
    cum_prev = cum - logw                                 # exclusive (= shifted cumsum)
    total = cum[:, :, :, -1:, :]                          # whole chunk
    to_end = (total - cum).exp().to(dt)                   # token s -> end of chunk
    from_start = cum_prev.exp().to(dt)                    # chunk start -> just before token t
    chunk_decay = total.exp().to(dt).squeeze(3)           # (B|1,H,G,N)

    rc = r.reshape(B, H, G, chunk_len, N)
    kc = k.reshape(B, H, G, chunk_len, N)
    vc = v.reshape(B, H, G, chunk_len, N)
    uu = u.reshape(1, H, 1, 1, N).to(dt)

    mid = cum_prev[:, :, :, chunk_len // 2:chunk_len // 2 + 1, :]
    rfac = (cum_prev - mid).double().exp()
    kfac = (mid - cum).double().exp()
    scores = torch.einsum("bhgtn,bhgsn->bhgts", rc * rfac, kc * kfac).to(dt).tril(-1)
    scores = scores + torch.diag_embed((rc * uu * kc).sum(-1))
    out = scores @ vc

    local = torch.einsum("bhgsn,bhgsm->bhgnm", kc * to_end, vc)   # (B,H,G,N,N)
    starts = []
    for g in range(G):
        starts.append(state)
        state = state * chunk_decay[:, :, g, :, None] + local[:, :, g]
    starts = torch.stack(starts, dim=2)
    out = out + (rc * from_start) @ starts
    return out.reshape(B, H, L, N), state


def run_chain(variant: str, r, k, v, x, u, state0, gy, seg_len: int, gstate_final=None):
    """Forward over consecutive BPTT segments carrying state, then one backward.

    r,k,v,gy: (B,T,C) fp32; x: (B,T,C) (v6) or (H,N) (v5) with decay
    ``exp(-exp(x))``; u: (H,N); state0: (B,H,N,N).  Returns dict of y,
    state_out and gradients w.r.t. r,k,v,x,u,state0 (the same contract the
    CUDA op offers)."""
    B, T, C = r.shape
    H, N = u.shape
    leaves = [t.clone().requires_grad_(True) for t in (r, k, v, x, u, state0)]
    r_, k_, v_, x_, u_, s_ = leaves
    w = torch.exp(-torch.exp(x_.float()))
    if variant == "v6":
        w4 = w.view(B, T, H, N).transpose(1, 2)
    else:
        w4 = None
    state = s_
    ys = []
    for t0 in range(0, T, seg_len):
        t1 = min(T, t0 + seg_len)
        sl = lambda a: a[:, t0:t1].reshape(B, t1 - t0, H, N).transpose(1, 2)
        if variant == "v6":
            ws = w4[:, :, t0:t1]
        else:
            ws = w.view(1, H, 1, N).expand(1, H, t1 - t0, N)
        o, state = wkv_chunked(sl(r_), sl(k_), sl(v_), ws, u_.view(1, H, 1, N), state)
        ys.append(o.transpose(1, 2).reshape(B, t1 - t0, C))
    y = torch.cat(ys, dim=1)
    loss = (y * gy).sum()
    if gstate_final is not None:
        loss = loss + (state * gstate_final).sum()
    grads = torch.autograd.grad(loss, leaves, allow_unused=True)
    names = ("gr", "gk", "gv", "gw", "gu", "gstate_in")
    out = {n: (g if g is not None else torch.zeros_like(l)) for n, g, l in zip(names, grads, leaves)}
    out["y"] = y.detach()
    out["state_out"] = state.detach()
    return out
