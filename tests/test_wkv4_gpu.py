"""GPU parity of the v4 op against the fp64 oracle (which restates
RWKV-v4neo/cuda/wkv_cuda_bf16.cu) -- forward, backward, chained segments."""
import numpy as np
import pytest
import torch

import inputs
import wkv_testlib as TL
from oracle import wkv_oracle as O

pytestmark = pytest.mark.gpu


def _pkg():
    import rwkv_infctx_trainer_b200 as W
    return W


def v4_inputs(B, T, C, dtype, seed):
    c = inputs.wkv4_case(B, T, C, seed)
    q = {n: TL.rounded(c[n], dtype) for n in ("k", "v", "gy", "u")}
    q["td"] = TL.rounded(c["td"], torch.float32)
    q["w"] = -np.exp(q["td"])
    return q


def oracle_chain(q, seg):
    B, T, C = q["k"].shape
    s = np.zeros((B, C, 3)); s[..., 2] = -1e38
    bounds = [(t0, min(T, t0 + seg)) for t0 in range(0, T, seg)]
    states, ys = [s], []
    for t0, t1 in bounds:
        y, s = O.wkv4_fwd(q["w"], q["u"], q["k"][:, t0:t1], q["v"][:, t0:t1], states[-1])
        ys.append(y); states.append(s)
    gs, gk, gv, gw, gu = None, [], [], 0, 0
    for (t0, t1), s_in in reversed(list(zip(bounds, states[:-1]))):
        g = O.wkv4_bwd(q["w"], q["u"], q["k"][:, t0:t1], q["v"][:, t0:t1], s_in,
                       q["gy"][:, t0:t1], gs)
        gs = g["gstate_in"]
        gk.insert(0, g["gk"]); gv.insert(0, g["gv"]); gw = gw + g["gw"]; gu = gu + g["gu"]
    return dict(y=np.concatenate(ys, 1), state=states[-1], gk=np.concatenate(gk, 1),
                gv=np.concatenate(gv, 1), gw=gw.sum(0), gu=gu.sum(0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,C,seg", [(1, 1, 32, 1), (2, 17, 64, 17), (2, 64, 96, 32),
                                       (3, 100, 64, 33), (2, 256, 256, 128)])
def test_v4_op_chain_matches_oracle(dtype, B, T, C, seg):
    """torch.ops.rwkv.wkv over chained segments with autograd carrying (gp,gq,go)"""
    W = _pkg()
    q = v4_inputs(B, T, C, dtype, seed=40 + T)
    want = oracle_chain(q, seg)
    td = TL.to_dev(q["td"], torch.float32).requires_grad_(True)
    u = TL.to_dev(q["u"], dtype).requires_grad_(True)
    k = TL.to_dev(q["k"], dtype).requires_grad_(True)
    v = TL.to_dev(q["v"], dtype).requires_grad_(True)
    state = torch.zeros((B, C, 3), device="cuda"); state[..., 2] = -1e38
    ys = []
    for t0 in range(0, T, seg):
        t1 = min(T, t0 + seg)
        y, state = W.wkv_op(td, u, k[:, t0:t1], v[:, t0:t1], state)
        ys.append(y)
    y = torch.cat(ys, 1)
    (y.float() * TL.to_dev(q["gy"], torch.float32)).sum().backward()
    tol = TL.TOL[dtype]
    TL.assert_close("y", y, want["y"], tol)
    TL.assert_close("gk", k.grad, want["gk"], tol)
    TL.assert_close("gv", v.grad, want["gv"], tol)
    TL.assert_close("gw", td.grad, want["gw"], tol)
    TL.assert_close("gu", u.grad, want["gu"], tol)
    so = TL.back(state)
    # (p,q) are stored relative to the shared exponent o: compare the represented values
    TL.assert_close("state.p", so[..., 0] * np.exp(so[..., 2]),
                    want["state"][..., 0] * np.exp(want["state"][..., 2]), tol)
    TL.assert_close("state.q", so[..., 1] * np.exp(so[..., 2]),
                    want["state"][..., 1] * np.exp(want["state"][..., 2]), tol)


def test_v4_state_gradient_convention():
    """(gp,gq,go) out of the kernel, as consumed by the next-earlier segment, matches the oracle's
    when compared as represented values gp*e^go"""
    W = _pkg()
    import rwkv_infctx_trainer_b200._lib as L
    B, T, C = 2, 48, 64
    q = v4_inputs(B, T, C, torch.float32, seed=9)
    s0 = np.zeros((B, C, 3)); s0[..., 2] = -1e38
    _, s1 = O.wkv4_fwd(q["w"], q["u"], q["k"], q["v"], s0)
    gso = np.stack([inputs.normal((B, C), 9, stream=20), inputs.normal((B, C), 9, stream=21),
                    inputs.uniform((B, C), 9, -1, 1, stream=22)], -1)
    want = O.wkv4_bwd(q["w"], q["u"], q["k"], q["v"], s1, q["gy"], gso)
    d = {n: TL.to_dev(q[n], torch.float32) for n in ("w", "u", "k", "v", "gy")}
    si, go = TL.to_dev(s1, torch.float32), TL.to_dev(gso, torch.float32)
    gw = torch.empty((B, C), device="cuda"); gu = torch.empty_like(gw)
    gk = torch.empty_like(d["k"]); gv = torch.empty_like(d["k"]); gsi = torch.empty_like(si)
    lib = L.load()
    n = lib.wkv4_backward_workspace(B, T, C)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    L.check(lib.wkv4_backward(B, T, C, L.WKV_F32, d["w"].data_ptr(), d["u"].data_ptr(),
                              d["k"].data_ptr(), d["v"].data_ptr(), si.data_ptr(),
                              d["gy"].data_ptr(), go.data_ptr(), gw.data_ptr(), gu.data_ptr(),
                              gk.data_ptr(), gv.data_ptr(), gsi.data_ptr(), ws.data_ptr(), n,
                              torch.cuda.current_stream().cuda_stream), "wkv4_backward")
    torch.cuda.synchronize()
    tol = 1e-3
    TL.assert_close("gk", gk, want["gk"], tol)
    TL.assert_close("gv", gv, want["gv"], tol)
    TL.assert_close("gw", gw, want["gw"], tol)
    TL.assert_close("gu", gu, want["gu"], tol)
    g, w_ = TL.back(gsi), want["gstate_in"]
    TL.assert_close("gp", g[..., 0] * np.exp(g[..., 2]), w_[..., 0] * np.exp(w_[..., 2]), tol)
    TL.assert_close("gq", g[..., 1] * np.exp(g[..., 2]), w_[..., 1] * np.exp(w_[..., 2]), tol)


def test_v4_workspace_too_small_is_an_error():
    import rwkv_infctx_trainer_b200._lib as L
    lib = L.load()
    t = torch.zeros(64, device="cuda")
    p = t.data_ptr()
    code = lib.wkv4_backward(1, 32, 4, L.WKV_F32, p, p, p, p, None, p, None, p, p, p, p, None,
                             p, 8, None)
    assert code == 5


def test_v4_op_called_from_torchscript():
    """RWKV-v4neo/src/model.py:266-279 reaches torch.ops.rwkv.wkv from inside a
    torch.jit.script method; the registered op must resolve there, forward and backward"""
    W = _pkg()
    B, T, C = 2, 40, 64
    q = v4_inputs(B, T, C, torch.bfloat16, seed=5)

    @torch.jit.script
    def scripted(td: torch.Tensor, u: torch.Tensor, k: torch.Tensor, v: torch.Tensor, s: torch.Tensor):
        out = torch.ops.rwkv.wkv(td, u, k, v, s)
        return out[0], out[1]

    td = TL.to_dev(q["td"], torch.float32).requires_grad_(True)
    u, k, v = (TL.to_dev(q[n], torch.bfloat16).requires_grad_(True) for n in ("u", "k", "v"))
    s0 = torch.zeros((B, C, 3), device="cuda"); s0[..., 2] = -1e38
    y, s1 = scripted(td, u, k, v, s0)
    (y.float() * TL.to_dev(q["gy"], torch.float32)).sum().backward()
    want = oracle_chain(q, T)
    tol = TL.TOL[torch.bfloat16]
    TL.assert_close("y", y, want["y"], tol)
    TL.assert_close("gk", k.grad, want["gk"], tol)
    TL.assert_close("gv", v.grad, want["gv"], tol)
    TL.assert_close("gw", td.grad, want["gw"], tol)
    TL.assert_close("gu", u.grad, want["gu"], tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_v4_handover_equals_recompute(dtype):
    """backward given the tile checkpoints that forward left (no forward sweeps) against backward
    rebuilding everything itself: two code paths, the same numbers up to summation order, and
    both at the oracle"""
    import rwkv_infctx_trainer_b200._lib as L
    lib = L.load()
    B, T, C = 2, 300, 128
    q = v4_inputs(B, T, C, dtype, seed=13)
    d = {n: TL.to_dev(q[n], dtype) for n in ("u", "k", "v", "gy")}
    w = TL.to_dev(q["w"], torch.float32)
    s0 = torch.zeros((B, C, 3), device="cuda"); s0[..., 2] = -1e38
    st, code = torch.cuda.current_stream().cuda_stream, L.DTYPE_CODE[dtype]
    nf, nb, nck = lib.wkv4_forward_workspace(B, T, C), lib.wkv4_backward_workspace(B, T, C), lib.wkv4_state_ckpt_bytes(B, T, C)
    assert nck > 0 and lib.wkv4_state_ckpt_bytes(B, 100, C) == 0
    wsf, wsb = torch.empty(nf, dtype=torch.uint8, device="cuda"), torch.empty(nb, dtype=torch.uint8, device="cuda")
    ck = torch.empty(nck, dtype=torch.uint8, device="cuda")
    y, s1 = torch.empty_like(d["k"]), torch.empty_like(s0)
    L.check(lib.wkv4_forward_ckpt(B, T, C, code, w.data_ptr(), d["u"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(),
                                  s0.data_ptr(), y.data_ptr(), s1.data_ptr(), wsf.data_ptr(), nf, ck.data_ptr(), nck, st), "fwd")
    outs = []
    for ckp, n in ((ck.data_ptr(), nck), (None, 0)):
        gw, gu = torch.empty((B, C), device="cuda"), torch.empty((B, C), device="cuda")
        gk, gv, gsi = torch.empty_like(d["k"]), torch.empty_like(d["k"]), torch.empty_like(s0)
        L.check(lib.wkv4_backward_ckpt(B, T, C, code, w.data_ptr(), d["u"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(),
                                       s0.data_ptr(), d["gy"].data_ptr(), None, gw.data_ptr(), gu.data_ptr(), gk.data_ptr(),
                                       gv.data_ptr(), gsi.data_ptr(), wsb.data_ptr(), nb, ckp, n, st), "bwd")
        outs.append((gw, gu, gk, gv, gsi))
    torch.cuda.synchronize()
    tol = TL.TOL[dtype]
    s0n = np.zeros((B, C, 3)); s0n[..., 2] = -1e38
    want = O.wkv4_bwd(q["w"], q["u"], q["k"], q["v"], s0n, q["gy"], None)
    for got in outs:
        for n, a in zip(("gw", "gu", "gk", "gv"), got):
            TL.assert_close(n, a, want[n], tol)
    for n, a, b in zip(("gw", "gu", "gk", "gv"), *outs):
        TL.assert_close(n + " (hand-over vs rebuilt)", a, TL.back(b), tol)
    for i in (0, 1):      # (gp,gq,go) stands for (gp,gq)*e^go
        x, y = (TL.back(o[4]) for o in outs)
        TL.assert_close("gstate_in", x[..., i] * np.exp(x[..., 2]), y[..., i] * np.exp(y[..., 2]), tol)
