"""The CPU oracle against the reference's own outputs (fixtures in tests/golden/,
made from the project's rwkv_inner) and against closed-form definitions."""
import ast
import os

import numpy as np
import pytest
import torch

import inputs
from oracle import wkv_oracle as O
from oracle import wkv_chunked_port as P

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CASES = ["v5_small", "v6_small", "v5_config0", "v6_config0shape"]


def load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = ast.literal_eval(str(z["meta"]))
    return meta, {k: z[k] for k in z.files if k != "meta"}


def f32(a):
    """The fixtures were made from float32 inputs."""
    return np.asarray(a, dtype=np.float32).astype(np.float64)


W_FLOOR = 0.005  # rwkv_inner clamps the decay there (RWKV-v6/src/module/rwkv_inner.py:40-45)


def _v6_fwd_clamped(r, k, v, x, u, s):
    return O.wkv6_fwd(r, k, v, np.maximum(np.exp(-np.exp(x)), W_FLOOR), u, s)


def _v6_bwd_clamped(r, k, v, x, u, s, gy, gs):
    lw = -np.exp(x)
    w = np.exp(lw)
    out = O.wkv6_bwd(r, k, v, np.maximum(w, W_FLOOR), u, s, gy, gs)
    out["gw"] = out.pop("gwdec") * w * lw * (w >= W_FLOOR)   # clamp passes no gradient
    return out


def oracle_chain(meta, case):
    """Naive fp64 recurrence over BPTT segments: forward carrying state, then
    backward in reverse carrying the state gradient.  For v6 the decay is
    clamped the way rwkv_inner clamps it, so the comparison is like for like
    (the unclamped recurrence is what the CUDA kernels are held to)."""
    v, seg, T = meta["variant"], meta["seg_len"], meta["T"]
    fwd = _v6_fwd_clamped if v == "v6" else O.wkv5_fwd_x
    bwd = _v6_bwd_clamped if v == "v6" else O.wkv5_bwd_x
    c = {k: f32(a) for k, a in case.items()}
    xs = (lambda a, t0, t1: a[:, t0:t1]) if v == "v6" else (lambda a, t0, t1: a)
    states = [c["state_in"]]
    ys = []
    bounds = [(t0, min(T, t0 + seg)) for t0 in range(0, T, seg)]
    for t0, t1 in bounds:
        y, s = fwd(c["r"][:, t0:t1], c["k"][:, t0:t1], c["v"][:, t0:t1], xs(c["x"], t0, t1),
                   c["u"], states[-1])
        ys.append(y); states.append(s)
    out = dict(y=np.concatenate(ys, 1), state_out=states[-1])
    gs = c["gstate_out"]
    parts = {n: [] for n in ("gr", "gk", "gv")}
    gw_parts, gu = [], 0
    for (t0, t1), s_in in reversed(list(zip(bounds, states[:-1]))):
        g = bwd(c["r"][:, t0:t1], c["k"][:, t0:t1], c["v"][:, t0:t1], xs(c["x"], t0, t1),
                c["u"], s_in, c["gy"][:, t0:t1], gs)
        gs = g["gstate_in"]
        for n in parts:
            parts[n].insert(0, g[n])
        gw_parts.insert(0, g["gw"]); gu = gu + g["gu"]
    for n in parts:
        out[n] = np.concatenate(parts[n], 1)
    H, N = meta["H"], meta["N"]
    out["gw"] = np.concatenate(gw_parts, 1) if v == "v6" else sum(gw_parts).sum(0).reshape(H, N)
    out["gu"] = gu.sum(0).reshape(H, N)
    out["gstate_in"] = gs
    return out


def strided(meta, name, a):
    s = meta["stride"]
    if s > 1 and (name in ("y", "gr", "gk", "gv") or (name == "gw" and meta["variant"] == "v6")):
        return a[:, ::s]
    return a


@pytest.mark.parametrize("name", CASES)
def test_naive_oracle_matches_reference_rwkv_inner(name):
    meta, gold = load(name)
    case = inputs.wkv56_case(meta["variant"], meta["B"], meta["T"], meta["H"], meta["N"],
                             meta["seed"], state=meta["state"], gstate=meta["gstate"])
    out = oracle_chain(meta, case)
    for n, ref in gold.items():
        err = O.max_rel_err(strided(meta, n, out[n]), ref)
        # rwkv_inner works in fp32 with fp64 decay factors; 2e-5 leaves room for that
        assert err < 2e-5, (name, n, err)


@pytest.mark.parametrize("name", CASES)
def test_chunked_port_matches_reference_rwkv_inner(name):
    meta, gold = load(name)
    case = inputs.wkv56_case(meta["variant"], meta["B"], meta["T"], meta["H"], meta["N"],
                             meta["seed"], state=meta["state"], gstate=meta["gstate"])
    t = {k: torch.tensor(a, dtype=torch.float32) for k, a in case.items()}
    out = P.run_chain(meta["variant"], t["r"], t["k"], t["v"], t["x"], t["u"], t["state_in"],
                      t["gy"], meta["seg_len"], t["gstate_out"])
    for n, ref in gold.items():
        err = O.max_rel_err(strided(meta, n, out[n].numpy()), ref)
        assert err < 2e-5, (name, n, err)


def test_chunked_port_single_token_branch():
    c = inputs.wkv56_case("v6", 2, 1, 2, 64, 5)
    t = {k: torch.tensor(a, dtype=torch.float32) for k, a in c.items()}
    out = P.run_chain("v6", t["r"], t["k"], t["v"], t["x"], t["u"], t["state_in"], t["gy"], 1,
                      t["gstate_out"])
    y, s = O.wkv6_fwd_x(f32(c["r"]), f32(c["k"]), f32(c["v"]), f32(c["x"]), f32(c["u"]),
                        f32(c["state_in"]))
    assert O.max_rel_err(out["y"].numpy(), y) < 1e-5
    assert O.max_rel_err(out["state_out"].numpy(), s) < 1e-5


def _v4_definition(td, u, k, v, p0, q0, o0):
    """Closed-form v4 output under autograd (fp64): explicit sums, no scan.
    y_t = (e^{o0 + t w} p0 + sum_{i<t} e^{(t-1-i)w + k_i} v_i + e^{u+k_t} v_t) / (same, v=1)."""
    w = -torch.exp(td)
    B, T, C = k.shape
    ys = []
    for t in range(T):
        i = torch.arange(t)
        e = torch.exp((t - 1 - i).view(1, -1, 1) * w + k[:, :t])
        carry = torch.exp(o0 + t * w)
        num = carry * p0 + (e * v[:, :t]).sum(1) + torch.exp(u + k[:, t]) * v[:, t]
        den = carry * q0 + e.sum(1) + torch.exp(u + k[:, t])
        ys.append(num / den)
    i = torch.arange(T)
    e = torch.exp((T - 1 - i).view(1, -1, 1) * w + k)
    pT = torch.exp(o0 + T * w) * p0 + (e * v).sum(1)
    qT = torch.exp(o0 + T * w) * q0 + e.sum(1)
    return torch.stack(ys, 1), pT, qT


def test_v4_oracle_matches_closed_form_autograd():
    B, T, C = 2, 24, 8
    c = inputs.wkv4_case(B, T, C, seed=3)
    tt = {n: torch.tensor(a, dtype=torch.float64) for n, a in c.items()}
    # non-trivial carried state: true (p,q) = (p,q)*e^o
    p0 = torch.tensor(inputs.normal((B, C), 3, stream=9)).requires_grad_(True)
    q0 = torch.tensor(inputs.uniform((B, C), 3, 0.5, 2.0, stream=10)).requires_grad_(True)
    o0 = torch.tensor(inputs.uniform((B, C), 3, -1.0, 1.0, stream=11))
    td = tt["td"].clone().requires_grad_(True)
    u = tt["u"].clone().requires_grad_(True)
    k = tt["k"].clone().requires_grad_(True)
    v = tt["v"].clone().requires_grad_(True)
    y, pT, qT = _v4_definition(td, u, k, v, p0, q0, o0)
    # upstream gradient on the true final state (P,Q)
    GP = torch.tensor(inputs.normal((B, C), 3, stream=12))
    GQ = torch.tensor(inputs.normal((B, C), 3, stream=13))
    loss = (y * tt["gy"]).sum() + (pT * GP).sum() + (qT * GQ).sum()
    gtd, gu, gk, gv, gp0, gq0 = torch.autograd.grad(loss, [td, u, k, v, p0, q0])

    w = -np.exp(c["td"])
    state_in = np.stack([p0.detach().numpy(), q0.detach().numpy(), o0.numpy()], -1)
    yo, so = O.wkv4_fwd(w, c["u"], c["k"], c["v"], state_in)
    assert O.max_rel_err(yo, y.detach().numpy()) < 1e-12
    # stored state (p,q,o) represents (p,q)*e^o
    assert O.max_rel_err(so[..., 0] * np.exp(so[..., 2]), pT.detach().numpy()) < 1e-12
    assert O.max_rel_err(so[..., 1] * np.exp(so[..., 2]), qT.detach().numpy()) < 1e-12
    # the kernel's incoming state gradient (gp,gq,go) stands for d/d(stored p,q) = (gp,gq)*e^{go+o}
    # with o the state's own exponent: pass go = 0 and gp = GP (true grad w.r.t. P) since
    # dL/d(stored p) = GP * e^o  =>  gp * e^{go + o} with gp = GP, go = 0.
    gso = np.stack([GP.numpy(), GQ.numpy(), np.zeros((B, C))], -1)
    g = O.wkv4_bwd(w, c["u"], c["k"], c["v"], state_in, c["gy"], gso)
    assert O.max_rel_err(g["gk"], gk.numpy()) < 1e-11
    assert O.max_rel_err(g["gv"], gv.numpy()) < 1e-11
    assert O.max_rel_err(g["gu"].sum(0), gu.numpy()) < 1e-11
    assert O.max_rel_err(g["gw"].sum(0), gtd.numpy()) < 1e-11
    gsi = g["gstate_in"]
    # dL/d(stored p0) = gp * e^{go + o0}; autograd gives dL/dp0 of p0*e^{o0} w.r.t. p0 = same thing
    assert O.max_rel_err(gsi[..., 0] * np.exp(gsi[..., 2] + o0.numpy()), gp0.numpy()) < 1e-11
    assert O.max_rel_err(gsi[..., 1] * np.exp(gsi[..., 2] + o0.numpy()), gq0.numpy()) < 1e-11


def test_v4_oracle_chain_equals_single_pass():
    """Two chained segments (state forward, (gp,gq,go) backward) == one long segment."""
    B, T, C = 2, 64, 16
    c = inputs.wkv4_case(B, T, C, seed=4)
    w = -np.exp(c["td"])
    s0 = np.zeros((B, C, 3)); s0[..., 2] = -1e38
    y, sT = O.wkv4_fwd(w, c["u"], c["k"], c["v"], s0)
    g = O.wkv4_bwd(w, c["u"], c["k"], c["v"], s0, c["gy"], None)
    h = T // 2
    y1, s1 = O.wkv4_fwd(w, c["u"], c["k"][:, :h], c["v"][:, :h], s0)
    y2, s2 = O.wkv4_fwd(w, c["u"], c["k"][:, h:], c["v"][:, h:], s1)
    assert O.max_rel_err(np.concatenate([y1, y2], 1), y) < 1e-13
    g2 = O.wkv4_bwd(w, c["u"], c["k"][:, h:], c["v"][:, h:], s1, c["gy"][:, h:], None)
    g1 = O.wkv4_bwd(w, c["u"], c["k"][:, :h], c["v"][:, :h], s0, c["gy"][:, :h], g2["gstate_in"])
    assert O.max_rel_err(np.concatenate([g1["gk"], g2["gk"]], 1), g["gk"]) < 1e-12
    assert O.max_rel_err(np.concatenate([g1["gv"], g2["gv"]], 1), g["gv"]) < 1e-12
    assert O.max_rel_err(g1["gw"] + g2["gw"], g["gw"]) < 1e-12
    assert O.max_rel_err(g1["gu"] + g2["gu"], g["gu"]) < 1e-12
