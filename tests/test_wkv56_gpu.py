"""GPU parity of the v5/v6 ops (through the package -> C ABI) against the fp64
oracle and the fixtures made from the reference's rwkv_inner.

Tolerances (max|ours-ref| / max|ref| per tensor): 1e-3 for fp32 I/O, 2e-2 for
bf16/fp16 I/O, on y, state_out and every gradient."""
import ast
import os

import numpy as np
import pytest
import torch

import inputs
import wkv_testlib as TL
from oracle import wkv_oracle as O

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _pkg():
    import rwkv_infctx_trainer_b200 as W
    return W


def run_abi(variant, q, dtype, layout, w_kind, path):
    """forward + backward through rwkv_infctx_trainer_b200.wkv56 (thin wrapper of the C ABI)"""
    W = _pkg()
    from rwkv_infctx_trainer_b200 import wkv56
    name = "wkv6" if variant == "v6" else "wkv5"
    d = {n: TL.to_dev(q[n], dtype) for n in ("r", "k", "v", "gy", "u")}
    x = q["x"]
    if w_kind == W.WKV_W_NEGEXP:
        w = TL.to_dev(-np.exp(x), torch.float32)
    else:
        w = TL.to_dev(x, dtype if variant == "v6" else torch.float32)
    tr = (lambda a: np.swapaxes(a, -1, -2)) if layout == W.WKV_STATE_VK else (lambda a: a)
    s_in = TL.to_dev(tr(q["state_in"]), torch.float32)
    gs_out = TL.to_dev(tr(q["gstate_out"]), torch.float32)
    y, s_out = wkv56.forward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, w_kind=w_kind,
                             layout=layout, path=path)
    gr, gk, gv, gw, gu, gsi = wkv56.backward(name, d["r"], d["k"], d["v"], w, d["u"], s_in,
                                             d["gy"], gs_out, w_kind=w_kind, layout=layout,
                                             path=path)
    torch.cuda.synchronize()
    return dict(y=y, state_out=tr(TL.back(s_out)), gr=gr, gk=gk, gv=gv, gw=gw, gu=gu,
                gstate_in=tr(TL.back(gsi)))


def compare(variant, got, want, dtype, q=None):
    tol = TL.TOL[dtype]
    errs = {}
    for n in ("y", "state_out", "gr", "gk", "gv", "gu", "gstate_in", "gw"):
        errs[n] = TL.assert_close(f"{variant}.{n}", got[n], want[n], tol)
    return errs


SHAPES = [(1, 1, 1), (1, 2, 1), (3, 15, 1), (1, 16, 2), (1, 17, 1), (2, 63, 1), (1, 64, 1),
          (1, 65, 3), (2, 129, 2), (1, 256, 1)]


@pytest.mark.parametrize("variant", ["v5", "v6"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,T,H", SHAPES)
def test_scalar_path_matches_oracle(variant, dtype, B, T, H):
    W = _pkg()
    q = TL.case56(variant, B, T, H, dtype, seed=100 + T)
    want = TL.oracle56(variant, q)
    got = run_abi(variant, q, dtype, W.WKV_STATE_KV, W.WKV_W_RAW, W.WKV_PATH_SCALAR)
    compare(variant, got, want, dtype)


@pytest.mark.parametrize("variant", ["v5", "v6"])
def test_scalar_path_reference_layout_and_negexp_decay(variant):
    """[value,key] state and the precomputed ew = -exp(x) that the project's Python wrappers pass"""
    W = _pkg()
    q = TL.case56(variant, 2, 96, 2, torch.float32, seed=7)
    want = TL.oracle56(variant, q)
    got = run_abi(variant, q, torch.float32, W.WKV_STATE_VK, W.WKV_W_NEGEXP, W.WKV_PATH_SCALAR)
    compare(variant, got, want, torch.float32)


@pytest.mark.parametrize("variant", ["v5", "v6"])
def test_zero_length_segment_passes_state_through(variant):
    """the v6 trainer issues T == 0 dummy segments (RWKV-v6/src/model.py:1164-1167)"""
    W = _pkg()
    from rwkv_infctx_trainer_b200 import wkv56
    B, H = 2, 2
    z = torch.zeros((B, 0, H * 64), device="cuda", dtype=torch.bfloat16)
    s = torch.randn((B, H, 64, 64), device="cuda")
    u = torch.zeros((H, 64), device="cuda", dtype=torch.bfloat16)
    w = z if variant == "v6" else torch.zeros((H, 64), device="cuda")
    y, so = wkv56.forward("wkv6" if variant == "v6" else "wkv5", z, z, z, w, u, s,
                          w_kind=W.WKV_W_RAW)
    assert y.shape == (B, 0, H * 64)
    assert torch.equal(so, s)


def test_zero_length_segment_inside_an_autograd_chain():
    """forward AND backward through a T == 0 segment between two real ones: the v6 trainer pads
    short documents with empty segments and back-propagates through them
    (RWKV-v6/src/model.py:1160-1167); state and state gradient must pass through unchanged"""
    W = _pkg()
    B, T, H = 2, 128, 2
    C = H * 64
    for variant, fn in (("v6", W.WKV6), ("v5", W.WKV5)):
        q = TL.case56(variant, B, T, H, torch.bfloat16, seed=71)
        mk = lambda n, dt: TL.to_dev(q[n], dt).requires_grad_(True)
        r, k, v, u = (mk(n, torch.bfloat16) for n in ("r", "k", "v", "u"))
        x = mk("x", torch.bfloat16 if variant == "v6" else torch.float32)
        s0 = mk("state_in", torch.float32)
        gy, gs = TL.to_dev(q["gy"], torch.bfloat16), TL.to_dev(q["gstate_out"], torch.float32)

        def chain(cuts):
            for t in (r, k, v, u, x, s0):
                t.grad = None
            state, ys = s0, []
            for t0, t1 in cuts:
                xs = x[:, t0:t1] if variant == "v6" else x
                y, state = fn.apply(B, t1 - t0, C, H, r[:, t0:t1], k[:, t0:t1], v[:, t0:t1], xs, u, state)
                ys.append(y)
            y = torch.cat(ys, 1)
            ((y.float() * gy.float()).sum() + (state * gs).sum()).backward()
            return [y.detach().clone(), state.detach().clone()] + [t.grad.clone() for t in (r, k, v, u, x, s0)]

        a = chain([(0, 64), (64, 128)])
        b = chain([(0, 64), (64, 64), (64, 128)])
        for p_, q_ in zip(a, b):
            assert torch.equal(p_, q_)


def _load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return ast.literal_eval(str(z["meta"])), {k: z[k] for k in z.files if k != "meta"}


@pytest.mark.parametrize("name", ["v5_small", "v6_small", "v5_config0", "v6_config0shape"])
@pytest.mark.parametrize("path", ["scalar"])
def test_autograd_chain_matches_reference_fixture(name, path):
    """BPTT the way the trainer does it: segments of seg_len with the state carried
    forward by the op's second output and its gradient carried back by autograd;
    compared with what the reference's rwkv_inner produced on the same inputs (fp32 tensors:
    the token-serial kernels; test_tensor_core_parity_gpu.py runs the same fixtures in bf16
    through the chunked kernels)."""
    W = _pkg()
    meta, gold = _load_golden(name)
    v, B, T, H, N, seg = (meta[k] for k in ("variant", "B", "T", "H", "N", "seg_len"))
    c = inputs.wkv56_case(v, B, T, H, N, meta["seed"], state=meta["state"], gstate=meta["gstate"])
    t = {n: torch.tensor(a, dtype=torch.float32, device="cuda") for n, a in c.items()}
    leaves = {n: t[n].clone().requires_grad_(True) for n in ("r", "k", "v", "x", "u", "state_in")}
    fn = W.WKV6 if v == "v6" else W.WKV5
    p = W.WKV_PATH_SCALAR if path == "scalar" else W.WKV_PATH_AUTO
    state = leaves["state_in"]
    ys = []
    for t0 in range(0, T, seg):
        t1 = min(T, t0 + seg)
        xs = leaves["x"][:, t0:t1] if v == "v6" else leaves["x"]
        y, state = fn.apply(B, t1 - t0, H * N, H, leaves["r"][:, t0:t1], leaves["k"][:, t0:t1],
                            leaves["v"][:, t0:t1], xs, leaves["u"], state, p)
        ys.append(y)
    y = torch.cat(ys, 1)
    loss = (y * t["gy"]).sum() + (state * t["gstate_out"]).sum()
    loss.backward()
    got = dict(y=y, state_out=state, gr=leaves["r"].grad, gk=leaves["k"].grad,
               gv=leaves["v"].grad, gw=leaves["x"].grad, gu=leaves["u"].grad,
               gstate_in=leaves["state_in"].grad)
    s = meta["stride"]
    for n, ref in gold.items():
        g = TL.back(got[n])
        if s > 1 and (n in ("y", "gr", "gk", "gv") or (n == "gw" and v == "v6")):
            g = g[:, ::s]
        # the fixture's two clamped decay elements (w < 0.005) sit in v6_config0shape: the
        # reference clamps, the kernels do not; 1e-3 still holds on every tensor but gw there
        tol = 1e-3
        e = O.max_rel_err(g, ref)
        if name == "v6_config0shape" and n == "gw":
            # exclude the clamped elements' own gradient (reference returns 0 for them)
            x = np.asarray(c["x"], dtype=np.float32)[:, ::s]
            mask = np.exp(-np.exp(x)) >= 0.005
            e = O.max_rel_err(g * mask, ref * mask)
        assert e <= tol, (name, n, e)


@pytest.mark.parametrize("variant", ["v5", "v6"])
def test_split_call_equals_single_call(variant):
    """size-independent property: one call over T tokens == two calls over T/2 with the
    state carried (forward) and the state gradient carried (backward)"""
    W = _pkg()
    dtype = torch.bfloat16
    B, T, H = 2, 512, 4
    q = TL.case56(variant, B, T, H, dtype, seed=21)
    one = run_abi(variant, q, dtype, W.WKV_STATE_KV, W.WKV_W_RAW, W.WKV_PATH_AUTO)
    h = T // 2
    def part(sl, s_in, gs_out):
        qq = dict(q)
        for n in ("r", "k", "v", "gy"):
            qq[n] = q[n][:, sl]
        if variant == "v6":
            qq["x"] = q["x"][:, sl]
        qq["state_in"], qq["gstate_out"] = s_in, gs_out
        return qq
    # forward first half, then second half from its state; backward in reverse
    a = run_abi(variant, part(slice(0, h), q["state_in"], np.zeros_like(q["gstate_out"])), dtype,
                W.WKV_STATE_KV, W.WKV_W_RAW, W.WKV_PATH_AUTO)
    b = run_abi(variant, part(slice(h, T), a["state_out"], q["gstate_out"]), dtype,
                W.WKV_STATE_KV, W.WKV_W_RAW, W.WKV_PATH_AUTO)
    a = run_abi(variant, part(slice(0, h), q["state_in"], b["gstate_in"]), dtype,
                W.WKV_STATE_KV, W.WKV_W_RAW, W.WKV_PATH_AUTO)
    tol = 2e-2
    cat = lambda n: np.concatenate([TL.back(a[n]), TL.back(b[n])], 1)
    for n in ("y", "gr", "gk", "gv"):
        TL.assert_close(n, cat(n), TL.back(one[n]), tol)
    TL.assert_close("state_out", b["state_out"], one["state_out"], tol)
    TL.assert_close("gstate_in", a["gstate_in"], one["gstate_in"], tol)
    TL.assert_close("gu", TL.back(a["gu"]) + TL.back(b["gu"]), TL.back(one["gu"]), tol)
    if variant == "v6":
        TL.assert_close("gw", cat("gw"), TL.back(one["gw"]), tol)
    else:
        TL.assert_close("gw", TL.back(a["gw"]) + TL.back(b["gw"]), TL.back(one["gw"]), tol)


def test_v6_strong_decay_stays_finite():
    """decay far below the reference's 0.005 clamp (x up to ~+3 => w ~ 1e-9): no Inf/NaN.  The
    token-serial path is held to the unclamped fp64 recurrence; the chunked path (what AUTO
    picks for bf16) floors the decay at 0.005 as the reference's rwkv_inner does and is held to
    the fp64 recurrence with that floor."""
    W = _pkg()
    import test_chunked_gpu as CG
    dtype = torch.bfloat16
    q = TL.case56("v6", 1, 192, 2, dtype, seed=33, x_shift=2.0)
    q["x"] = TL.rounded(q["x"], dtype)
    for path, want in ((W.WKV_PATH_SCALAR, TL.oracle56("v6", q)),
                       (W.WKV_PATH_AUTO, CG.floored_oracle("v6", q))):
        got = run_abi("v6", q, dtype, W.WKV_STATE_KV, W.WKV_W_RAW, path)
        for n, a in got.items():
            a = TL.back(a) if torch.is_tensor(a) else a
            assert np.isfinite(a).all(), n
        compare("v6", got, want, dtype)


def test_dropin_wrappers_v5_v6():
    """WKV5_CUDA / WKV6STATE_CUDA: the reference's Function signatures, in-place state in the
    kernels' [value,key] layout, per-batch state (B > 1)"""
    W = _pkg()
    B, T, H = 2, 80, 2
    C = H * 64
    for variant in ("v5", "v6"):
        dtype = torch.bfloat16
        q = TL.case56(variant, B, T, H, dtype, seed=55, gstate=False)
        want = TL.oracle56(variant, q)
        d = {n: TL.to_dev(q[n], dtype).requires_grad_(True) for n in ("r", "k", "v", "u")}
        s_vk = TL.to_dev(np.swapaxes(q["state_in"], -1, -2), torch.float32)
        if variant == "v5":
            w = TL.to_dev(q["x"], torch.float32).requires_grad_(True)
            y = W.RUN_WKV5_CUDA(B, T, C, H, s_vk, d["r"], d["k"], d["v"], w, d["u"])
        else:
            w = TL.to_dev(q["x"], dtype).requires_grad_(True)
            y = W.RUN_WKV6STATE_CUDA(B, T, C, H, d["r"], d["k"], d["v"], w, d["u"], s_vk)
        y.backward(TL.to_dev(q["gy"], dtype))
        tol = 2e-2
        TL.assert_close("y", y, want["y"], tol)
        TL.assert_close("state", np.swapaxes(TL.back(s_vk), -1, -2), want["state_out"], tol)
        TL.assert_close("gr", d["r"].grad, want["gr"], tol)
        TL.assert_close("gk", d["k"].grad, want["gk"], tol)
        TL.assert_close("gv", d["v"].grad, want["gv"], tol)
        TL.assert_close("gu", d["u"].grad, want["gu"].sum(0).reshape(H, 64), tol)
        gw_want = want["gw"] if variant == "v6" else want["gw"].sum(0).reshape(H, 64)
        TL.assert_close("gw", w.grad, gw_want, tol)


def test_bad_arguments_raise_not_crash():
    W = _pkg()
    from rwkv_infctx_trainer_b200 import wkv56
    z = torch.zeros((1, 4, 64), device="cuda", dtype=torch.bfloat16)
    s = torch.zeros((1, 1, 64, 64), device="cuda")
    with pytest.raises(RuntimeError):
        wkv56.forward("wkv6", z, z, z, z.cpu(), z[0, 0], s, w_kind=W.WKV_W_RAW)
    with pytest.raises(RuntimeError, match="chunked"):
        f = torch.zeros((1, 4, 64), device="cuda", dtype=torch.float32)
        wkv56.forward("wkv6", f, f, f, f, f[0, 0], s, w_kind=W.WKV_W_RAW, path=W.WKV_PATH_CHUNKED)
    torch.cuda.synchronize()
