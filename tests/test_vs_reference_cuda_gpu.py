"""Our kernels against the RWKV-infctx-trainer project's own CUDA kernels, compiled
unchanged for sm_100a by oracle/build.py into oracle/_ref/ (prebuilt; skipped when
absent).  Only inputs on which those kernels are right are used: v4 anything; v5
forward with B == 1 or zero state, backward with zero state; v6 with B == 1."""
import ctypes
import os

import numpy as np
import pytest
import torch

import wkv_testlib as TL
from oracle import build as OB

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
TOL = 2e-2


def _ref(name):
    path = os.path.join(OB.REF_DIR, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} not prebuilt")
    return ctypes.CDLL(path)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _pkg():
    import rwkv_infctx_trainer_b200 as W
    return W


def test_v4_matches_reference_kernels_two_chained_segments():
    W = _pkg()
    lib = _ref("libref_wkv4.so")
    import test_wkv4_gpu as V4
    B, T, C, seg = 2, 256, 256, 128
    q = V4.v4_inputs(B, T, C, BF, seed=77)
    w = TL.to_dev(q["w"], torch.float32)
    u, k, v, gy = (TL.to_dev(q[n], BF) for n in ("u", "k", "v", "gy"))
    # reference: forward seg 0, seg 1; backward seg 1, seg 0
    s0 = torch.zeros((B, C, 3), device="cuda"); s0[..., 2] = -1e38
    ks, vs, gys = [k[:, :seg].contiguous(), k[:, seg:].contiguous()], \
        [v[:, :seg].contiguous(), v[:, seg:].contiguous()], \
        [gy[:, :seg].contiguous(), gy[:, seg:].contiguous()]
    ry = [torch.empty_like(ks[0]), torch.empty_like(ks[1])]
    s1, s2 = torch.empty_like(s0), torch.empty_like(s0)
    lib.ref_wkv4_forward(B, seg, C, _p(w), _p(u), _p(ks[0]), _p(vs[0]), _p(s0), _p(ry[0]), _p(s1))
    lib.ref_wkv4_forward(B, seg, C, _p(w), _p(u), _p(ks[1]), _p(vs[1]), _p(s1), _p(ry[1]), _p(s2))
    mk = lambda *s: torch.empty(s, device="cuda", dtype=BF)
    rgw, rgu = [mk(B, C), mk(B, C)], [mk(B, C), mk(B, C)]
    rgk, rgv = [mk(B, seg, C), mk(B, seg, C)], [mk(B, seg, C), mk(B, seg, C)]
    g1, g0 = torch.empty_like(s0), torch.empty_like(s0)
    lib.ref_wkv4_backward(B, seg, C, _p(w), _p(u), _p(ks[1]), _p(vs[1]), _p(s1), _p(gys[1]), None,
                          _p(rgw[1]), _p(rgu[1]), _p(rgk[1]), _p(rgv[1]), _p(g1))
    lib.ref_wkv4_backward(B, seg, C, _p(w), _p(u), _p(ks[0]), _p(vs[0]), _p(s0), _p(gys[0]),
                          _p(g1), _p(rgw[0]), _p(rgu[0]), _p(rgk[0]), _p(rgv[0]), _p(g0))
    torch.cuda.synchronize()
    # ours through the op
    td = TL.to_dev(q["td"], torch.float32).requires_grad_(True)
    uu, kk, vv = (t.clone().requires_grad_(True) for t in (u, k, v))
    state = s0.clone()
    ys = []
    for t0 in (0, seg):
        y, state = W.wkv_op(td, uu, kk[:, t0:t0 + seg], vv[:, t0:t0 + seg], state)
        ys.append(y)
    y = torch.cat(ys, 1)
    (y.float() * gy.float()).sum().backward()
    TL.assert_close("y", y, TL.back(torch.cat(ry, 1)), TOL)
    TL.assert_close("gk", kk.grad, TL.back(torch.cat(rgk, 1)), TOL)
    TL.assert_close("gv", vv.grad, TL.back(torch.cat(rgv, 1)), TOL)
    TL.assert_close("gw", td.grad, TL.back((rgw[0].float() + rgw[1].float()).sum(0)), TOL)
    TL.assert_close("gu", uu.grad, TL.back((rgu[0].float() + rgu[1].float()).sum(0)), TOL)
    a, b = TL.back(state), TL.back(s2)
    TL.assert_close("p", a[..., 0] * np.exp(a[..., 2]), b[..., 0] * np.exp(b[..., 2]), TOL)
    TL.assert_close("q", a[..., 1] * np.exp(a[..., 2]), b[..., 1] * np.exp(b[..., 2]), TOL)


@pytest.mark.parametrize("dtype", [BF, torch.float32])
def test_v5_matches_reference_kernels(dtype):
    W = _pkg()
    from rwkv_infctx_trainer_b200 import wkv56
    lib = _ref("libref_wkv5.so")
    tol = TL.TOL[dtype]
    is_bf16 = int(dtype == BF)
    H = 2
    C = H * 64
    # forward, B == 1, non-zero state, [value,key] layout, state updated in place
    q = TL.case56("v5", 1, 192, H, dtype, seed=61)
    r, k, v, u, gy = (TL.to_dev(q[n], dtype) for n in ("r", "k", "v", "u", "gy"))
    ew = TL.to_dev(-np.exp(q["x"]), torch.float32)
    eew = torch.exp(ew)
    s_ref = TL.to_dev(np.swapaxes(q["state_in"], -1, -2), torch.float32)
    s_our = s_ref.clone()
    y_ref = torch.empty_like(r)
    lib.ref_wkv5_forward(is_bf16, 1, 192, C, H, _p(s_ref), _p(r), _p(k), _p(v), _p(eew), _p(u),
                         _p(y_ref))
    torch.cuda.synchronize()
    y, _ = wkv56.forward("wkv5", r, k, v, ew, u, s_our, w_kind=W.WKV_W_NEGEXP,
                         layout=W.WKV_STATE_VK, state_out=s_our)
    TL.assert_close("y", y, TL.back(y_ref), tol)
    TL.assert_close("state", s_our, TL.back(s_ref), tol)
    # backward, B == 2, zero state (the reference kernel's valid domain)
    B, T = 2, 160
    q = TL.case56("v5", B, T, H, dtype, seed=62, state=False, gstate=False)
    r, k, v, u, gy = (TL.to_dev(q[n], dtype) for n in ("r", "k", "v", "u", "gy"))
    ew = TL.to_dev(-np.exp(q["x"]), torch.float32)
    eew = torch.exp(ew)
    zero = torch.zeros((B, H, 64, 64), device="cuda")
    mk = lambda *s: torch.empty(s, device="cuda", dtype=dtype)
    rgr, rgk, rgv, rgw, rgu = mk(B, T, C), mk(B, T, C), mk(B, T, C), mk(B, C), mk(B, C)
    lib.ref_wkv5_backward(is_bf16, B, T, C, H, _p(zero), _p(r), _p(k), _p(v), _p(eew), _p(ew),
                          _p(u), _p(gy), _p(rgr), _p(rgk), _p(rgv), _p(rgw), _p(rgu))
    torch.cuda.synchronize()
    gr, gk, gv, gw, gu, _ = wkv56.backward("wkv5", r, k, v, ew, u, zero, gy, None,
                                           w_kind=W.WKV_W_NEGEXP, layout=W.WKV_STATE_VK)
    TL.assert_close("gr", gr, TL.back(rgr), tol)
    TL.assert_close("gk", gk, TL.back(rgk), tol)
    TL.assert_close("gv", gv, TL.back(rgv), tol)
    TL.assert_close("gw", gw.sum(0), TL.back(rgw.float().sum(0)), tol)
    TL.assert_close("gu", gu.sum(0), TL.back(rgu.float().sum(0)), tol)


@pytest.mark.parametrize("path", ["scalar", "auto"])
def test_v6_matches_reference_state_kernels_b1(path):
    W = _pkg()
    from rwkv_infctx_trainer_b200 import wkv56
    lib = _ref("libref_wkv6state.so")
    p = W.WKV_PATH_SCALAR if path == "scalar" else W.WKV_PATH_AUTO
    H, T = 3, 256
    C = H * 64
    q = TL.case56("v6", 1, T, H, BF, seed=63, gstate=False)
    # every decay above the chunked kernels' 0.005 floor, so that both paths compute the same function
    q["x"] = TL.rounded(np.minimum(q["x"], 1.6), BF)
    r, k, v, u, gy = (TL.to_dev(q[n], BF) for n in ("r", "k", "v", "u", "gy"))
    # the literal lower-level call: ew = -exp(x) in fp32, from the bf16 activation (TimeMix.py:49-51)
    ew = (-torch.exp(TL.to_dev(q["x"], BF).float())).contiguous()
    a = wkv56._args("wkv6", 1, T, H, BF, W.WKV_W_NEGEXP, W.WKV_STATE_VK, p)
    from rwkv_infctx_trainer_b200 import _lib as L
    assert L.load().wkv56_uses_chunked(ctypes.byref(a), 1) == int(path == "auto")
    # both sides start from the same bf16-rounded state (the reference keeps state in bf16)
    s_bf = TL.to_dev(np.swapaxes(q["state_in"], -1, -2), BF)
    s_in32 = s_bf.float().contiguous()
    s_ref = s_bf.clone()
    y_ref = torch.empty_like(r)
    lib.ref_wkv6_forward(1, T, C, H, _p(r), _p(k), _p(v), _p(ew), _p(u), _p(s_ref), _p(y_ref))
    mk = lambda *s: torch.empty(s, device="cuda", dtype=BF)
    rgr, rgk, rgv, rgw, rgu, rgs = mk(1, T, C), mk(1, T, C), mk(1, T, C), mk(1, T, C), mk(1, C), \
        mk(1, H, 64, 64)
    lib.ref_wkv6_backward(1, T, C, H, _p(r), _p(k), _p(v), _p(ew), _p(u), _p(s_bf), _p(gy),
                          _p(rgr), _p(rgk), _p(rgv), _p(rgw), _p(rgu), _p(rgs))
    torch.cuda.synchronize()
    y, s_out = wkv56.forward("wkv6", r, k, v, ew, u, s_in32, w_kind=W.WKV_W_NEGEXP,
                             layout=W.WKV_STATE_VK, path=p)
    gr, gk, gv, gw, gu, gs = wkv56.backward("wkv6", r, k, v, ew, u, s_in32, gy, None,
                                            w_kind=W.WKV_W_NEGEXP, layout=W.WKV_STATE_VK, path=p)
    TL.assert_close("y", y, TL.back(y_ref), TOL)
    TL.assert_close("state", s_out, TL.back(s_ref), TOL)
    TL.assert_close("gr", gr, TL.back(rgr), TOL)
    TL.assert_close("gk", gk, TL.back(rgk), TOL)
    TL.assert_close("gv", gv, TL.back(rgv), TOL)
    TL.assert_close("gw", gw, TL.back(rgw), TOL)
    TL.assert_close("gu", gu, TL.back(rgu), TOL)
    TL.assert_close("gs", gs, TL.back(rgs), TOL)


def test_v6_stateless_alias_module():
    """the ``wkv6`` module of RWKV-v6/src/module/cuda/wkv6_op.cpp:8-22 (no state in, none out):
    equals the stateful call from a zero state"""
    W = _pkg()
    from rwkv_infctx_trainer_b200 import wkv56
    B, T, H = 2, 200, 2
    C = H * 64
    q = TL.case56("v6", B, T, H, BF, seed=65, state=False, gstate=False)
    r, k, v, u, gy = (TL.to_dev(q[n], BF) for n in ("r", "k", "v", "u", "gy"))
    ew = (-torch.exp(TL.to_dev(q["x"], BF).float())).contiguous()
    y = torch.empty_like(r)
    W.wkv6_cuda_kernel.forward(B, T, C, H, r, k, v, ew, u, y)
    mk = lambda *s: torch.empty(s, device="cuda", dtype=BF)
    gr, gk, gv, gw, gu = mk(B, T, C), mk(B, T, C), mk(B, T, C), mk(B, T, C), mk(B, C)
    W.wkv6_cuda_kernel.backward(B, T, C, H, r, k, v, ew, u, gy, gr, gk, gv, gw, gu)
    want = TL.oracle56("v6", q)
    TL.assert_close("y", y, want["y"], TOL)
    TL.assert_close("gr", gr, want["gr"], TOL)
    TL.assert_close("gk", gk, want["gk"], TOL)
    TL.assert_close("gv", gv, want["gv"], TOL)
    TL.assert_close("gw", gw, want["gw"], TOL)
    TL.assert_close("gu", gu, want["gu"], TOL)
