"""The tcgen05 chunked v5/v6 kernels (bf16) against the fp64 oracle.

The chunked kernels floor the decay at 0.005, the floor the reference's rwkv_inner applies
(RWKV-v6/src/module/rwkv_inner.py:40-45); the oracle is given the same floored decay, and the
gradient w.r.t. a floored decay element is zero (what autograd through the reference's clamp
gives).  With the benchmark's decay distribution the floor is hit about 3 times per million."""
import numpy as np
import pytest
import torch

import wkv_testlib as TL
from oracle import wkv_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
FLOOR = 0.005
# outputs held to the floored oracle in the decay-extremes test
EXTREME_CHECKED = ("y", "state_out", "gr", "gk", "gv", "gw", "gu", "gstate_in")


def _pkg():
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import wkv56
    wkv56.CHECK_STATUS = True
    return W, wkv56


def floored_oracle(variant, q):
    x = q["x"]
    lw = -np.exp(x)
    w = np.exp(lw)
    wf = np.maximum(w, FLOOR)
    live = w >= FLOOR
    if variant == "v6":
        y, so = O.wkv6_fwd(q["r"], q["k"], q["v"], wf, q["u"], q["state_in"])
        g = O.wkv6_bwd(q["r"], q["k"], q["v"], wf, q["u"], q["state_in"], q["gy"], q["gstate_out"])
        g["gw"] = g.pop("gwdec") * wf * np.log(wf) * live
    else:
        y, so = O.wkv5_fwd(q["r"], q["k"], q["v"], wf, q["u"], q["state_in"])
        g = O.wkv5_bwd(q["r"], q["k"], q["v"], wf, q["u"], q["state_in"], q["gy"], q["gstate_out"])
        g["gw"] = g.pop("gwdec") * (wf * np.log(wf) * live).reshape(1, -1)
    g["y"], g["state_out"] = y, so
    return g


def run(variant, q, layout, wkv56, W, path):
    name = "wkv6" if variant == "v6" else "wkv5"
    d = {n: TL.to_dev(q[n], BF) for n in ("r", "k", "v", "gy", "u")}
    w = TL.to_dev(q["x"], BF if variant == "v6" else torch.float32)
    tr = (lambda a: np.swapaxes(a, -1, -2)) if layout == W.WKV_STATE_VK else (lambda a: a)
    s_in = TL.to_dev(tr(q["state_in"]), torch.float32)
    gs = TL.to_dev(tr(q["gstate_out"]), torch.float32)
    y, so = wkv56.forward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, w_kind=W.WKV_W_RAW,
                          layout=layout, path=path)
    gr, gk, gv, gw, gu, gsi = wkv56.backward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, d["gy"],
                                             gs, w_kind=W.WKV_W_RAW, layout=layout, path=path)
    torch.cuda.synchronize()
    return dict(y=y, state_out=tr(TL.back(so)), gr=gr, gk=gk, gv=gv, gw=gw, gu=gu,
                gstate_in=tr(TL.back(gsi)))


SHAPES = [(1, 64, 1), (2, 128, 2), (1, 1, 1), (1, 31, 1), (2, 65, 1), (1, 100, 3), (3, 192, 2),
          (1, 1000, 1), (2, 4096, 2)]


@pytest.mark.parametrize("variant", ["v6", "v5"])
@pytest.mark.parametrize("B,T,H", SHAPES)
def test_chunked_matches_oracle(variant, B, T, H):
    W, wkv56 = _pkg()
    q = TL.case56(variant, B, T, H, BF, seed=200 + T)
    want = floored_oracle(variant, q)
    got = run(variant, q, W.WKV_STATE_KV, wkv56, W, W.WKV_PATH_CHUNKED)
    for n in ("y", "state_out", "gr", "gk", "gv", "gw", "gu", "gstate_in"):
        TL.assert_close(f"{variant}.{n}", got[n], want[n], 2e-2, extra=f"(B={B},T={T},H={H})")


@pytest.mark.parametrize("variant", ["v6", "v5"])
def test_chunked_value_key_state_layout(variant):
    W, wkv56 = _pkg()
    q = TL.case56(variant, 2, 160, 2, BF, seed=17)
    want = floored_oracle(variant, q)
    got = run(variant, q, W.WKV_STATE_VK, wkv56, W, W.WKV_PATH_CHUNKED)
    for n in ("y", "state_out", "gr", "gk", "gv", "gw", "gu", "gstate_in"):
        TL.assert_close(f"{variant}.{n}", got[n], want[n], 2e-2)


@pytest.mark.parametrize("shift", [2.0, 3.5, -3.0])
def test_chunked_v6_decay_extremes(shift):
    """x shifted by +2 / +3.5 (most decays far below the floor: w down to 1e-30) and by -3
    (decay ~ 1): finite everywhere and within tolerance of the floored fp64 recurrence"""
    W, wkv56 = _pkg()
    q = TL.case56("v6", 1, 256, 2, BF, seed=33, x_shift=shift)
    q["x"] = TL.rounded(q["x"], BF)
    want = floored_oracle("v6", q)
    got = run("v6", q, W.WKV_STATE_KV, wkv56, W, W.WKV_PATH_CHUNKED)
    for n, a in got.items():
        a = TL.back(a) if torch.is_tensor(a) else a
        assert np.isfinite(a).all(), n
    for n in EXTREME_CHECKED:
        TL.assert_close(f"v6.{n}", got[n], want[n], 2e-2, extra=f"(shift={shift})")


def test_chunked_v6_mild_and_steep_chunks_mixed():
    """the kernels factor a chunk around one point when its decay is mild and around block
    midpoints otherwise; here chunks of both kinds alternate inside one call (and inside one head)"""
    W, wkv56 = _pkg()
    q = TL.case56("v6", 2, 512, 2, BF, seed=41)
    x = q["x"].copy()
    x[:, 64:128] += 3.0          # a steep chunk
    x[:, 200:210] += 4.0         # ten steep tokens inside an otherwise mild chunk
    x[:, 320:448, :64] += 2.5    # steep in one head only
    q["x"] = TL.rounded(x, BF)
    want = floored_oracle("v6", q)
    got = run("v6", q, W.WKV_STATE_KV, wkv56, W, W.WKV_PATH_CHUNKED)
    for n in EXTREME_CHECKED:
        TL.assert_close(f"v6.{n}", got[n], want[n], 2e-2)


def test_chunked_bitwise_repeatable():
    """no atomics anywhere: the same call twice gives identical bits"""
    W, wkv56 = _pkg()
    q = TL.case56("v6", 2, 320, 2, BF, seed=5)
    a = run("v6", q, W.WKV_STATE_KV, wkv56, W, W.WKV_PATH_CHUNKED)
    b = run("v6", q, W.WKV_STATE_KV, wkv56, W, W.WKV_PATH_CHUNKED)
    for n in a:
        x, y = (TL.back(t) if torch.is_tensor(t) else t for t in (a[n], b[n]))
        assert np.array_equal(x, y), n


@pytest.mark.parametrize("variant", ["v6", "v5"])
def test_checkpoint_handover_equals_recompute(variant):
    """backward given the chunk-start states that forward saved == backward recomputing them"""
    W, wkv56 = _pkg()
    name = "wkv6" if variant == "v6" else "wkv5"
    q = TL.case56(variant, 2, 200, 2, BF, seed=77)
    d = {n: TL.to_dev(q[n], BF) for n in ("r", "k", "v", "gy", "u")}
    w = TL.to_dev(q["x"], BF if variant == "v6" else torch.float32)
    s_in = TL.to_dev(q["state_in"], torch.float32)
    gs = TL.to_dev(q["gstate_out"], torch.float32)
    y, so, ck = wkv56.forward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, w_kind=W.WKV_W_RAW,
                              save_ckpt=True)
    assert ck is not None
    a = wkv56.backward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, d["gy"], gs,
                       w_kind=W.WKV_W_RAW, ckpt=ck)
    b = wkv56.backward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, d["gy"], gs,
                       w_kind=W.WKV_W_RAW)
    torch.cuda.synchronize()
    for x, z in zip(a, b):
        assert torch.equal(x, z)
