"""Time groups of the chunked v5/v6 kernels: a chain of chunks cut into G groups that run in
parallel (summary pass per group, scan over the groups, full pass per group) must give what
the uncut chain gives -- the same function, up to the order of a few fp32 additions -- for
any G, for segments that are not a multiple of the chunk or the group length, in both state
layouts, with and without the forward hand-over, and when the library picks G itself."""
import numpy as np
import pytest
import torch

import wkv_testlib as TL
import test_chunked_gpu as CG

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
NAMES = ("y", "state_out", "gr", "gk", "gv", "gw", "gu", "gstate_in")


def run(variant, q, layout, groups, handover, W, wkv56):
    name = "wkv6" if variant == "v6" else "wkv5"
    d = {n: TL.to_dev(q[n], BF) for n in ("r", "k", "v", "gy", "u")}
    w = TL.to_dev(q["x"], BF if variant == "v6" else torch.float32)
    tr = (lambda a: np.swapaxes(a, -1, -2)) if layout == W.WKV_STATE_VK else (lambda a: a)
    s_in = TL.to_dev(tr(q["state_in"]), torch.float32)
    gs = TL.to_dev(tr(q["gstate_out"]), torch.float32)
    out = wkv56.forward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, w_kind=W.WKV_W_RAW, layout=layout,
                        path=W.WKV_PATH_CHUNKED, save_ckpt=handover, time_groups=groups)
    y, so = out[0], out[1]
    ck = out[2] if handover else None
    gr, gk, gv, gw, gu, gsi = wkv56.backward(name, d["r"], d["k"], d["v"], w, d["u"], s_in, d["gy"], gs,
                                             w_kind=W.WKV_W_RAW, layout=layout, path=W.WKV_PATH_CHUNKED,
                                             ckpt=ck, time_groups=groups)
    torch.cuda.synchronize()
    return dict(y=y, state_out=tr(TL.back(so)), gr=gr, gk=gk, gv=gv, gw=gw, gu=gu, gstate_in=tr(TL.back(gsi)))


@pytest.mark.parametrize("variant", ["v6", "v5"])
@pytest.mark.parametrize("B,T,H,groups", [(2, 512, 2, 2), (1, 1000, 1, 3), (1, 1000, 1, 16), (2, 300, 1, 5),
                                           (1, 4096, 2, 64), (1, 129, 2, 7)])
def test_groups_equal_the_uncut_chain(variant, B, T, H, groups):
    W, wkv56 = CG._pkg()
    q = TL.case56(variant, B, T, H, BF, seed=300 + T + groups)
    one = run(variant, q, W.WKV_STATE_KV, 1, True, W, wkv56)
    cut = run(variant, q, W.WKV_STATE_KV, groups, True, W, wkv56)
    want = CG.floored_oracle(variant, q)
    for n in NAMES:
        # against each other: the group scan only re-associates fp32 sums of the carried matrices
        TL.assert_close(f"{variant}.{n} G={groups} vs G=1", cut[n], TL.back(one[n]) if torch.is_tensor(one[n]) else one[n], 4e-3)
        TL.assert_close(f"{variant}.{n} G={groups} vs oracle", cut[n], want[n], 2e-2)


@pytest.mark.parametrize("variant", ["v6", "v5"])
def test_groups_value_key_layout_and_no_handover(variant):
    """[value,key] state (the group scan reads and writes the caller's layout) and a backward
    call that has to rebuild the chunk-start states itself, through the same three passes"""
    W, wkv56 = CG._pkg()
    q = TL.case56(variant, 2, 700, 2, BF, seed=8)
    want = CG.floored_oracle(variant, q)
    got = run(variant, q, W.WKV_STATE_VK, 4, False, W, wkv56)
    for n in NAMES:
        TL.assert_close(f"{variant}.{n}", got[n], want[n], 2e-2)


def test_library_picks_groups_when_chains_are_few():
    """the long-context shape in small: one batch row, 5 heads, 4096 tokens -- 5 chains of 64
    chunks, which the library cuts by itself (time_groups = 0) -- against the oracle, and bitwise
    repeatable"""
    W, wkv56 = CG._pkg()
    q = TL.case56("v6", 1, 4096, 5, BF, seed=12)
    want = CG.floored_oracle("v6", q)
    a = run("v6", q, W.WKV_STATE_KV, 0, True, W, wkv56)
    b = run("v6", q, W.WKV_STATE_KV, 0, True, W, wkv56)
    for n in NAMES:
        TL.assert_close(f"v6.{n}", a[n], want[n], 2e-2)
        x, y = (TL.back(t) if torch.is_tensor(t) else t for t in (a[n], b[n]))
        assert np.array_equal(x, y), n
    # the forward workspace is larger than the status block alone: the call was split
    import ctypes
    from rwkv_infctx_trainer_b200 import _lib as L
    r = TL.to_dev(q["r"], BF)
    args = wkv56._args("wkv6", 1, 4096, 5, BF, W.WKV_W_RAW, W.WKV_STATE_KV, W.WKV_PATH_AUTO)
    assert L.load().wkv6_forward_workspace(ctypes.byref(args)) > 256
    args.time_groups = 1
    assert L.load().wkv6_forward_workspace(ctypes.byref(args)) == 256
