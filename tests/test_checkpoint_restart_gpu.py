"""Activation checkpointing re-runs a block's forward inside backward
(RWKV-v6/src/model.py:657-665).  With a ``SavedStates`` shared by the two runs, the second run of
the WKV op restarts every 8-chunk group from the fp32 state the first run stored instead of
scanning over T again -- and must give bit-identical outputs, so that the checkpointed step has
exactly the gradients of the plain one."""
import numpy as np
import pytest
import torch
from torch.utils.checkpoint import checkpoint

import wkv_testlib as TL
import test_chunked_gpu as CG

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("variant", ["v6", "v5"])
@pytest.mark.parametrize("B,T,H,groups", [(2, 1536, 2, 1), (1, 1000, 2, 0), (1, 4096, 3, 0), (2, 200, 1, 1)])
def test_restart_from_saved_states_is_bit_identical(variant, B, T, H, groups):
    W, wkv56 = CG._pkg()
    name = "wkv6" if variant == "v6" else "wkv5"
    q = TL.case56(variant, B, T, H, BF, seed=400 + T)
    d = {n: TL.to_dev(q[n], BF) for n in ("r", "k", "v", "u")}
    w = TL.to_dev(q["x"], BF if variant == "v6" else torch.float32)
    s_in = TL.to_dev(q["state_in"], torch.float32)
    saved = wkv56.SavedStates()
    args = (name, d["r"], d["k"], d["v"], w, d["u"], s_in)
    y0, s0, c0 = wkv56.forward(*args, w_kind=W.WKV_W_RAW, save_ckpt=True, time_groups=groups, saved=saved)
    assert saved.filled and saved.restarts == 0
    y1, s1, c1 = wkv56.forward(*args, w_kind=W.WKV_W_RAW, save_ckpt=True, time_groups=groups, saved=saved)
    assert saved.restarts == 1
    torch.cuda.synchronize()
    assert torch.equal(y0, y1) and torch.equal(s0, s1)
    # the hand-over to backward as well: states, scaled r, chunk decays, mild flags (then padding)
    al = lambda x: (x + 255) // 256 * 256
    n = (T + 63) // 64
    used = al(B * H * (n + 1) * 8192) + al(B * T * H * 128) + al(B * H * n * 256) + B * H * n
    assert torch.equal(c0[:used], c1[:used])
    want = CG.floored_oracle(variant, q)
    TL.assert_close("y", y1, want["y"], 2e-2)
    TL.assert_close("state_out", s1, want["state_out"], 2e-2)


def test_checkpointed_block_uses_the_saved_states_and_matches_the_plain_step():
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import wkv56
    torch.manual_seed(1)
    B, T, C, H = 2, 1024, 128, 2
    x = torch.randn((B, T, C), device="cuda") * 0.5
    Wr, Wk, Wv, Ww, Wo = (torch.nn.Parameter(torch.randn((C, C), device="cuda") * C ** -0.5) for _ in range(5))
    u = torch.nn.Parameter(torch.rand((H, 64), device="cuda") - 0.5)
    s0 = torch.randn((B, H, 64, 64), device="cuda") * 0.3
    params = (Wr, Wk, Wv, Ww, Wo, u)

    def block(x, saved):
        r, k, v, w = ((x @ M).to(BF) for M in (Wr, Wk, Wv, Ww))
        y, s = W.wkv6(r, k, v, (w.float() - 1.0).to(BF), u.to(BF), s0, saved=saved)
        return (y.float() @ Wo).sum() + s.sum()

    def grads(fn):
        for p in params:
            p.grad = None
        fn().backward()
        return [p.grad.clone() for p in params]

    plain = grads(lambda: block(x, None))
    saved = wkv56.SavedStates()
    ck = grads(lambda: checkpoint(block, x, saved, use_reentrant=False))
    assert saved.restarts == 1          # the run inside backward did not scan again
    for a, b in zip(plain, ck):
        assert torch.equal(a, b)
