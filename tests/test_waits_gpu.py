"""The bounded device-side waits really give up, and the kernels unwind when they do.

Nothing here hangs or faults the GPU: a wait is made to run out by never issuing the TMA load
it waits for (a host-side decision passed to the kernel) and by cutting the number of polls
from 4e6 to a few thousand.  The kernels must return, report through the status word, free
their tensor memory, and leave the context usable -- the next call must work."""
import ctypes

import pytest
import torch

import wkv_testlib as TL

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def test_bounded_wait_gives_up_and_raises_the_abort_flag():
    from rwkv_infctx_trainer_b200 import _lib as L
    lib = L.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    code = lib.wkv_selftest_wait_timeout(status.data_ptr(), 1000, torch.cuda.current_stream().cuda_stream)
    assert code == 0
    torch.cuda.synchronize()
    # 16: the plain wait ran out; 32: the abortable wait (64x the polls) ended as well
    assert int(status.item()) == 16 | 32
    assert lib.wkv_selftest_wait_timeout(status.data_ptr(), 0, None) == 2          # refused: no limit
    assert lib.wkv_selftest_wait_timeout(status.data_ptr(), 10 ** 7, None) == 2    # refused: too long for a test


@pytest.mark.parametrize("kernel,backward,bit", [(0, 0, 1), (1, 1, 2), (2, 1, 4)])
def test_kernels_unwind_when_a_load_never_arrives(kernel, backward, bit):
    """kernel 0 = forward, 1 = dS scan, 2 = per-chunk backward: the load of chunk (step) 1 is
    left out, the waits are cut to 2000 polls; the status word carries the kernel's bit, and the
    same call without the fault then gives the right answer"""
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import _lib as L, wkv56
    import test_chunked_gpu as CG
    lib = L.load()
    B, T, H = 1, 256, 2
    q = TL.case56("v6", B, T, H, BF, seed=91)
    d = {n: TL.to_dev(q[n], BF) for n in ("r", "k", "v", "gy", "u", "x")}
    s_in = TL.to_dev(q["state_in"], torch.float32)
    gso = TL.to_dev(q["gstate_out"], torch.float32)
    out = {n: torch.empty_like(d["r"]) for n in ("y", "gr", "gk", "gv", "gw")}
    so, gsi = torch.empty_like(s_in), torch.empty_like(s_in)
    gu = torch.empty((B, H * 64), device="cuda")
    a = wkv56._args("wkv6", B, T, H, BF, W.WKV_W_RAW, W.WKV_STATE_KV, W.WKV_PATH_CHUNKED, 1,
                    r=d["r"], k=d["k"], v=d["v"], w=d["x"], u=d["u"], state_in=s_in, y=out["y"], state_out=so,
                    gy=d["gy"], gstate_out=gso, gr=out["gr"], gk=out["gk"], gv=out["gv"], gw=out["gw"], gu=gu,
                    gstate_in=gsi)
    n = lib.wkv6_backward_workspace(ctypes.byref(a)) if backward else lib.wkv6_forward_workspace(ctypes.byref(a))
    ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = ws.data_ptr(), n
    st = torch.cuda.current_stream().cuda_stream
    code = lib.wkv56_selftest_abort(ctypes.byref(a), 1, backward, kernel, 1, 2000, st)
    assert code == 0
    torch.cuda.synchronize()          # returns: nothing hangs
    status = int(ws[:4].view(torch.int32).item())
    assert status & bit, status
    # the context is intact: the same arguments without the fault give the oracle's answer
    wkv56.CHECK_STATUS = True
    got = CG.run("v6", q, W.WKV_STATE_KV, wkv56, W, W.WKV_PATH_CHUNKED)
    want = CG.floored_oracle("v6", q)
    for name in ("y", "state_out", "gr", "gk", "gv", "gw", "gu", "gstate_in"):
        TL.assert_close(name, got[name], want[name], 2e-2)


def test_status_word_reaches_the_host_without_a_sync():
    """in normal use (CHECK_STATUS off) a call whose kernel gave up is reported by the next call on
    that device, or by poll_status()"""
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import wkv56
    wkv56.CHECK_STATUS = False
    try:
        B, T, H = 1, 128, 1
        q = TL.case56("v6", B, T, H, BF, seed=92)
        d = {n: TL.to_dev(q[n], BF) for n in ("r", "k", "v", "u", "x")}
        s_in = TL.to_dev(q["state_in"], torch.float32)
        wkv56.forward("wkv6", d["r"], d["k"], d["v"], d["x"], d["u"], s_in, w_kind=W.WKV_W_RAW)
        wkv56.poll_status(wait=True)          # a healthy call: nothing raised
        # a word that says "gave up", queued the way a call queues its own
        ev = torch.cuda.Event(); ev.record()
        word = torch.full((1,), 4, dtype=torch.int32).pin_memory()
        wkv56._pending.setdefault(0, []).append((ev, word, "wkv6_backward"))
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="device-side wait ran out"):
            wkv56.forward("wkv6", d["r"], d["k"], d["v"], d["x"], d["u"], s_in, w_kind=W.WKV_W_RAW)
        wkv56.poll_status(wait=True)          # reported once, then cleared
    finally:
        wkv56.CHECK_STATUS = True
