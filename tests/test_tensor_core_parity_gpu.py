"""The tcgen05 chunked kernels against what the reference itself produced.

* against the RWKV-infctx-trainer project's own v6 state kernels
  (RWKV-v6/src/module/cuda/wkv6state_cuda_v1.cu:295-308, compiled unchanged into
  oracle/_ref/): ours take the bf16 activation x (WKV_W_RAW) on WKV_PATH_CHUNKED, theirs the
  ew = -exp(float(x_bf16)) its Python wrapper would precompute
  (RWKV-v6/src/module/TimeMix.py:49-51); both start from the same bf16-rounded state;
* against the fixtures made from the reference's rwkv_inner (tests/golden/*.npz), inputs
  rounded to bf16 so that the call really runs on the chunked kernels;
* at the grids the benchmark launches (hundreds of co-resident CTAs, two per SM), where the
  fp64 oracle runs on a sample of (batch, head) units and the token-serial kernel on all.

Tolerance: max|ours-ref| / max|ref| <= 2e-2 per tensor (bf16 I/O).
"""
import ast
import ctypes
import os

import numpy as np
import pytest
import torch

import inputs
import wkv_testlib as TL
from oracle import build as OB
from oracle import wkv_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
TOL = 2e-2
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _pkg():
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import wkv56
    wkv56.CHECK_STATUS = True
    return W, wkv56


def _ref(name):
    path = os.path.join(OB.REF_DIR, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} not prebuilt")
    return ctypes.CDLL(path)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def assert_runs_chunked(W, wkv56, variant, r, w, w_kind, path):
    """the call with these arguments is served by the tensor-core kernels, not the token-serial ones"""
    from rwkv_infctx_trainer_b200 import _lib as L
    B, T, C = r.shape
    a = wkv56._args(variant, B, T, C // 64, r.dtype, w_kind, W.WKV_STATE_KV, path)
    assert L.load().wkv56_uses_chunked(ctypes.byref(a), int(variant == "wkv6")) == 1


def _run_reference_v6(lib, r, k, v, ew, u, s_bf, gy, H):
    _, T, C = r.shape
    s_ref = s_bf.clone()
    y_ref = torch.empty_like(r)
    lib.ref_wkv6_forward(1, T, C, H, _p(r), _p(k), _p(v), _p(ew), _p(u), _p(s_ref), _p(y_ref))
    mk = lambda *s: torch.empty(s, device="cuda", dtype=BF)
    g = dict(gr=mk(1, T, C), gk=mk(1, T, C), gv=mk(1, T, C), gw=mk(1, T, C), gu=mk(1, C),
             gs=mk(1, H, 64, 64))
    lib.ref_wkv6_backward(1, T, C, H, _p(r), _p(k), _p(v), _p(ew), _p(u), _p(s_bf), _p(gy),
                          _p(g["gr"]), _p(g["gk"]), _p(g["gv"]), _p(g["gw"]), _p(g["gu"]), _p(g["gs"]))
    torch.cuda.synchronize()
    g["y"], g["state"] = y_ref, s_ref
    return g


@pytest.mark.parametrize("time_groups", [1, 2])
def test_v6_chunked_matches_reference_state_kernels(time_groups):
    """every decay above the 0.005 floor of the chunked kernels: the two implementations
    compute the same function, and must agree on y, state and every gradient"""
    W, wkv56 = _pkg()
    lib = _ref("libref_wkv6state.so")
    H, T = 3, 256
    q = TL.case56("v6", 1, T, H, BF, seed=63, gstate=False)
    # exp(-exp(x)) >= 0.005  <=>  x <= log(-log(0.005)) = 1.667; keep clear of it after bf16 rounding
    q["x"] = TL.rounded(np.minimum(q["x"], 1.6), BF)
    assert np.exp(-np.exp(q["x"])).min() > 0.005
    r, k, v, u, gy, x = (TL.to_dev(q[n], BF) for n in ("r", "k", "v", "u", "gy", "x"))
    ew = (-torch.exp(x.float())).contiguous()
    s_bf = TL.to_dev(np.swapaxes(q["state_in"], -1, -2), BF)
    s_in32 = s_bf.float().contiguous()
    ref = _run_reference_v6(lib, r, k, v, ew, u, s_bf, gy, H)
    assert_runs_chunked(W, wkv56, "wkv6", r, x, W.WKV_W_RAW, W.WKV_PATH_CHUNKED)
    y, s_out = wkv56.forward("wkv6", r, k, v, x, u, s_in32, w_kind=W.WKV_W_RAW, layout=W.WKV_STATE_VK,
                             path=W.WKV_PATH_CHUNKED, time_groups=time_groups)
    gr, gk, gv, gw, gu, gs = wkv56.backward("wkv6", r, k, v, x, u, s_in32, gy, None, w_kind=W.WKV_W_RAW,
                                            layout=W.WKV_STATE_VK, path=W.WKV_PATH_CHUNKED,
                                            time_groups=time_groups)
    got = dict(y=y, state=s_out, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu, gs=gs)
    for n in ("y", "state", "gr", "gk", "gv", "gw", "gu", "gs"):
        TL.assert_close(n, got[n], TL.back(ref[n]), TOL)


def test_v6_chunked_vs_reference_kernels_below_the_floor():
    """Decays below 0.005: the chunked kernels floor them (as the reference's rwkv_inner does,
    RWKV-v6/src/module/rwkv_inner.py:40-45), the reference CUDA kernel does not.  x is shifted
    so that about 4 % of the decays fall below the floor; the deviation this causes is measured
    here, and bounded: the tensors that do not depend on the floored elements' own gradient stay
    inside the bf16 tolerance, gw is compared where the decay is above the floor."""
    W, wkv56 = _pkg()
    lib = _ref("libref_wkv6state.so")
    H, T = 2, 256
    q = TL.case56("v6", 1, T, H, BF, seed=64, gstate=False, x_shift=1.4)
    q["x"] = TL.rounded(q["x"], BF)
    below = np.exp(-np.exp(q["x"])) < 0.005
    assert 0.01 < below.mean() < 0.2
    r, k, v, u, gy, x = (TL.to_dev(q[n], BF) for n in ("r", "k", "v", "u", "gy", "x"))
    ew = (-torch.exp(x.float())).contiguous()
    s_bf = TL.to_dev(np.swapaxes(q["state_in"], -1, -2), BF)
    s_in32 = s_bf.float().contiguous()
    ref = _run_reference_v6(lib, r, k, v, ew, u, s_bf, gy, H)
    y, s_out = wkv56.forward("wkv6", r, k, v, x, u, s_in32, w_kind=W.WKV_W_RAW, layout=W.WKV_STATE_VK,
                             path=W.WKV_PATH_CHUNKED)
    gr, gk, gv, gw, gu, gs = wkv56.backward("wkv6", r, k, v, x, u, s_in32, gy, None, w_kind=W.WKV_W_RAW,
                                            layout=W.WKV_STATE_VK, path=W.WKV_PATH_CHUNKED)
    got = dict(y=y, state=s_out, gr=gr, gk=gk, gv=gv, gu=gu, gs=gs)
    dev = {n: TL.err(got[n], TL.back(ref[n])) for n in got}
    live = ~below
    dev["gw_live"] = O.max_rel_err(TL.back(gw) * live, TL.back(ref["gw"]) * live)
    dev["gw_floored_ours_max"] = float(np.abs(TL.back(gw) * below).max())
    print("deviation from the unfloored reference kernel with %.1f%% of decays floored: %s"
          % (100 * below.mean(), {n: "%.2e" % e for n, e in dev.items()}))
    # a floored element keeps 0.005 of the state where the reference keeps less: a bounded change
    for n in ("y", "state", "gr", "gk", "gv", "gu", "gs", "gw_live"):
        assert dev[n] <= 5e-2, (n, dev[n])
    assert dev["gw_floored_ours_max"] == 0.0      # no gradient through the floor


def _load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return ast.literal_eval(str(z["meta"])), {k: z[k] for k in z.files if k != "meta"}


@pytest.mark.parametrize("name", ["v5_small", "v6_small", "v5_config0", "v6_config0shape"])
def test_reference_fixtures_through_the_chunked_kernels(name):
    """the BPTT chain of the fixture (segments with the state and its gradient carried by
    autograd) on bf16 tensors, so that every call is served by the tcgen05 kernels; held to what
    the reference's rwkv_inner produced in fp32 on the unrounded inputs"""
    W, wkv56 = _pkg()
    meta, gold = _load_golden(name)
    v, B, T, H, N, seg = (meta[k] for k in ("variant", "B", "T", "H", "N", "seg_len"))
    c = inputs.wkv56_case(v, B, T, H, N, meta["seed"], state=meta["state"], gstate=meta["gstate"])
    t = {n: torch.tensor(a, dtype=torch.float32, device="cuda") for n, a in c.items()}
    leaves = {n: t[n].to(BF).requires_grad_(True) for n in ("r", "k", "v", "u")}
    leaves["x"] = (t["x"].to(BF) if v == "v6" else t["x"].clone()).requires_grad_(True)
    leaves["state_in"] = t["state_in"].clone().requires_grad_(True)
    fn = W.WKV6 if v == "v6" else W.WKV5
    name_abi = "wkv6" if v == "v6" else "wkv5"
    state = leaves["state_in"]
    ys = []
    for t0 in range(0, T, seg):
        t1 = min(T, t0 + seg)
        xs = leaves["x"][:, t0:t1] if v == "v6" else leaves["x"]
        rs = leaves["r"][:, t0:t1].contiguous()
        assert_runs_chunked(W, wkv56, name_abi, rs, xs, W.WKV_W_RAW, W.WKV_PATH_CHUNKED)
        y, state = fn.apply(B, t1 - t0, H * N, H, rs, leaves["k"][:, t0:t1], leaves["v"][:, t0:t1], xs,
                            leaves["u"], state, W.WKV_PATH_CHUNKED)
        ys.append(y)
    y = torch.cat(ys, 1)
    loss = (y.float() * t["gy"]).sum() + (state * t["gstate_out"]).sum()
    loss.backward()
    got = dict(y=y, state_out=state, gr=leaves["r"].grad, gk=leaves["k"].grad, gv=leaves["v"].grad,
               gw=leaves["x"].grad, gu=leaves["u"].grad, gstate_in=leaves["state_in"].grad)
    s = meta["stride"]
    for n, ref in gold.items():
        g = TL.back(got[n])
        if s > 1 and (n in ("y", "gr", "gk", "gv") or (n == "gw" and v == "v6")):
            g = g[:, ::s]
        e = O.max_rel_err(g, ref)
        assert e <= TOL, (name, n, e)


def _unit(d, b, h, variant):
    """the (batch b, head h) unit of a case on the device as a B=1, H=1 numpy case of its own"""
    sl = slice(h * 64, (h + 1) * 64)
    u = {n: TL.back(d[n][b:b + 1, :, sl]) for n in ("r", "k", "v", "gy")}
    u["u"] = TL.back(d["u"][h:h + 1])
    u["x"] = TL.back(d["x"][b:b + 1, :, sl] if variant == "v6" else d["x"][h:h + 1])
    u["state_in"] = TL.back(d["state_in"][b:b + 1, h:h + 1])
    u["gstate_out"] = TL.back(d["gstate_out"][b:b + 1, h:h + 1])
    return u


def _torch_case(variant, B, T, H, seed):
    """the benchmark's distributions, drawn on the device (the numpy generator is too slow at
    these sizes); returned as device tensors plus what the oracle needs on demand"""
    g = torch.Generator(device="cuda").manual_seed(seed)
    C = H * 64
    d = {n: torch.randn((B, T, C), generator=g, device="cuda").to(BF) for n in ("r", "k", "v", "gy")}
    d["u"] = (torch.rand((H, 64), generator=g, device="cuda") * 2 - 1).to(BF)
    if variant == "v6":
        d["x"] = (torch.randn((B, T, C), generator=g, device="cuda") * 0.5 - 0.6).to(BF)
    else:
        d["x"] = torch.rand((H, 64), generator=g, device="cuda") * 5 - 6
    d["state_in"] = torch.randn((B, H, 64, 64), generator=g, device="cuda") * 0.5
    d["gstate_out"] = torch.randn((B, H, 64, 64), generator=g, device="cuda") * 0.5
    return d


@pytest.mark.parametrize("variant,B,T,H", [("v6", 4, 4096, 64), ("v5", 8, 2048, 32)])
def test_chunked_at_the_benchmark_grid(variant, B, T, H):
    """One BPTT segment of the v6 7B-shape workload (256 chains, 16384 per-chunk CTAs, two CTAs
    per SM) and of the v5 1.5B-shape workload.  Every (batch, head) unit is independent, so the
    fp64 oracle checks a sample of units spread over the grid, and the token-serial kernel (itself
    held to the oracle and to the reference kernels elsewhere) checks all of them on the GPU."""
    import test_chunked_gpu as CG
    W, wkv56 = _pkg()
    name = "wkv6" if variant == "v6" else "wkv5"
    d = _torch_case(variant, B, T, H, seed=3)
    args = (d["r"], d["k"], d["v"], d["x"], d["u"], d["state_in"])
    assert_runs_chunked(W, wkv56, name, d["r"], d["x"], W.WKV_W_RAW, W.WKV_PATH_AUTO)
    y, so, ck = wkv56.forward(name, *args, w_kind=W.WKV_W_RAW, path=W.WKV_PATH_CHUNKED, save_ckpt=True)
    got = wkv56.backward(name, *args, d["gy"], d["gstate_out"], w_kind=W.WKV_W_RAW,
                         path=W.WKV_PATH_CHUNKED, ckpt=ck)
    ys, sos = wkv56.forward(name, *args, w_kind=W.WKV_W_RAW, path=W.WKV_PATH_SCALAR)
    ser = wkv56.backward(name, *args, d["gy"], d["gstate_out"], w_kind=W.WKV_W_RAW,
                         path=W.WKV_PATH_SCALAR)
    torch.cuda.synchronize()
    names = ("gr", "gk", "gv", "gw", "gu", "gstate_in")

    def rel(a, b):      # per-tensor max|a-b| / max|b| on the device
        a, b = a.float(), b.float()
        return float((a - b).abs().max() / b.abs().max())

    assert rel(y, ys) <= TOL and rel(so, sos) <= TOL
    for n, a, b in zip(names, got, ser):
        assert torch.isfinite(a.float()).all(), n
        assert rel(a, b) <= TOL, (n, rel(a, b))
    # the same per unit: no single (batch, head) may hide behind the global maximum
    yu = (y.float() - ys.float()).abs().view(B, T, H, 64).amax(dim=(1, 3)) / \
        ys.float().abs().view(B, T, H, 64).amax(dim=(1, 3))
    assert float(yu.max()) <= TOL, float(yu.max())
    gv_u = (got[2].float() - ser[2].float()).abs().view(B, T, H, 64).amax(dim=(1, 3)) / \
        ser[2].float().abs().view(B, T, H, 64).amax(dim=(1, 3))
    assert float(gv_u.max()) <= TOL, float(gv_u.max())
    # fp64 oracle on six units spread over the grid (first, last, and across SM boundaries)
    outs = dict(y=y, state_out=so, **dict(zip(names, got)))
    for b, h in [(0, 0), (0, H - 1), (B // 2, H // 3), (B - 1, 1), (B - 1, H // 2), (B - 1, H - 1)]:
        want = CG.floored_oracle(variant, _unit(d, b, h, variant))
        sl = slice(h * 64, (h + 1) * 64)
        pick = dict(y=outs["y"][b:b + 1, :, sl], state_out=outs["state_out"][b:b + 1, h:h + 1],
                    gr=outs["gr"][b:b + 1, :, sl], gk=outs["gk"][b:b + 1, :, sl],
                    gv=outs["gv"][b:b + 1, :, sl], gstate_in=outs["gstate_in"][b:b + 1, h:h + 1],
                    gu=outs["gu"][b:b + 1, sl])
        pick["gw"] = outs["gw"][b:b + 1, :, sl] if variant == "v6" else outs["gw"][b:b + 1, sl]
        for n, a in pick.items():
            TL.assert_close(f"{variant}[{b},{h}].{n}", a, want[n], TOL)


def test_v4_at_the_benchmark_grid():
    """one 2048-token segment of the v4 workload (B=8, C=2048, fp32 I/O: 32 pieces of 64 tokens
    folded per channel) from a non-trivial carried state; fp64 oracle on 64 channels spread over C"""
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import _lib as L
    B, T, C = 8, 2048, 2048
    g = torch.Generator(device="cuda").manual_seed(11)
    k, v, gy = (torch.randn((B, T, C), generator=g, device="cuda") for _ in range(3))
    td = torch.rand(C, generator=g, device="cuda") * 6 - 5
    u = torch.rand(C, generator=g, device="cuda") * 2 - 1
    w = -torch.exp(td)
    s0 = torch.zeros((B, C, 3), device="cuda"); s0[..., 2] = -1e38
    lib, st = L.load(), torch.cuda.current_stream().cuda_stream
    nf, nb = lib.wkv4_forward_workspace(B, T, C), lib.wkv4_backward_workspace(B, T, C)
    wsf = torch.empty(max(nf, 16), dtype=torch.uint8, device="cuda")
    wsb = torch.empty(max(nb, 16), dtype=torch.uint8, device="cuda")
    y0, s1, y, s2 = torch.empty_like(k), torch.empty_like(s0), torch.empty_like(k), torch.empty_like(s0)
    # a first segment (k and v swapped: just other data) builds the carried state
    L.check(lib.wkv4_forward(B, T, C, 0, w.data_ptr(), u.data_ptr(), v.data_ptr(), k.data_ptr(),
                             s0.data_ptr(), y0.data_ptr(), s1.data_ptr(), wsf.data_ptr(), nf, st), "fwd0")
    L.check(lib.wkv4_forward(B, T, C, 0, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                             s1.data_ptr(), y.data_ptr(), s2.data_ptr(), wsf.data_ptr(), nf, st), "fwd1")
    gso = torch.randn((B, C, 3), generator=g, device="cuda") * 0.1
    gw, gu = torch.empty((B, C), device="cuda"), torch.empty((B, C), device="cuda")
    gk, gv, gsi = torch.empty_like(k), torch.empty_like(k), torch.empty_like(s0)
    L.check(lib.wkv4_backward(B, T, C, 0, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                              s1.data_ptr(), gy.data_ptr(), gso.data_ptr(), gw.data_ptr(), gu.data_ptr(),
                              gk.data_ptr(), gv.data_ptr(), gsi.data_ptr(), wsb.data_ptr(), nb, st), "bwd")
    torch.cuda.synchronize()
    ch = torch.arange(0, C, C // 64, device="cuda")
    wn, un = TL.back(w[ch]), TL.back(u[ch])
    kn, vn, gyn = (TL.back(t[:, :, ch]) for t in (k, v, gy))
    s1n, gson = TL.back(s1[:, ch]), TL.back(gso[:, ch])
    yw, s2w = O.wkv4_fwd(wn, un, kn, vn, s1n)
    gwant = O.wkv4_bwd(wn, un, kn, vn, s1n, gyn, gson)
    tol = 1e-3
    TL.assert_close("y", y[:, :, ch], yw, tol)
    a, b = TL.back(s2[:, ch]), s2w
    TL.assert_close("p", a[..., 0] * np.exp(a[..., 2]), b[..., 0] * np.exp(b[..., 2]), tol)
    TL.assert_close("q", a[..., 1] * np.exp(a[..., 2]), b[..., 1] * np.exp(b[..., 2]), tol)
    TL.assert_close("gk", gk[:, :, ch], gwant["gk"], tol)
    TL.assert_close("gv", gv[:, :, ch], gwant["gv"], tol)
    TL.assert_close("gw", gw[:, ch], gwant["gw"], tol)
    TL.assert_close("gu", gu[:, ch], gwant["gu"], tol)
    ga, gb = TL.back(gsi[:, ch]), gwant["gstate_in"]
    # (gp, gq) are stored relative to the shared exponent go: compare the represented values
    for i, n in enumerate(("gp", "gq")):
        TL.assert_close(n, ga[..., i] * np.exp(ga[..., 2]), gb[..., i] * np.exp(gb[..., 2]), tol)
