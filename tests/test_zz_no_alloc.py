"""wkv4_backward_static: the v4 backward for callers that cannot provide scratch memory
(a binding with no device allocator of its own, or a loop that must not cudaMalloc
between steps).  It keeps the tile-start states in an array inside the library instead of
a caller workspace, so its results must agree with wkv4_backward's -- on a first call and
on a second call that reuses the same array with other sizes and inputs.  For segments
under 128 tokens both entry points run the same kernel and the results are identical bit
for bit; longer segments take the time-parallel kernels in wkv4_backward, and the two are
held to the parity tolerance of the other v4 tests (1e-3 fp32, 2e-2 bf16, max|a-b|/max|b|).
Runs last (file name) so that a failure here cannot hide any other test."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


def _run_both(B, T, C, dtype, seed):
    import rwkv_infctx_trainer_b200._lib as L
    lib = L.load()
    c = inputs.wkv4_case(B, T, C, seed)
    dev = "cuda"
    mk = lambda a, dt: torch.tensor(np.asarray(a), dtype=torch.float32).to(dt).to(dev).contiguous()
    w = mk(-np.exp(c["td"]), torch.float32)
    u, k, v, gy = (mk(c[n], dtype) for n in ("u", "k", "v", "gy"))
    # a non-trivial carried state and incoming state gradient
    s0 = torch.zeros((B, C, 3), device=dev); s0[..., 2] = -1e38
    y = torch.empty_like(k); s1 = torch.empty_like(s0)
    stream = torch.cuda.current_stream().cuda_stream
    code = L.DTYPE_CODE[dtype]
    nf = lib.wkv4_forward_workspace(B, T, C)
    wsf = torch.empty(max(nf, 16), dtype=torch.uint8, device=dev)
    L.check(lib.wkv4_forward(B, T, C, code, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                             s0.data_ptr(), y.data_ptr(), s1.data_ptr(), wsf.data_ptr(), nf, stream),
            "wkv4_forward")
    gso = mk(np.stack([inputs.normal((B, C), seed, stream=30), inputs.normal((B, C), seed, stream=31),
                       inputs.uniform((B, C), seed, -1, 1, stream=32)], -1), torch.float32)

    def outputs():
        return dict(gw=torch.full((B, C), 7.0, device=dev), gu=torch.full((B, C), 7.0, device=dev),
                    gk=torch.empty_like(k), gv=torch.empty_like(k), gsi=torch.empty_like(s0))

    a, b = outputs(), outputs()
    n = lib.wkv4_backward_workspace(B, T, C)
    assert n <= lib.wkv4_backward_static_limit()
    ws = torch.empty(n, dtype=torch.uint8, device=dev)
    common = (B, T, C, code, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(), s1.data_ptr(),
              gy.data_ptr(), gso.data_ptr())
    L.check(lib.wkv4_backward(*common, a["gw"].data_ptr(), a["gu"].data_ptr(), a["gk"].data_ptr(),
                              a["gv"].data_ptr(), a["gsi"].data_ptr(), ws.data_ptr(), n, stream),
            "wkv4_backward")
    L.check(lib.wkv4_backward_static(*common, b["gw"].data_ptr(), b["gu"].data_ptr(),
                                     b["gk"].data_ptr(), b["gv"].data_ptr(), b["gsi"].data_ptr(),
                                     stream), "wkv4_backward_static")
    torch.cuda.synchronize()
    return a, b


def _rel(x, y):
    x, y = x.double(), y.double()
    return float((x - y).abs().max() / y.abs().max().clamp_min(1e-30))


def test_static_scratch_backward_equals_workspace_backward_twice_in_a_row():
    for B, T, C, dtype, seed in ((2, 200, 256, torch.bfloat16, 1), (3, 77, 128, torch.float32, 2)):
        a, b = _run_both(B, T, C, dtype, seed)
        for name in a:
            assert torch.isfinite(b[name].float()).all(), name
        if T < 128:
            # same kernel, same arithmetic, only the scratch location differs
            for name in a:
                assert torch.equal(a[name], b[name]), f"{name} differs (B={B},T={T},C={C})"
        else:
            tol = 2e-2 if dtype == torch.bfloat16 else 1e-3
            for name in ("gw", "gu", "gk", "gv"):
                assert _rel(b[name].float(), a[name].float()) <= tol, name
            # (gp,gq,go) stands for (gp,gq)*e^go: compare what it represents
            for i in (0, 1):
                x = b["gsi"][..., i].double() * torch.exp(b["gsi"][..., 2].double())
                y = a["gsi"][..., i].double() * torch.exp(a["gsi"][..., 2].double())
                assert _rel(x, y) <= tol, ("gstate_in", i)


def test_static_scratch_rejects_oversized_problem_without_launching():
    """B=8, T=4096, C=2048 in bf16 needs more scratch than the built-in array holds.  The buffers
    are real and of full size, so that if the size check ever regressed the call would run on
    valid memory and fail this assert rather than fault the device."""
    import rwkv_infctx_trainer_b200._lib as L
    lib = L.load()
    limit = lib.wkv4_backward_static_limit()
    B, T, C = 8, 4096, 2048
    assert lib.wkv4_backward_workspace(B, T, C) > limit
    bf = torch.bfloat16
    k, v, gy, gk, gv = (torch.zeros((B, T, C), device="cuda", dtype=bf) for _ in range(5))
    w = -torch.ones(C, device="cuda")
    u = torch.zeros(C, device="cuda", dtype=bf)
    gw, gu = torch.zeros((B, C), device="cuda"), torch.zeros((B, C), device="cuda")
    code = lib.wkv4_backward_static(B, T, C, L.WKV_BF16, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                    None, gy.data_ptr(), None, gw.data_ptr(), gu.data_ptr(), gk.data_ptr(),
                                    gv.data_ptr(), None, torch.cuda.current_stream().cuda_stream)
    assert code == 8
    assert b"built-in" in lib.wkv_error_string(code)
    torch.cuda.synchronize()
