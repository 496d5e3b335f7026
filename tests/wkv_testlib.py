"""Helpers shared by the GPU parity tests: build inputs on the device, run the
CUDA ops through the package (which calls the C ABI), run the fp64 oracle on the
same (dtype-rounded) inputs, compare with max|a-b|/max|b|."""
from __future__ import annotations

import numpy as np
import torch

import inputs
from oracle import wkv_oracle as O

TOL = {torch.float32: 1e-3, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def to_dev(a, dtype, dev="cuda"):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(dtype).to(dev).contiguous()


def back(t):
    """device tensor -> float64 numpy (exact for fp32/bf16/fp16 values)"""
    return t.detach().float().cpu().double().numpy()


def rounded(a, dtype):
    """what the kernel sees: the fp64 input rounded to the activation dtype"""
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(dtype).double().numpy()


def err(a, b):
    return O.max_rel_err(back(a) if torch.is_tensor(a) else a, b)


def assert_close(name, got, want, tol, extra=""):
    e = err(got, want)
    assert np.isfinite(e) and e <= tol, f"{name}: max rel err {e:.3e} > {tol:.1e} {extra}"
    return e


def case56(variant, B, T, H, dtype, seed, state=True, gstate=True, x_shift=0.0):
    c = inputs.wkv56_case(variant, B, T, H, 64, seed, state=state, gstate=gstate)
    if x_shift:
        c["x"] = c["x"] + x_shift
    q = dict(c)
    for n in ("r", "k", "v", "gy", "u"):
        q[n] = rounded(c[n], dtype)
    q["x"] = rounded(c["x"], dtype) if variant == "v6" else rounded(c["x"], torch.float32)
    q["state_in"] = rounded(c["state_in"], torch.float32)
    q["gstate_out"] = rounded(c["gstate_out"], torch.float32)
    return q


def oracle56(variant, q):
    fwd = O.wkv6_fwd_x if variant == "v6" else O.wkv5_fwd_x
    bwd = O.wkv6_bwd_x if variant == "v6" else O.wkv5_bwd_x
    y, so = fwd(q["r"], q["k"], q["v"], q["x"], q["u"], q["state_in"])
    g = bwd(q["r"], q["k"], q["v"], q["x"], q["u"], q["state_in"], q["gy"], q["gstate_out"])
    g["y"], g["state_out"] = y, so
    return g
