"""Generate the fixtures in this directory from the RWKV-infctx-trainer project's
own pure-PyTorch WKV path.

Run once, in a container that has the project checked out read-only (default
``/root/reference``; override with WKV_REFERENCE_ROOT):

    python tests/golden/make_golden.py

It imports ``rwkv_inner`` from RWKV-v5/src/module/rwkv_inner.py and
RWKV-v6/src/module/rwkv_inner.py (stubbing the trainer-only packages their
``CoreDependencies`` imports at module top), drives it the way the trainer's
BPTT loop does -- consecutive segments with the state carried, one backward over
the whole chain -- and stores the outputs and gradients as float32 ``.npz``.
Inputs are not stored: ``inputs.py`` rebuilds them from the seed.

The fixtures pin the CPU oracle (tests/test_oracle.py); the GPU parity tests
then compare the CUDA kernels with that oracle and with these fixtures.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import inputs  # noqa: E402

REF_ROOT = os.environ.get("WKV_REFERENCE_ROOT", "/root/reference")


def _stub_trainer_packages():
    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        m.__path__ = []
        sys.modules[name] = m
        return m
    ident = lambda f: f
    mod("lightning")
    mod("lightning.pytorch")
    mod("lightning.pytorch.utilities", rank_zero_info=print, rank_zero_only=ident)
    mod("lightning.pytorch.strategies", DeepSpeedStrategy=object)
    mod("deepspeed")
    mod("deepspeed.ops")
    mod("deepspeed.ops.adam", DeepSpeedCPUAdam=object, FusedAdam=object)
    mod("deepspeed.runtime")
    mod("deepspeed.runtime.lr_schedules")
    if "wandb" not in sys.modules:
        try:
            import wandb  # noqa: F401
        except Exception:
            mod("wandb")


def load_rwkv_inner(version_dir: str):
    """Import <project>/<version_dir>/src/module/rwkv_inner.py as its own package."""
    os.environ["RWKV_JIT_ON"] = "0"
    os.environ["RWKV_TORCH_COMPILE"] = "0"
    _stub_trainer_packages()
    for name in [n for n in sys.modules if n == "src" or n.startswith("src.")]:
        del sys.modules[name]
    root = os.path.join(REF_ROOT, version_dir)
    for pkg, path in (("src", os.path.join(root, "src")),
                      ("src.module", os.path.join(root, "src", "module"))):
        m = types.ModuleType(pkg)
        m.__path__ = [path]
        sys.modules[pkg] = m
    return importlib.import_module("src.module.rwkv_inner").rwkv_inner


def run_reference_chain(rwkv_inner, variant, case, H, N, seg_len):
    t = {n: torch.tensor(a, dtype=torch.float32) for n, a in case.items()}
    B, T, C = t["r"].shape
    leaves = [t[n].clone().requires_grad_(True) for n in ("r", "k", "v", "x", "u", "state_in")]
    r, k, v, x, u, s = leaves
    w = torch.exp(-torch.exp(x))
    state = s
    ys = []
    for t0 in range(0, T, seg_len):
        t1 = min(T, t0 + seg_len)
        sl = lambda a: a[:, t0:t1].reshape(B, t1 - t0, H, N).transpose(1, 2)
        ws = sl(w) if variant == "v6" else w.view(1, H, 1, N).expand(1, H, t1 - t0, N)
        o, state = rwkv_inner(sl(r), sl(k), sl(v), ws, u.view(1, H, 1, N), state, 128, 64)
        ys.append(o.transpose(1, 2).reshape(B, t1 - t0, C))
    y = torch.cat(ys, 1)
    loss = (y * t["gy"]).sum() + (state * t["gstate_out"]).sum()
    g = torch.autograd.grad(loss, leaves)
    out = dict(y=y.detach(), state_out=state.detach(), gr=g[0], gk=g[1], gv=g[2], gw=g[3],
               gu=g[4], gstate_in=g[5])
    return {n: a.numpy().astype(np.float32) for n, a in out.items()}


CASES = [
    # name, variant, project dir, B, T, H, N, seed, seg_len, state, gstate, token stride stored
    ("v5_small", "v5", "RWKV-v5", 2, 256, 2, 64, 11, 128, True, True, 1),
    ("v6_small", "v6", "RWKV-v6", 2, 256, 2, 64, 12, 128, True, True, 1),
    # the CPU-runnable benchmark case: B=2, T=512 as 4 segments of 128, H=4, N=64, zero state, seed 0
    ("v5_config0", "v5", "RWKV-v5", 2, 512, 4, 64, 0, 128, False, False, 4),
    ("v6_config0shape", "v6", "RWKV-v6", 2, 512, 4, 64, 0, 128, False, False, 4),
]


def main():
    torch.manual_seed(0)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name, variant, vdir, B, T, H, N, seed, seg, st, gst, stride in CASES:
        fn = load_rwkv_inner(vdir)
        case = inputs.wkv56_case(variant, B, T, H, N, seed, state=st, gstate=gst)
        out = run_reference_chain(fn, variant, case, H, N, seg)
        meta = dict(variant=variant, B=B, T=T, H=H, N=N, seed=seed, seg_len=seg,
                    state=st, gstate=gst, stride=stride)
        if stride > 1:
            for n in ("y", "gr", "gk", "gv"):
                out[n] = out[n][:, ::stride]
            if variant == "v6":
                out["gw"] = out["gw"][:, ::stride]
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            meta=np.array(repr(meta)), **out)
        print(name, {n: a.shape for n, a in out.items()})


if __name__ == "__main__":
    main()
