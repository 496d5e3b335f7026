"""Generate ``timemix_v4.npz`` / ``timemix_v5.npz`` / ``timemix_v6.npz`` from the RWKV-infctx-trainer
project's own time-mix blocks (RWKV-v4neo/src/model.py ``RWKV_TimeMix``, RWKV-v5/src/module/TimeMix.py
``RWKV_TimeMix``, RWKV-v6/src/module/TimeMix.py ``RWKV_TimeMix6_0``), run on the CPU: v5 and v6 in fp32
through their pure-PyTorch WKV path; v4, whose WKV op exists in CUDA only, with that one op stood in
for by a token-by-token fp64 recurrence (``cpu_wkv4``) -- the v4 fixture pins the block around the op,
the op itself is held to the project's CUDA kernel by the GPU tests.

    python tests/golden/make_golden_timemix.py

Each block is built for layer 1 of 4 with n_embd = 128 (2 heads), its parameters are replaced by
seeded values (the project's initialisation leaves the low-rank maps at zero, which would hide
them), and it is driven over a 256-token sequence cut into two 128-token segments with the
(shift, wkv) state carried WITH its gradient.  Stored: the parameters, the output, the final
state, and the gradients of ``sum(out * gout) + sum(state * gstate)`` w.r.t. the input, the
initial state and every parameter; and (``init.*``) the deterministic part of the project's
parameter initialisation.  The input and the two cotangents are rebuilt from ``inputs.py`` by
the test.
"""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import inputs  # noqa: E402
import make_golden as mg  # noqa: E402

B, T, SEG, C, H, LAYER, NLAYER = 2, 256, 128, 128, 2, 1, 4


def load_block(version_dir, cls):
    os.environ["RWKV_NO_CUDA"] = "1"
    mg.load_rwkv_inner(version_dir)          # sets up the stubs and the `src` package for this version
    return getattr(importlib.import_module("src.module.TimeMix"), cls)


def seeded_parameters(block, seed):
    """Replace every parameter: projections ~ N(0, 1/sqrt(fan_in)), low-rank maps ~ N(0, 0.1), mixes in
    (0, 1), decay in (-6, -0.5), bonus in (-1, 1), GroupNorm weight ~ 1 +- 0.2, bias ~ +- 0.2."""
    with torch.no_grad():
        for i, (name, p) in enumerate(sorted(block.named_parameters())):
            shape = tuple(p.shape)
            if name.endswith(".weight") and p.dim() == 2:
                a = inputs.normal(shape, seed, std=shape[1] ** -0.5, stream=20 + i)
            elif name in ("time_maa_w1", "time_maa_w2", "time_decay_w1", "time_decay_w2"):
                a = inputs.normal(shape, seed, std=0.1, stream=20 + i)
            elif name.startswith("time_maa") or name.startswith("time_mix"):
                a = inputs.uniform(shape, seed, 0.05, 0.95, stream=20 + i)
            elif name == "time_decay":
                a = inputs.uniform(shape, seed, -6.0, -0.5, stream=20 + i)
            elif name in ("time_faaaa", "time_first"):
                a = inputs.uniform(shape, seed, -1.0, 1.0, stream=20 + i)
            elif name == "ln_x.weight":
                a = 1.0 + inputs.uniform(shape, seed, -0.2, 0.2, stream=20 + i)
            elif name == "ln_x.bias":
                a = inputs.uniform(shape, seed, -0.2, 0.2, stream=20 + i)
            else:
                raise KeyError(name)
            p.copy_(torch.tensor(a, dtype=torch.float32))


def block_inputs(seed):
    """x ~ N(0,1), initial shift ~ N(0,1), initial wkv state ~ N(0,0.5), and the two cotangents"""
    return dict(
        x=inputs.normal((B, T, C), seed, stream=1), shift=inputs.normal((B, C), seed, stream=2),
        state=inputs.normal((B, H, 64, 64), seed, std=0.5, stream=3),
        gout=inputs.normal((B, T, C), seed, stream=4), gstate=inputs.normal((B, H, 64, 64), seed, std=0.1, stream=5))


def cpu_wkv4(w, u, k, v, last_state):
    """The v4 recurrence of RWKV-v4neo/cuda/wkv_cuda_bf16.cu:7-53 in plain torch (fp64, token by token,
    differentiable by autograd), standing in for the project's CUDA-only op `rwkv::wkv` so that the
    project's v4 block can run on the CPU: w is the raw time_decay (the op uses -exp(w),
    wkv_op_bf16.cpp:34), state = (aa, bb, pp) with pp the running maximum of the exponents."""
    wd = -torch.exp(w.double())
    ud, kd, vd = u.double(), k.double(), v.double()
    aa, bb, pp = last_state.double().unbind(-1)
    ys = []
    for t in range(kd.shape[1]):
        kt, vt = kd[:, t], vd[:, t]
        ww = ud + kt
        p = torch.maximum(pp, ww)
        e1, e2 = torch.exp(pp - p), torch.exp(ww - p)
        ys.append((e1 * aa + e2 * vt) / (e1 * bb + e2))
        ww = wd + pp
        p = torch.maximum(ww, kt)
        e1, e2 = torch.exp(ww - p), torch.exp(kt - p)
        aa, bb, pp = e1 * aa + e2 * vt, e1 * bb + e2, p
    return [torch.stack(ys, 1).to(k.dtype), torch.stack((aa, bb, pp), -1).float()]


def make_v4():
    """The v4 block (RWKV-v4neo/src/model.py:197-279), bf16 k/v/time_first as that code forces them."""
    os.environ["RWKV_JIT_ON"] = "0"
    os.environ["RWKV_TORCH_COMPILE"] = "0"
    mg._stub_trainer_packages()
    sys.modules["lightning"].LightningModule = torch.nn.Module
    for name in [n for n in sys.modules if n == "src" or n.startswith("src.")]:
        del sys.modules[name]
    import types
    m = types.ModuleType("src")
    m.__path__ = [os.path.join(mg.REF_ROOT, "RWKV-v4neo", "src")]
    sys.modules["src"] = m
    model = importlib.import_module("src.model")
    torch.library.define("rwkv::wkv", "(Tensor w, Tensor u, Tensor k, Tensor v, Tensor last_state) -> Tensor[]")
    torch.library.impl("rwkv::wkv", "CompositeImplicitAutograd")(cpu_wkv4)
    seed, name = 33, "timemix_v4"
    block = model.RWKV_TimeMix(LAYER, NLAYER, C, C).float()
    init = {"init." + n: p.detach().clone() for n, p in block.named_parameters() if n.startswith("time_")}
    seeded_parameters(block, seed)
    block.time_first.data = block.time_first.data.to(torch.bfloat16)     # (the block's forward insists on it)
    d = {k: torch.tensor(v, dtype=torch.float32) for k, v in block_inputs(seed).items()}
    wkv0 = torch.stack((torch.tensor(inputs.normal((B, C), seed, stream=6), dtype=torch.float32),
                        torch.tensor(inputs.uniform((B, C), seed, 0.5, 1.5, stream=7), dtype=torch.float32),
                        torch.tensor(inputs.uniform((B, C), seed, -1.0, 1.0, stream=8), dtype=torch.float32)), -1)
    x = d["x"].clone().requires_grad_(True)
    shift0 = d["shift"].clone().requires_grad_(True)
    state, outs = model.TimeMixState(shift0, wkv0), []
    for t0 in range(0, T, SEG):
        o, state = block(x[:, t0:t0 + SEG], state)
        outs.append(o)
    out = torch.cat(outs, 1)
    loss = (out * d["gout"]).sum()
    params = dict(block.named_parameters())
    leaves = [x, shift0] + [params[n] for n in sorted(params)]
    grads = torch.autograd.grad(loss, leaves)
    rec = dict(out=out.detach(), state_out=state.wkv_state.detach(), wkv_state_in=wkv0, gx=grads[0], gshift=grads[1])
    for n, g in zip(sorted(params), grads[2:]):
        rec["param." + n] = params[n].detach()
        rec["grad." + n] = g
    rec.update(init)
    rec = {k: v.float().numpy().astype(np.float32) for k, v in rec.items()}
    meta = dict(B=B, T=T, seg=SEG, C=C, H=H, layer=LAYER, n_layer=NLAYER, seed=seed, cls="RWKV_TimeMix_v4")
    np.savez_compressed(os.path.join(HERE, name + ".npz"), meta=np.array(repr(meta)), **rec)
    print(name, "out", tuple(rec["out"].shape), "max|out|", float(np.abs(rec["out"]).max()),
          {k: float(np.abs(v).max()) for k, v in rec.items() if k.startswith("grad.")})


def main():
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    make_v4()
    for name, vdir, cls, seed in (("timemix_v5", "RWKV-v5", "RWKV_TimeMix", 31),
                                  ("timemix_v6", "RWKV-v6", "RWKV_TimeMix6_0", 32)):
        Block = load_block(vdir, cls)
        block = Block(LAYER, NLAYER, C, H, 64, C).float()
        # the deterministic part of the project's initialisation (the rest is random)
        init = {"init." + n: p.detach().clone() for n, p in block.named_parameters()
                if n.startswith("time_") and not n.endswith(("_w1", "_w2"))}
        seeded_parameters(block, seed)
        d = {k: torch.tensor(v, dtype=torch.float32) for k, v in block_inputs(seed).items()}
        x = d["x"].clone().requires_grad_(True)
        shift0 = d["shift"].clone().requires_grad_(True)
        state0 = d["state"].clone().requires_grad_(True)
        state, outs = (shift0, state0), []
        for t0 in range(0, T, SEG):
            o, state = block(x[:, t0:t0 + SEG], state)
            outs.append(o)
        out = torch.cat(outs, 1)
        loss = (out * d["gout"]).sum() + (state[1] * d["gstate"]).sum()
        params = dict(block.named_parameters())
        leaves = [x, shift0, state0] + [params[n] for n in sorted(params)]
        grads = torch.autograd.grad(loss, leaves)
        rec = dict(out=out.detach(), state_out=state[1].detach(), gx=grads[0], gshift=grads[1], gstate_in=grads[2])
        for n, g in zip(sorted(params), grads[3:]):
            rec["param." + n] = params[n].detach()
            rec["grad." + n] = g
        rec.update(init)
        rec = {k: v.numpy().astype(np.float32) for k, v in rec.items()}
        meta = dict(B=B, T=T, seg=SEG, C=C, H=H, layer=LAYER, n_layer=NLAYER, seed=seed, cls=cls)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), meta=np.array(repr(meta)), **rec)
        print(name, "out", tuple(rec["out"].shape), "max|out|", float(np.abs(rec["out"]).max()),
              {k: float(np.abs(v).max()) for k, v in rec.items() if k.startswith("grad.")})


if __name__ == "__main__":
    main()
