"""The time-mix blocks (`RWKV_TimeMix`, `RWKV_TimeMix6_0`) against fixtures made from the
RWKV-infctx-trainer project's own blocks (tests/golden/make_golden_timemix.py: the project's
modules, fp32, CPU, pure-PyTorch WKV path).  Ours run in bf16 on the fused kernels; the
sequence is cut into two segments and the (shift, wkv) state carries its gradient, as in the
fixture.  Tolerance: bf16 I/O, 3e-2 of the largest reference value per tensor.
"""
import ast
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import inputs  # noqa: E402

TOL = 3e-2


def _load(name):
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    return ast.literal_eval(str(z["meta"])), z


def _block_inputs(meta):
    B, T, C, H, seed = meta["B"], meta["T"], meta["C"], meta["H"], meta["seed"]
    return dict(
        x=inputs.normal((B, T, C), seed, stream=1), shift=inputs.normal((B, C), seed, stream=2),
        state=inputs.normal((B, H, 64, 64), seed, std=0.5, stream=3),
        gout=inputs.normal((B, T, C), seed, stream=4), gstate=inputs.normal((B, H, 64, 64), seed, std=0.1, stream=5))


def _new_block(W, meta):
    cls = getattr(W, meta["cls"])
    if meta["cls"] == "RWKV_TimeMix_v4":
        return cls(meta["layer"], meta["n_layer"], meta["C"], meta["C"])
    return cls(meta["layer"], meta["n_layer"], meta["C"], meta["H"], 64, meta["C"])


def _make(meta, z, device):
    import rwkv_infctx_trainer_b200 as W
    block = _new_block(W, meta)
    sd = {k[len("param."):]: torch.tensor(z[k]) for k in z.files if k.startswith("param.")}
    block.load_state_dict(sd, strict=True)      # same names and shapes as the project's block
    return block.to(device)


@pytest.mark.parametrize("name", ["timemix_v4", "timemix_v5", "timemix_v6"])
def test_state_dict_of_the_reference_block_loads(name):
    meta, z = _load(name)
    block = _make(meta, z, "cpu")
    assert sorted(n for n, _ in block.named_parameters()) == sorted(
        k[len("param."):] for k in z.files if k.startswith("param."))


@pytest.mark.parametrize("name", ["timemix_v4", "timemix_v5", "timemix_v6"])
def test_default_initialisation_is_the_reference_blocks(name):
    import rwkv_infctx_trainer_b200 as W
    meta, z = _load(name)
    block = _new_block(W, meta)
    params = dict(block.named_parameters())
    checked = 0
    for k in z.files:
        if k.startswith("init."):
            ref = torch.tensor(z[k])
            assert params[k[5:]].shape == ref.shape
            assert torch.allclose(params[k[5:]].detach(), ref, rtol=1e-5, atol=1e-6), k
            checked += 1
    assert checked >= 5


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["timemix_v5", "timemix_v6"])
def test_block_matches_reference_block(name):
    meta, z = _load(name)
    block = _make(meta, z, "cuda")
    d = {k: torch.tensor(v, dtype=torch.float32, device="cuda") for k, v in _block_inputs(meta).items()}
    x = d["x"].clone().requires_grad_(True)
    shift0 = d["shift"].clone().requires_grad_(True)
    state0 = d["state"].clone().requires_grad_(True)
    state, outs = (shift0, state0), []
    for t0 in range(0, meta["T"], meta["seg"]):
        o, state = block(x[:, t0:t0 + meta["seg"]], state)
        outs.append(o)
    out = torch.cat(outs, 1)
    assert out.dtype == torch.bfloat16 and state[1].dtype == torch.float32
    loss = (out.float() * d["gout"]).sum() + (state[1] * d["gstate"]).sum()
    params = dict(block.named_parameters())
    names = sorted(params)
    grads = torch.autograd.grad(loss, [x, shift0, state0] + [params[n] for n in names])
    got = dict(out=out, state_out=state[1], gx=grads[0], gshift=grads[1], gstate_in=grads[2])
    got.update({"grad." + n: g for n, g in zip(names, grads[3:])})
    worst = {}
    for k, g in got.items():
        ref = torch.tensor(z[k], device="cuda")
        worst[k] = float((g.detach().float().view_as(ref) - ref).abs().max() / ref.abs().max().clamp_min(1e-20))
    bad = {k: v for k, v in worst.items() if not v <= TOL}
    assert not bad, (bad, worst)


@pytest.mark.gpu
def test_v4_block_matches_reference_block():
    """the v4 block around the op (RWKV-v4neo/src/model.py:197-279): two chained segments, the wkv
    state carried with its gradient; the gradient w.r.t. the initial wkv state is left out (the
    op reports it in its max-shifted convention, the fixture's autograd in the plain one)"""
    import rwkv_infctx_trainer_b200 as W
    meta, z = _load("timemix_v4")
    block = _make(meta, z, "cuda")
    d = {k: torch.tensor(v, dtype=torch.float32, device="cuda") for k, v in _block_inputs(meta).items()}
    x = d["x"].clone().requires_grad_(True)
    shift0 = d["shift"].clone().requires_grad_(True)
    state = W.TimeMixState(shift0, torch.tensor(z["wkv_state_in"], device="cuda"))
    outs = []
    for t0 in range(0, meta["T"], meta["seg"]):
        o, state = block(x[:, t0:t0 + meta["seg"]], state)
        outs.append(o)
    out = torch.cat(outs, 1)
    loss = (out.float() * d["gout"]).sum()
    params = dict(block.named_parameters())
    names = sorted(params)
    grads = torch.autograd.grad(loss, [x, shift0] + [params[n] for n in names])
    got = dict(out=out, gx=grads[0], gshift=grads[1])
    got.update({"grad." + n: g for n, g in zip(names, grads[2:])})
    worst = {}
    for k, g in got.items():
        ref = torch.tensor(z[k], device="cuda")
        worst[k] = float((g.detach().float().view_as(ref) - ref).abs().max() / ref.abs().max().clamp_min(1e-20))
    # the state after the last token: what it stands for, (aa, bb) e^{pp}, relative to the larger of the two
    so, ref = state.wkv_state.detach().double(), torch.tensor(z["state_out"], device="cuda").double()
    m = torch.maximum(so[..., 2], ref[..., 2])
    for i, nme in ((0, "state_out.aa"), (1, "state_out.bb")):
        a, b = so[..., i] * torch.exp(so[..., 2] - m), ref[..., i] * torch.exp(ref[..., 2] - m)
        worst[nme] = float((a - b).abs().max() / b.abs().max())
    bad = {k: v for k, v in worst.items() if not v <= TOL}
    assert not bad, (bad, worst)
