"""The time-mix blocks that call the WKV op, with the op and its elementwise neighbours on the
library's kernels.

``RWKV_TimeMix6_0``  mirrors RWKV-v6/src/module/TimeMix.py:121-300 (``_forward_cuda``)
``RWKV_TimeMix``     mirrors RWKV-v5/src/module/TimeMix.py:161-323 (``_forward_cuda``)
``RWKV_TimeMix_v4``  mirrors ``RWKV_TimeMix`` of RWKV-v4neo/src/model.py:197-279, with its
                     ``TimeMixState`` (RWKV-v4neo/src/model.py:138-142)

Same constructor arguments, same parameter names and shapes (a state_dict of the project's
module loads), same ``forward(x, last_state) -> (out, (shift_state, wkv_state))``.  What is
different from the project's blocks:

* token shift + (data-dependent) lerp, GroupNorm * gate are one fused kernel each
  (``timemix.ddlerp``, ``timemix.lnx_gate``); the projections stay library GEMMs;
* the WKV state is fp32 ``[B,H,64,64]`` indexed [key,value], per batch row, returned as a new
  tensor that carries its gradient: segments of one sequence can be chained without
  truncating back-propagation (the project's v6 block cannot: RWKV-v6/src/model.py:291-299);
* the block computes in bf16: ``x`` is cast to bf16 and so is every parameter at its point of
  use (what autocast does for the project's block); parameters may be kept in fp32.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .timemix import ddlerp, lnx_gate
from .wkv4 import wkv_op
from .wkv5 import WKV5
from .wkv6 import WKV6

BF16 = torch.bfloat16
HEAD_SIZE_DIVISOR = 8


def _layer_ratios(layer_id, n_layer):
    r01 = layer_id / max(n_layer - 1, 1)
    r1a0 = 1.0 - layer_id / n_layer
    return r01, r1a0


def _decay_speed(dim_att, r01):
    n = torch.arange(dim_att, dtype=torch.float32) / max(dim_att - 1, 1)
    return -6.0 + 5.0 * n.pow(0.7 + 1.3 * r01)


def _bonus(dim_att, r01):
    n = torch.arange(dim_att, dtype=torch.float32)
    zigzag = ((n + 1) % 3 - 1) * 0.1
    return r01 * (1.0 - n / max(dim_att - 1, 1)) + zigzag


def _lin(x, layer):
    return F.linear(x, layer.weight.to(x.dtype))


class _TimeMixBase(nn.Module):
    def _common(self, layer_id, n_layer, n_embd, n_head, head_size, dim_att):
        if head_size != 64 or dim_att != n_head * head_size:
            raise ValueError("head_size must be 64 and dim_att = n_head * 64")
        self.layer_id, self.n_layer, self.n_embd, self.dim_att = layer_id, n_layer, n_embd, dim_att
        self.n_head, self.head_size, self.head_size_divisor = n_head, head_size, HEAD_SIZE_DIVISOR
        self.receptance = nn.Linear(n_embd, dim_att, bias=False)
        self.key = nn.Linear(n_embd, dim_att, bias=False)
        self.value = nn.Linear(n_embd, dim_att, bias=False)
        self.output = nn.Linear(dim_att, n_embd, bias=False)
        self.gate = nn.Linear(n_embd, dim_att, bias=False)

    @staticmethod
    def _inputs(x, last_state):
        shift, wkv_state = last_state
        x = x.to(BF16).contiguous()
        return x, shift.to(BF16).contiguous(), wkv_state


class RWKV_TimeMix6_0(_TimeMixBase):
    """v6 block.  ``chunk_len``, ``precision`` (parameters of the project's pure-PyTorch path) and
    ``max_ctx_len`` (a compile-time bound of its kernel) are accepted and have no effect here."""

    def __init__(self, layer_id, n_layer, n_embd, n_head, head_size, dim_att, chunk_len: int = 128,
                 precision: int = 64, max_ctx_len: int = 4096):
        super().__init__()
        self._common(layer_id, n_layer, n_embd, n_head, head_size, dim_att)
        self.chunk_len, self.precision, self.max_ctx_len = chunk_len, precision, max_ctx_len
        r01, r1a0 = _layer_ratios(layer_id, n_layer)
        with torch.no_grad():
            ddd = (torch.arange(n_embd, dtype=torch.float32) / n_embd).view(1, 1, n_embd)
            base, half = 1.0 - ddd.pow(r1a0), 1.0 - ddd.pow(0.5 * r1a0)
            self.time_maa_x = nn.Parameter(base.clone())
            self.time_maa_w = nn.Parameter(base.clone())
            self.time_maa_k = nn.Parameter(base.clone())
            self.time_maa_v = nn.Parameter(base - 0.3 * r01)
            self.time_maa_r = nn.Parameter(half.clone())
            self.time_maa_g = nn.Parameter(half.clone())
            mix_dim, decay_dim = 32, 64
            self.time_maa_w1 = nn.Parameter(torch.empty(n_embd, mix_dim * 5).uniform_(-1e-4, 1e-4))
            self.time_maa_w2 = nn.Parameter(torch.zeros(5, mix_dim, n_embd))
            self.time_decay = nn.Parameter(_decay_speed(dim_att, r01).view(1, 1, dim_att))
            self.time_decay_w1 = nn.Parameter(torch.empty(n_embd, decay_dim).uniform_(-1e-4, 1e-4))
            self.time_decay_w2 = nn.Parameter(torch.zeros(decay_dim, n_embd))
            self.time_faaaa = nn.Parameter(_bonus(dim_att, r01).view(n_head, head_size))
        self.ln_x = nn.GroupNorm(n_head, dim_att, eps=1e-5 * HEAD_SIZE_DIVISOR ** 2)

    def forward(self, x, last_state):
        x, shift, wkv_state = self._inputs(x, last_state)
        B, T, C = x.shape
        H = self.n_head
        # the five mixes: a first lerp feeds the low-rank map that makes them data-dependent
        xxx = ddlerp(x, shift, self.time_maa_x.view(1, C))[0]
        xxx = torch.tanh(xxx @ self.time_maa_w1.to(BF16)).view(B * T, 5, -1).transpose(0, 1)
        m = torch.bmm(xxx, self.time_maa_w2.to(BF16)).view(5, B, T, C)
        maa = torch.cat((self.time_maa_w, self.time_maa_k, self.time_maa_v, self.time_maa_r,
                         self.time_maa_g), 0).view(5, C)
        xw, xk, xv, xr, xg = ddlerp(x, shift, maa, m).unbind(0)
        r, k, v = _lin(xr, self.receptance), _lin(xk, self.key), _lin(xv, self.value)
        g = F.silu(_lin(xg, self.gate))
        w = self.time_decay.to(BF16) + torch.tanh(xw @ self.time_decay_w1.to(BF16)) @ self.time_decay_w2.to(BF16)
        y, wkv_state = WKV6.apply(B, T, self.dim_att, H, r, k, v, w, self.time_faaaa, wkv_state)
        y = lnx_gate(y, g, self.ln_x.weight, self.ln_x.bias, self.ln_x.eps, H)
        return _lin(y, self.output), (x[:, -1], wkv_state)


class RWKV_TimeMix(_TimeMixBase):
    """v5 block (static per-channel decay, static token-shift mixes)."""

    def __init__(self, layer_id, n_layer, n_embd, n_head, head_size, dim_att, chunk_len: int = 128,
                 precision: int = 64):
        super().__init__()
        self._common(layer_id, n_layer, n_embd, n_head, head_size, dim_att)
        self.chunk_len, self.precision = chunk_len, precision
        r01, r1a0 = _layer_ratios(layer_id, n_layer)
        with torch.no_grad():
            ddd = (torch.arange(n_embd, dtype=torch.float32) / n_embd).view(1, 1, n_embd)
            self.time_mix_k = nn.Parameter(ddd.pow(r1a0))
            self.time_mix_v = nn.Parameter(ddd.pow(r1a0) + 0.3 * r01)
            self.time_mix_r = nn.Parameter(ddd.pow(0.5 * r1a0))
            self.time_mix_g = nn.Parameter(ddd.pow(0.5 * r1a0))
            self.time_decay = nn.Parameter(_decay_speed(dim_att, r01).view(n_head, head_size))
            self.time_faaaa = nn.Parameter(_bonus(dim_att, r01).view(n_head, head_size))
        self.ln_x = nn.GroupNorm(n_head, dim_att)

    def forward(self, x, last_state):
        x, shift, wkv_state = self._inputs(x, last_state)
        B, T, C = x.shape
        H = self.n_head
        # x*mix + x_prev*(1-mix)  =  x + (x_prev - x)*(1-mix)
        maa = 1.0 - torch.cat((self.time_mix_k, self.time_mix_v, self.time_mix_r, self.time_mix_g), 0).view(4, C)
        xk, xv, xr, xg = ddlerp(x, shift, maa).unbind(0)
        r, k, v = _lin(xr, self.receptance), _lin(xk, self.key), _lin(xv, self.value)
        g = F.silu(_lin(xg, self.gate))
        y, wkv_state = WKV5.apply(B, T, self.dim_att, H, r, k, v, self.time_decay, self.time_faaaa, wkv_state)
        # ln_x(y / 8) with eps  ==  GroupNorm(y) with eps * 64
        y = lnx_gate(y, g, self.ln_x.weight, self.ln_x.bias, self.ln_x.eps * HEAD_SIZE_DIVISOR ** 2, H)
        return _lin(y, self.output), (x[:, -1], wkv_state)


class TimeMixState:
    """(shift_state [B,C], wkv_state [B,C,3]) of the v4 block."""

    def __init__(self, shift_state: torch.Tensor, wkv_state: torch.Tensor):
        self.shift_state = shift_state
        self.wkv_state = wkv_state


class RWKV_TimeMix_v4(nn.Module):
    """v4 block: three static token-shift mixes (one fused pass), k/v/r projections, the v4 WKV op
    (``rwkv::wkv`` with the raw ``time_decay`` / ``time_first``), sigmoid(r) gate, output projection.
    ``forward(x, TimeMixState) -> (out, TimeMixState)``; the wkv state is fp32 ``[B,C,3]`` and
    carries its gradient (in the op's max-shifted convention) to the previous segment."""

    def __init__(self, layer_id, n_layer, n_embd, dim_att):
        super().__init__()
        self.layer_id, self.n_layer, self.n_embd, self.dim_att = layer_id, n_layer, n_embd, dim_att
        r01, r1a0 = _layer_ratios(layer_id, n_layer)
        with torch.no_grad():
            h = torch.arange(dim_att, dtype=torch.float32)
            self.time_decay = nn.Parameter(-5.0 + 8.0 * (h / max(dim_att - 1, 1)).pow(0.7 + 1.3 * r01))
            self.time_first = nn.Parameter(torch.full((dim_att,), 0.3).log() + ((h + 1) % 3 - 1) * 0.5)
            ddd = (torch.arange(n_embd, dtype=torch.float32) / n_embd).view(1, 1, n_embd)
            self.time_mix_k = nn.Parameter(ddd.pow(r1a0))
            self.time_mix_v = nn.Parameter(ddd.pow(r1a0) + 0.3 * r01)
            self.time_mix_r = nn.Parameter(ddd.pow(0.5 * r1a0))
        self.key = nn.Linear(n_embd, dim_att, bias=False)
        self.value = nn.Linear(n_embd, dim_att, bias=False)
        self.receptance = nn.Linear(n_embd, dim_att, bias=False)
        self.output = nn.Linear(dim_att, n_embd, bias=False)

    def forward(self, x, last_state: TimeMixState):
        x = x.to(BF16).contiguous()
        C = x.shape[-1]
        # x*mix + x_prev*(1-mix)  =  x + (x_prev - x)*(1-mix)
        maa = 1.0 - torch.cat((self.time_mix_k, self.time_mix_v, self.time_mix_r), 0).view(3, C)
        xk, xv, xr = ddlerp(x, last_state.shift_state.to(BF16).contiguous(), maa).unbind(0)
        k, v = _lin(xk, self.key), _lin(xv, self.value)
        sr = torch.sigmoid(_lin(xr, self.receptance))
        y, new_wkv_state = wkv_op(self.time_decay, self.time_first.to(BF16), k, v, last_state.wkv_state)
        return _lin(sr * y, self.output), TimeMixState(x[:, -1], new_wkv_state)
