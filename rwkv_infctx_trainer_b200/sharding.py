"""Splitting one WKV call across the GPUs of a node.

Every (batch row, head) pair is an independent recurrence (the reference kernels map one
CUDA block to each: RWKV-v5/src/module/cuda/wkv5_cuda.cu:137-139), so the op shards with no
exchange step.  Heads are split first: a rank then owns whole rows of the per-head
parameters ``u`` / ``w`` and their gradients need no reduction; the batch is split only when
there are more ranks than heads.  The recurrent state shard ``[B_local, H_local, 64, 64]``
stays on its GPU across BPTT segments.
"""
from __future__ import annotations

from typing import NamedTuple


class Shard(NamedTuple):
    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def units(self) -> int:
        return (self.b1 - self.b0) * (self.h1 - self.h0)


def _split(n: int, parts: int, idx: int) -> tuple[int, int]:
    base, rem = divmod(n, parts)
    lo = idx * base + min(idx, rem)
    return lo, lo + base + (1 if idx < rem else 0)


def shard_units(B: int, H: int, world: int, rank: int) -> Shard:
    """The (batch range, head range) that ``rank`` of ``world`` owns."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    if world <= H:
        h0, h1 = _split(H, world, rank)
        return Shard(0, B, h0, h1)
    # more ranks than heads: groups of ranks share a head and split the batch
    per_head = world // H
    extra = world - per_head * H          # the first `extra` heads get one more rank
    bound = extra * (per_head + 1)
    if rank < bound:
        head, sub, parts = rank // (per_head + 1), rank % (per_head + 1), per_head + 1
    else:
        head, sub, parts = extra + (rank - bound) // per_head, (rank - bound) % per_head, per_head
    b0, b1 = _split(B, parts, sub)
    return Shard(b0, b1, head, head + 1)


def aggregate_throughput(units_local: float, elapsed_ms_local: float, device=None) -> tuple[float, float]:
    """Whole-job (units, elapsed_ms): units summed over ranks, time = max over ranks.
    Works on any initialised torch.distributed backend (NCCL on GPUs, gloo on CPU);
    without a process group it returns the local values."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(units_local), float(elapsed_ms_local)
    t = torch.tensor([elapsed_ms_local], dtype=torch.float64, device=device)
    u = torch.tensor([units_local], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return float(u.item()), float(t.item())
