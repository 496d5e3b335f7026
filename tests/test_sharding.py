"""Host-side multi-GPU logic on CPU: the (batch x head) partition and the whole-job
aggregation, the latter across two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rwkv_infctx_trainer_b200.sharding import aggregate_throughput, shard_units


@pytest.mark.parametrize("B,H,world", [(4, 64, 1), (4, 64, 2), (4, 64, 8), (1, 40, 8), (8, 3, 8),
                                       (5, 2, 7), (2, 1, 2)])
def test_shards_are_disjoint_and_cover_every_unit(B, H, world):
    seen = set()
    for rank in range(world):
        s = shard_units(B, H, world, rank)
        for b in range(s.b0, s.b1):
            for h in range(s.h0, s.h1):
                assert (b, h) not in seen
                seen.add((b, h))
    assert len(seen) == B * H
    if world <= H:  # heads first: every rank keeps the whole batch, sizes differ by at most one head
        sizes = [shard_units(B, H, world, r).h1 - shard_units(B, H, world, r).h0 for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
        assert all(shard_units(B, H, world, r).b1 - shard_units(B, H, world, r).b0 == B for r in range(world))


def test_benchmark_shapes():
    assert shard_units(4, 64, 8, 3) == (0, 4, 24, 32)       # 7B shape: 8 heads per GPU
    assert shard_units(1, 40, 8, 7) == (0, 1, 35, 40)       # long-context shape: 5 heads per GPU


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        s = shard_units(4, 64, world, rank)
        units, ms = aggregate_throughput(s.units * 4096, 10.0 + 5.0 * rank)
        out[rank] = (units, ms)
    finally:
        dist.destroy_process_group()


def test_aggregate_over_two_gloo_ranks():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for r in range(2):
        units, ms = out[r]
        assert units == 4 * 64 * 4096       # both shards together = every unit
        assert ms == 15.0                   # the slower rank sets the time


def test_aggregate_without_process_group_is_identity():
    assert aggregate_throughput(7.0, 3.0) == (7.0, 3.0)
