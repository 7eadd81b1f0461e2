"""Data-parallel decode over two ranks on CPU (gloo): the host logic that runs when N > 1.

The GPU kernels are not involved: each rank "decodes" its share with a deterministic
function of the prompt, which is enough to check that requests are partitioned without
overlap, that the merged result is complete, ordered and identical on every rank, and
that the timing and throughput reductions behave as the benchmark assumes.
"""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cacheir_b200.sharding import (gather_token_streams, max_over_ranks, run_sharded, shard_range, shard_requests,
                                   sum_over_ranks)


def test_shard_range_partitions_exactly():
    for total in (0, 1, 2, 7, 32, 33):
        for world in (1, 2, 3, 8):
            seen: list[int] = []
            sizes = []
            for rank in range(world):
                r = shard_range(total, world, rank)
                seen.extend(r)
                sizes.append(len(r))
            assert seen == list(range(total))
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
    with pytest.raises(ValueError):
        shard_range(-1, 2, 0)


def test_single_process_passthrough():
    reqs = [(f"r{i}", [i, i + 1]) for i in range(5)]
    assert shard_requests(reqs) == reqs
    assert gather_token_streams({"a": [1]}) == {"a": [1]}
    assert max_over_ranks(2.5) == 2.5 and sum_over_ranks(3.0) == 3.0
    out = run_sharded(reqs, lambda mine: {rid: [t * 2 for t in ids] for rid, ids in mine})
    assert list(out) == [rid for rid, _ in reqs]


def _fake_decode(mine):
    return {rid: [(sum(ids) * 31 + j) % 97 for j in range(4)] for rid, ids in mine}


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        reqs = [(f"req-{i}", [i, 2 * i + 1, 5]) for i in range(7)]
        mine = shard_requests(reqs)
        merged = run_sharded(reqs, _fake_decode)
        slow = max_over_ranks(1.0 + rank)                 # rank 1 is the slow one
        total = sum_over_ranks(float(len(mine)))
        dup_error = False
        try:                                              # the same request on two ranks is a bug, not a merge
            gather_token_streams({"dup": [rank]})
        except ValueError:
            dup_error = True
        results[rank] = {"mine": [rid for rid, _ in mine], "merged": merged, "slow": slow, "total": total,
                         "dup_error": dup_error}
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(120)
def test_two_ranks_partition_gather_and_reduce():
    world = 2
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.kill()
    assert not stuck and all(p.exitcode == 0 for p in procs)
    reqs = [(f"req-{i}", [i, 2 * i + 1, 5]) for i in range(7)]
    expected = _fake_decode(reqs)
    r0, r1 = results[0], results[1]
    assert r0["mine"] == [f"req-{i}" for i in range(4)] and r1["mine"] == [f"req-{i}" for i in range(4, 7)]
    assert r0["merged"] == expected and r1["merged"] == expected
    assert list(r0["merged"]) == [rid for rid, _ in reqs]           # request order survives the gather
    assert r0["slow"] == 2.0 and r1["slow"] == 2.0                  # every rank reports the slowest rank's time
    assert r0["total"] == 7.0 and r1["total"] == 7.0
    assert r0["dup_error"] and r1["dup_error"]
