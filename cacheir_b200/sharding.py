"""Data parallelism by sequence: the only multi-GPU form the batched decode step needs.

Each rank owns a replica of the weights and its own KV page pool; the decode step of one
sequence never reads another sequence's pages, so requests are partitioned across ranks and
the data path has no collective. What crosses ranks is control-plane only: the generated
token streams gathered for the caller, and scalar reductions for timing (max over ranks)
and throughput (sum over ranks). Those go through ``torch.distributed`` with whatever
backend the process group was created with (NCCL on GPUs, gloo in the CPU tests).

The reference runs one process on one device (its continuous-batching scheduler,
cacheir/runtime/scheduler.py:160-208, has no multi-device form); this module is the
multi-GPU extension of that launcher and keeps its request/result vocabulary.
"""
from __future__ import annotations

from typing import Any, Callable, Mapping, Sequence

import torch
import torch.distributed as dist


def _world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_range(total: int, world_size: int, rank: int) -> range:
    """Contiguous, balanced slice of ``range(total)`` owned by ``rank``.

    The first ``total % world_size`` ranks get one extra item; every index is owned by
    exactly one rank and the slices are in rank order, so concatenating the per-rank
    results restores request order.
    """
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if total < 0:
        raise ValueError("total must be non-negative")
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_requests(requests: Sequence[Any], world_size: int | None = None, rank: int | None = None) -> list[Any]:
    """The requests this rank decodes."""
    r, w = _world()
    rank = r if rank is None else rank
    world_size = w if world_size is None else world_size
    return [requests[i] for i in shard_range(len(requests), world_size, rank)]


def gather_token_streams(local: Mapping[str, list[int]]) -> dict[str, list[int]]:
    """Union of every rank's ``{request id: tokens}``; identical on all ranks, rank order kept."""
    _, world = _world()
    if world == 1:
        return dict(local)
    parts: list[Any] = [None] * world
    dist.all_gather_object(parts, dict(local))
    merged: dict[str, list[int]] = {}
    for part in parts:
        for rid, tokens in part.items():
            if rid in merged:
                raise ValueError(f"request {rid!r} was decoded by more than one rank")
            merged[rid] = list(tokens)
    return merged


def _reduce_scalar(value: float, op: Any, device: torch.device | None) -> float:
    _, world = _world()
    if world == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or torch.device("cpu"))
    dist.all_reduce(t, op=op)
    return float(t.item())


def max_over_ranks(value: float, device: torch.device | None = None) -> float:
    """Slowest rank's time: the figure every multi-GPU timing reports."""
    return _reduce_scalar(value, dist.ReduceOp.MAX, device)


def sum_over_ranks(value: float, device: torch.device | None = None) -> float:
    """Whole-job count (tokens, sequences) from per-rank counts."""
    return _reduce_scalar(value, dist.ReduceOp.SUM, device)


def run_sharded(requests: Sequence[tuple[str, list[int]]], decode: Callable[[list[tuple[str, list[int]]]], Mapping[str, list[int]]]
                ) -> dict[str, list[int]]:
    """Decode ``requests`` ((request id, prompt ids) pairs) with one launcher per rank.

    ``decode`` runs this rank's share (typically ``BatchedDecodeLauncher`` submit +
    ``run_until_complete``) and returns ``{request id: tokens}``; the result is the merged
    mapping in the original request order, the same on every rank.
    """
    mine = shard_requests(list(requests))
    local = decode(mine) if mine else {}
    merged = gather_token_streams(local)
    return {rid: merged[rid] for rid, _ in requests if rid in merged}
