"""Oscillator / channel sharding across GPUs (one process per GPU).

The scans have no cross-series dependency, so a layer with ``P`` oscillators (or
``D`` Mamba channels) is split into contiguous shards, each rank scans its own
shard, and nothing is exchanged on the data path.  The only collectives are an
optional all-gather of ``x`` when a caller wants the full state on every rank,
and the two scalar reductions a benchmark needs.  The reference has no
distributed code at all; this is new functionality whose oracle is the
single-device result.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

__all__ = ["shard_range", "shard_channels", "gather_channels", "aggregate_throughput"]


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous ``[start, stop)`` of ``total`` items owned by ``rank``; the first
    ``total % world`` ranks own one item more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_channels(t: torch.Tensor, world: int, rank: int, dim: int = -1) -> torch.Tensor:
    """This rank's contiguous slice of ``t`` along ``dim`` (a copy, so that the shard is dense)."""
    start, stop = shard_range(t.size(dim), world, rank)
    return t.narrow(dim, start, stop - start).contiguous()


def gather_channels(x_local: torch.Tensor, total: int, group=None) -> torch.Tensor:
    """All-gathers channel shards ``[..., P_rank]`` into ``[..., total]`` on every rank."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = [shard_range(total, world, r) for r in range(world)]
    widest = max(b - a for a, b in sizes)
    is_complex = x_local.is_complex()
    src = torch.view_as_real(x_local.contiguous()) if is_complex else x_local.contiguous()
    moved = src.movedim(-2 if is_complex else -1, 0)            # channel first
    pad = torch.zeros((widest,) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
    pad[: moved.size(0)] = moved
    parts: List[torch.Tensor] = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    full = torch.cat([p[: b - a] for p, (a, b) in zip(parts, sizes)], dim=0)
    full = full.movedim(0, -2 if is_complex else -1).contiguous()
    del rank
    return torch.view_as_complex(full) if is_complex else full


def aggregate_throughput(units_local: int, ms_local: float, device, group=None) -> Tuple[int, float]:
    """``(sum of units over ranks, max of milliseconds over ranks)`` -- whole-job
    throughput is the first divided by the second."""
    t = torch.tensor([float(units_local)], dtype=torch.float64, device=device)
    m = torch.tensor([float(ms_local)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
    return int(round(t.item())), float(m.item())
