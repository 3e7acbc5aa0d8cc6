"""Token-row sharding across ranks.

Every op of the path is independent per token row, so a T-token batch is split
into contiguous row ranges, one per rank, and no rank ever needs another rank's
rows: there is no collective on the data path.  The only cross-rank traffic is
the timing reduction below (one scalar).
"""
from __future__ import annotations

import torch.distributed as dist


def token_range(rank: int, world: int, n_tokens: int) -> tuple[int, int]:
    """Contiguous [start, stop) of `n_tokens` rows owned by `rank`; the first
    n_tokens % world ranks own one extra row.  Empty for ranks beyond n_tokens."""
    if world < 1 or not 0 <= rank < world or n_tokens < 0:
        raise ValueError(f"bad shard request rank={rank} world={world} n_tokens={n_tokens}")
    base, extra = divmod(n_tokens, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def tokens_per_rank(world: int, n_tokens: int, scaling: str) -> list[int]:
    """weak: every rank processes n_tokens rows (job = world * n_tokens);
    strong: the n_tokens rows are split across ranks."""
    if scaling == "weak":
        return [n_tokens] * world
    if scaling == "strong":
        return [b - a for a, b in (token_range(r, world, n_tokens) for r in range(world))]
    raise ValueError(f"unknown scaling mode {scaling!r}")


def _reduce(value: float, op) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=op)
    return float(t.item())


def max_over_ranks(value: float) -> float:
    return _reduce(value, dist.ReduceOp.MAX)


def sum_over_ranks(value: float) -> float:
    return _reduce(value, dist.ReduceOp.SUM)


def barrier() -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def job_throughput(units_per_rank: float, ms: float) -> float:
    """Whole-job units/s: units of every rank over the slowest rank's time."""
    total = sum_over_ranks(units_per_rank)
    worst = max_over_ranks(ms)
    return total / (worst * 1e-3)
