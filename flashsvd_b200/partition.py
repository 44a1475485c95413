"""Batch partition of independent sequences over ranks (one process per GPU).

Decode of independent sequences needs no data-path collective: every rank holds a full replica
of the factors and its own KV cache and decodes the sequences ``sequences_of_rank`` gives it.
Ranks meet only to reduce the step time (max over ranks) and to gather token ids on the host.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def sequences_of_rank(n_seq: int, rank: int, world: int) -> list:
    """Indices of the sequences rank ``rank`` decodes: contiguous blocks whose sizes differ by
    at most one (the first ``n_seq % world`` ranks take one more)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(int(n_seq), int(world))
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def aggregate_tokens_per_s(tokens_per_rank, ms_per_rank) -> float:
    """Whole-job throughput: all tokens of all ranks over the slowest rank's time."""
    return float(sum(tokens_per_rank)) / (max(ms_per_rank) * 1e-3)


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def max_over_ranks(t: torch.Tensor) -> torch.Tensor:
    if _world() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t


def sum_over_ranks(t: torch.Tensor) -> torch.Tensor:
    if _world() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t


def gather_tokens(tokens_by_seq: dict, n_seq: int):
    """Token lists of all sequences in sequence order on rank 0 (None elsewhere)."""
    if _world() == 1:
        return [tokens_by_seq[i] for i in range(n_seq)]
    parts = [None] * _world() if dist.get_rank() == 0 else None
    dist.gather_object(tokens_by_seq, parts, dst=0)
    if dist.get_rank() != 0:
        return None
    merged = {}
    for p in parts:
        merged.update(p)
    return [merged[i] for i in range(n_seq)]
