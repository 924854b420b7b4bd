"""Multi-GPU host logic: the decode path shards by sequence and nothing else.

Every sequence owns its cache (anchor, deltas, tail, state words) and a decode step never reads
another sequence's rows, so N GPUs run N independent shards of the batch: one process per GPU,
no collective on the data path.  ``torch.distributed`` is used only for the barrier around a
timed region, for the max-over-ranks of its device time, and for summing the units each rank
processed.  The reference is single-GPU, batch-one (flashloop/engine.py:176-177, 376-377), so
these functions have no counterpart there.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def sequence_shard(total_sequences: int, world_size: int, rank: int) -> tuple[int, int]:
    """(first sequence, number of sequences) of ``rank`` when ``total_sequences`` are dealt in
    contiguous blocks; the first ``total % world`` ranks hold one more."""

    total_sequences, world_size, rank = int(total_sequences), int(world_size), int(rank)
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    if total_sequences < 0:
        raise ValueError("total_sequences must be non-negative")
    base, extra = divmod(total_sequences, world_size)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


def sequence_seed(rank: int, layer: int, sequence: int) -> int:
    """Distinct synthetic-data seed per (rank, layer, local sequence)."""

    return (int(rank) * 1000 + int(layer)) * 100 + int(sequence)


def _active(group=None) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def barrier(device: torch.device | None = None, group=None) -> None:
    """Rank barrier (when there is more than one rank) followed by a device synchronise."""

    if _active(group):
        dist.barrier(group=group)
    if device is not None and device.type == "cuda":
        torch.cuda.synchronize(device)


def max_over_ranks(value: float, device: torch.device, group=None) -> float:
    """Largest ``value`` of any rank: the time a multi-GPU step is charged."""

    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if _active(group):
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sum_over_ranks(value: float, device: torch.device, group=None) -> float:
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if _active(group):
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())


def job_throughput(local_units: float, local_ms: float, device: torch.device, group=None) -> tuple[float, float]:
    """(units of all ranks per second, milliseconds charged): units are summed over ranks and
    divided by the slowest rank's time."""

    ms = max_over_ranks(local_ms, device, group)
    units = sum_over_ranks(local_units, device, group)
    return (units / (ms * 1e-3) if ms > 0 else float("nan")), ms
