"""Multi-GPU partitioning of the MoDA operators: by (batch x KV-head), no collective.

Every (batch, KV-head) pair is an independent problem in forward and backward (the G
query heads of a KV head are rows of the same folded query tensor, and dk/dv/depth
grads of a head depend only on that head's queries), so ranks take contiguous slices
of the flattened (b, h) index space and never exchange data on the hot path.  The
reference has no multi-GPU operator path (its only distributed code is DDP around the
DeiT model: vision_tasks/deit/main.py:345); this module is what a data-parallel
caller of the operator needs.  ``gather_units`` collects per-unit results for
validation over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch


@dataclass(frozen=True)
class UnitRange:
    """Half-open range [start, stop) of flattened units u = b * H + h."""
    start: int
    stop: int

    def __len__(self) -> int:
        return self.stop - self.start


def partition_units(n_units: int, world_size: int, rank: int) -> UnitRange:
    """Contiguous, balanced split: the first ``n_units % world_size`` ranks get one extra."""
    assert world_size >= 1 and 0 <= rank < world_size and n_units >= 0
    base, extra = divmod(n_units, world_size)
    start = rank * base + min(rank, extra)
    return UnitRange(start, start + base + (1 if rank < extra else 0))


def units_to_slices(rng: UnitRange, H: int) -> List[tuple]:
    """[(b, h_start, h_stop), ...] covering the unit range with one entry per batch row."""
    out = []
    u = rng.start
    while u < rng.stop:
        b, h0 = divmod(u, H)
        h1 = min(H, h0 + (rng.stop - u))
        out.append((b, h0, h1))
        u += h1 - h0
    return out


def unit_seed(base_seed: int, tensor_id: int, unit: int) -> int:
    """Seed of one (tensor, batch, head) stream, so a shard's contents do not depend on
    how many ranks share the job."""
    return (base_seed * 1000003 + tensor_id * 10007 + unit * 101 + 12345) % (2 ** 63 - 1)


def gather_units(local: torch.Tensor, n_units: int, world_size: int, rank: int) -> torch.Tensor:
    """All-gather per-unit rows.  ``local`` is [len(partition), ...]; returns
    [n_units, ...] in unit order on every rank.  Ranks may hold different counts."""
    import torch.distributed as dist
    if world_size == 1:
        return local
    counts = [len(partition_units(n_units, world_size, r)) for r in range(world_size)]
    width = max(counts)
    pad = torch.zeros((width,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    bufs = [torch.empty_like(pad) for _ in range(world_size)]
    dist.all_gather(bufs, pad)
    return torch.cat([b[:c] for b, c in zip(bufs, counts)], dim=0)


def shard_heads(x: torch.Tensor, slices: Sequence[tuple]) -> List[torch.Tensor]:
    """Views [1, T, h1-h0, D] of a [B, T, H, D] tensor for each (b, h0, h1); no copies —
    the library consumes the strided views in place."""
    return [x[b : b + 1, :, h0:h1] for (b, h0, h1) in slices]
