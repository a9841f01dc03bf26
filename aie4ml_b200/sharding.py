"""Batch sharding across GPUs: one process per GPU, identical plan, disjoint row ranges.

Every operator of the lowered graph is independent along the flattened leading (batch / sequence)
axis, weights are replicated, so the forward pass needs no collective.  The only exchange is an
optional gather of the outputs at the end (``gather_outputs``), which uses ``torch.distributed``
(NCCL over NVLink on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

from typing import List, Tuple

import numpy as np


def shard_rows(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open row range of ``rank``; sizes differ by at most one, earlier ranks get the extras."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f'bad rank/world {rank}/{world}')
    base, extra = divmod(int(total), int(world))
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_inputs(inputs: dict, rank: int, world: int) -> dict:
    """Slice every graph input along its leading axis for ``rank``."""
    out = {}
    for name, arr in inputs.items():
        s, e = shard_rows(arr.shape[0], rank, world)
        out[name] = arr[s:e]
    return out


def gather_outputs(local, total_rows: int, group=None):
    """All-gather row shards into the full tensor on every rank.

    ``local`` is a torch tensor ``[rows_r, ...]`` (any strides).  Equal shards gather straight into the result with one
    ``all_gather_into_tensor``; unequal ones are padded to the largest shard first and trimmed afterwards."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = [shard_rows(total_rows, r, world) for r in range(world)]
    biggest = max(e - s for s, e in sizes)
    if all(e - s == biggest for s, e in sizes):
        out = torch.empty((total_rows, *local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest, *local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    out = torch.empty((world * biggest, *local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    pieces: List = [out[r * biggest: r * biggest + (e - s)] for r, (s, e) in enumerate(sizes)]
    return torch.cat(pieces, dim=0)
