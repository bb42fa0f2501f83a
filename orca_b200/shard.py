"""Row ownership and exchange for the multi-GPU path (one process per GPU, torch.distributed).

The reference is single-device; this split is a design of this package.  Layer-1 row i of a batch's
row list [src | dst | neg | uncached] belongs to rank ``i % world`` at local slot ``i // world``; edge
e of the batch (its src, dst and neg rows in the top layer and its two scores) belongs to rank
``e % world`` at local slot ``e // world``.  Interleaving keeps the ranks balanced although the
number of layer-1 rows is only known on the device.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def rows_per_rank(capacity: int, world: int) -> int:
    return -(-capacity // world)


def owner_slot(i, world: int, rpr: int):
    """Index of global row i inside the all-gathered buffer [world, rpr, ...] flattened."""
    return (i % world) * rpr + i // world


def local_count(n: int, rank: int, world: int) -> int:
    """How many of the ids 0..n-1 belong to `rank`."""
    return (n - rank + world - 1) // world if n > rank else 0


def all_gather_rows(local: torch.Tensor, group=None) -> torch.Tensor:
    """[rpr, ...] on every rank -> [world, rpr, ...] on every rank (NCCL on GPU tensors, gloo on CPU)."""
    world = dist.get_world_size(group)
    out = local.new_empty((world,) + tuple(local.shape))
    dist.all_gather_into_tensor(out.view(-1), local.contiguous().view(-1), group=group)
    return out


_ASSEMBLE_INDEX = {}


def assemble_index(b: int, parts: int, world: int, per_rank: int, device) -> torch.Tensor:
    """For every row of the [parts * b] batch-order array, its position in the flattened
    [world, per_rank] all-gathered buffer (rank r holds `parts` blocks of local_count(b, r, world))."""
    key = (b, parts, world, per_rank, str(device))
    idx = _ASSEMBLE_INDEX.get(key)
    if idx is None:
        e = torch.arange(b)
        r, j = e % world, e // world
        n_r = torch.tensor([local_count(b, q, world) for q in range(world)])[r]
        idx = torch.cat([r * per_rank + p * n_r + j for p in range(parts)]).to(device)
        _ASSEMBLE_INDEX[key] = idx
    return idx


def assemble_edges(gathered: torch.Tensor, b: int, parts: int) -> torch.Tensor:
    """gathered[r] holds rank r's edge-major blocks: `parts` blocks of local_count(b, r, world) rows
    each (padded at the end).  Returns the [parts * b, ...] array in batch order, block by block."""
    world, per_rank = gathered.shape[0], gathered.shape[1]
    idx = assemble_index(b, parts, world, per_rank, gathered.device)
    return gathered.reshape((world * per_rank,) + tuple(gathered.shape[2:])).index_select(0, idx)
