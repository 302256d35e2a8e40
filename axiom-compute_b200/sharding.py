"""Row sharding of a quantised matrix over the GPUs of one node, and assembly of the output.

Rows are independent dot products against a shared x (that is literally what the reference
function computes), so rank g of G owns the contiguous rows [begin, begin + count): a contiguous
byte range of q and a contiguous slice of y.  x is replicated.  The one exchange step is an
all-gather of the y slices (NCCL over NVLink on GPUs; gloo in the CPU tests of this logic).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_rows(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """(first row, row count) of `rank`: an even split, the first rows % world ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, rem = divmod(rows, world)
    begin = rank * base + min(rank, rem)
    return begin, base + (1 if rank < rem else 0)


def shard_byte_range(rows: int, blocks_per_row: int, block_bytes: int, world: int, rank: int) -> Tuple[int, int]:
    """(byte offset, byte length) of the rank's rows inside the full q buffer."""
    begin, count = shard_rows(rows, world, rank)
    row_bytes = blocks_per_row * block_bytes
    return begin * row_bytes, count * row_bytes


def all_gather_rows(y_local: torch.Tensor, rows: int, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Assemble the full y (length `rows`) from every rank's slice, in rank order.

    With an even split this is a single all_gather_into_tensor on the current stream; with a
    ragged split the slices are padded to the largest one and trimmed afterwards."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    begin, count = shard_rows(rows, world, rank)
    if y_local.numel() != count:
        raise ValueError(f"rank {rank} holds {y_local.numel()} rows, its shard has {count}")
    if out is None:
        out = torch.empty(rows, dtype=y_local.dtype, device=y_local.device)
    if rows % world == 0:
        dist.all_gather_into_tensor(out, y_local.contiguous(), group=group)
        return out
    width = rows // world + 1
    padded = torch.zeros(width, dtype=y_local.dtype, device=y_local.device)
    padded[:count] = y_local
    gathered = torch.empty(world * width, dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(gathered, padded, group=group)
    for r in range(world):
        b, c = shard_rows(rows, world, r)
        out[b:b + c] = gathered[r * width:r * width + c]
    return out
