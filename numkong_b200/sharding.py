"""Multi-GPU plumbing for the packed-contraction path: one process per GPU over torch.distributed.

The path shards by rows, exactly like the reference's callers split rows of A across threads
(README.md:199-212 of the reference): every rank multiplies its own rows against the same packed B, or
scores the queries against its own slice of the corpus / documents. The only exchanges are a broadcast
of the packed operand that every rank needs and, for nearest-k searches, one gather of each rank's k best
followed by a merge. Collectives run on NCCL for CUDA tensors and on gloo for CPU tensors (tests).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def row_shard(total_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) row range of `rank`; the first (total % world) ranks get one extra row."""
    base, extra = divmod(total_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def token_balanced_shards(offsets: torch.Tensor, world_size: int):
    """Splits ragged units (documents with token offsets, length n+1) into `world_size` contiguous runs of
    whole units with nearly equal token counts. Returns a list of (first_unit, last_unit_exclusive)."""
    offsets = torch.as_tensor(offsets, dtype=torch.int64).cpu()
    n, total = offsets.numel() - 1, int(offsets[-1])
    cuts = [0]
    for r in range(1, world_size):
        target = total * r // world_size
        cuts.append(int(torch.searchsorted(offsets, torch.tensor(target), right=False).clamp(max=n)))
    cuts.append(n)
    for i in range(1, len(cuts)):
        cuts[i] = max(cuts[i], cuts[i - 1])
    return [(cuts[i], cuts[i + 1]) for i in range(world_size)]


def broadcast_bytes(buffer: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
    """Broadcasts a uint8 tensor (a packed blob: position independent, so a plain byte copy is valid)
    into every rank's own memory. All ranks pass a tensor of the same size."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(buffer, src=src, group=group)
    return buffer


def merge_topk(values: torch.Tensor, ids: torch.Tensor, top: int, group=None, dst: int = 0):
    """Merges per-rank nearest-k lists (rows x k, ascending) with ONE gather. Returns (values, ids) on `dst`
    (None elsewhere). Ties go to the lower id; slots with id < 0 are empty."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if world == 1:
        return values, ids
    packed = torch.cat([values.to(torch.float64), ids.to(torch.float64)], dim=1).contiguous()  # ids < 2^53 stay exact
    if packed.is_cuda and dist.get_backend(group) == "gloo":
        packed = packed.cpu()  # gloo moves host memory only; the merged lists then stay on the host
    gathered = [torch.empty_like(packed) for _ in range(world)] if rank == dst else None
    dist.gather(packed, gathered, dst=dst, group=group)
    if rank != dst:
        return None, None
    k = values.shape[1]
    all_vals = torch.cat([g[:, :k] for g in gathered], dim=1)
    all_ids = torch.cat([g[:, k:] for g in gathered], dim=1).to(torch.int64)
    all_vals = torch.where(all_ids < 0, torch.full_like(all_vals, float("inf")), all_vals)
    # order by (value, id): sort by id first, then a stable sort by value
    by_id = torch.argsort(all_ids, dim=1, stable=True)
    all_vals, all_ids = torch.gather(all_vals, 1, by_id), torch.gather(all_ids, 1, by_id)
    by_val = torch.argsort(all_vals, dim=1, stable=True)[:, :top]
    return torch.gather(all_vals, 1, by_val).to(values.dtype), torch.gather(all_ids, 1, by_val)
