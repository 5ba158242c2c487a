"""Multi-GPU plumbing for the packed-contraction path: one process per GPU over torch.distributed.

The path shards by rows, exactly like the reference's callers split rows of A across threads
(README.md:199-212 of the reference): every rank multiplies its own rows against the same packed B, or
scores the queries against its own slice of the corpus / documents. The only exchanges are a broadcast
of the packed operand that every rank needs and, for nearest-k searches, one gather of each rank's k best
followed by a merge. Collectives run on NCCL for CUDA tensors and on gloo for CPU tensors (tests); the packed operand
can instead travel through the NVSwitch's multicast with the library's own copy and barrier kernels (SwitchBroadcast).
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


class SwitchBroadcast:
    """One-to-all delivery of a byte buffer (a packed matrix) through the NVSwitch's multicast: the sender issues every
    16 bytes once (`multimem.st`, nkb_multicast_store) and the switch writes them into every GPU's copy, so the sender's
    link carries the data once whatever the group size; a bounded flag barrier between the GPUs (nkb_peer_barrier) orders
    the receivers' streams behind the copy. Receivers run no kernel but the barrier.

        channel = SwitchBroadcast(nbytes)        # set-up, collective: symmetric buffer + multicast mapping
        blob = channel.send(blob_on_src, src=0)  # every rank calls it; returns this rank's copy (a view of the buffer)

    `available` is False where the GPUs have no multicast mapping (no NVSwitch fabric, one GPU): `send` then falls back to
    the group's ordinary broadcast (NCCL) into the same buffer. Ranks must leave together (`close`) - a process that exits
    while its memory is still bound to the multicast object disturbs the others.
    """

    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 15) // 16 * 16
        self.buffer = symm.empty(self.nbytes, dtype=torch.uint8, device=device)
        self._handle = symm.rendezvous(self.buffer, self.group)
        self._flags = symm.empty(64, dtype=torch.int32, device=device)
        self._flags.zero_()
        self._flag_handle = symm.rendezvous(self._flags, self.group)
        self._epoch = 0
        base = int(self._handle.buffer_ptrs[self.rank])
        inside = self.buffer.data_ptr() - base
        multicast = int(self._handle.multicast_ptr)
        self.available = multicast != 0 and self.world <= 16 and 0 <= inside and inside + self.nbytes <= int(self._handle.buffer_size)
        self._multicast = multicast + inside if self.available else 0
        flag_base = int(self._flag_handle.buffer_ptrs[self.rank])
        flag_inside = self._flags.data_ptr() - flag_base
        import ctypes
        self._peer_flags = (ctypes.c_void_p * self.world)(*[int(ptr) + flag_inside for ptr in self._flag_handle.buffer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # every rank's flags are zero before anyone's first barrier

    def barrier(self) -> None:
        """Orders everything enqueued behind it on any rank's current stream after everything enqueued before it on all."""
        from . import _lib
        self._epoch += 1
        _lib.lib.nkb_set_stream(torch.cuda.current_stream().cuda_stream)
        if _lib.lib.nkb_peer_barrier(self._peer_flags, self.world, self.rank, self._epoch) != 0:
            raise RuntimeError("peer barrier: " + _lib.last_error())

    def send(self, source: torch.Tensor = None, src: int = 0, blocks: int = 0) -> torch.Tensor:
        """`source` (uint8, on `src` only; other ranks may pass None) lands in every rank's buffer; returns that buffer's
        first `source.numel()` bytes - on every rank the size of the buffer when `source` is None."""
        from . import _lib
        count = self.nbytes if source is None else int(source.numel())
        if not self.available:
            view = self.buffer[:count]
            if self.rank == src:
                view.copy_(source.reshape(-1).view(torch.uint8))
            dist.broadcast(view, src=src, group=self.group)
            return view
        self.barrier()  # nobody still reads what the buffer held before
        if self.rank == src:
            flat = source.reshape(-1).view(torch.uint8)
            padded = (count + 15) // 16 * 16
            if padded != count or flat.data_ptr() % 16:
                staged = torch.zeros(padded, dtype=torch.uint8, device=flat.device)
                staged[:count] = flat
                flat = staged
            _lib.lib.nkb_set_stream(torch.cuda.current_stream().cuda_stream)
            if _lib.lib.nkb_multicast_store(self._multicast, flat.data_ptr(), padded, blocks) != 0:
                raise RuntimeError("multicast store: " + _lib.last_error())
        self.barrier()
        return self.buffer[:count]

    def close(self) -> None:
        """Collective: all ranks drop their mapping together, with nothing in flight."""
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self._handle = self._flag_handle = None
        self.buffer = self._flags = None


def merge_topk(values: torch.Tensor, ids: torch.Tensor, top: int, group=None, dst: int = 0, merge=None):
    """Merges per-rank nearest-k lists (rows x k, f32 distances and i64 ids, ascending) with ONE gather and the library's
    own merge kernel (nkb_merge_topk). Returns (values, ids) on `dst` (None elsewhere). Ties go to the lower id; slots
    with id < 0 are empty.

    Every rank's lists travel as one byte record per row (k f32 values followed by k i64 ids, 12 bytes per entry), over
    NCCL for CUDA tensors. `merge(values[parts, rows, k], ids[parts, rows, k], top)` replaces the device kernel; the
    CPU-only tests of this host logic pass a reference merge, nothing else should."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if world == 1:
        return values, ids
    rows, k = values.shape
    record = torch.cat([values.to(torch.float32).contiguous().view(torch.uint8).reshape(rows, k * 4),
                        ids.to(torch.int64).contiguous().view(torch.uint8).reshape(rows, k * 8)], dim=1).contiguous()
    if record.is_cuda and dist.get_backend(group) == "gloo":
        record = record.cpu()  # gloo moves host memory only; the library then stages the merge through the device
    gathered = torch.empty((world, rows, k * 12), dtype=torch.uint8, device=record.device) if rank == dst else None
    dist.gather(record, list(gathered.unbind(0)) if rank == dst else None, dst=dst, group=group)
    if rank != dst:
        return None, None
    all_vals = gathered[:, :, :k * 4].contiguous().view(torch.float32).reshape(world, rows, k)
    all_ids = gathered[:, :, k * 4:].contiguous().view(torch.int64).reshape(world, rows, k)
    if merge is None:
        from . import merge_topk as merge
    out_vals, out_ids = merge(all_vals if all_vals.is_cuda else all_vals.numpy(), all_ids if all_ids.is_cuda else all_ids.numpy(), top)
    if not isinstance(out_vals, torch.Tensor):
        out_vals, out_ids = torch.from_numpy(out_vals), torch.from_numpy(out_ids)
    return out_vals.to(values.dtype), out_ids
