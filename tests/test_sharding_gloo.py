"""The multi-rank host logic on CPU: world_size 2, gloo backend, child processes."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from numkong_b200 import sharding


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _reference_merge(values, ids, top):
    """Stand-in for the device merge kernel (no GPU here): [parts, rows, k] lists -> the `top` smallest by (value, id)."""
    parts, rows, k = values.shape
    flat_v = np.transpose(values, (1, 0, 2)).reshape(rows, parts * k)
    flat_i = np.transpose(ids, (1, 0, 2)).reshape(rows, parts * k)
    flat_v = np.where(flat_i < 0, np.inf, flat_v)
    order = np.lexsort((flat_i, flat_v), axis=1)[:, :top]
    return np.take_along_axis(flat_v, order, axis=1), np.take_along_axis(flat_i, order, axis=1)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # 1. the packed blob reaches every rank bit for bit
        blob = torch.arange(4096, dtype=torch.int64).to(torch.uint8) if rank == 0 else torch.zeros(4096, dtype=torch.uint8)
        sharding.broadcast_bytes(blob, src=0)
        assert torch.equal(blob, torch.arange(4096, dtype=torch.int64).to(torch.uint8))
        # 2. nearest-k merge: each rank searches its own slice of a corpus, rank 0 merges with one gather
        rng = np.random.default_rng(5)
        full = torch.from_numpy(rng.standard_normal((6, 40)).astype(np.float32))
        full[2, 7] = full[2, 31]                       # a tie across ranks: the lower id must win
        lo, hi = sharding.row_shard(40, world, rank)
        local = full[:, lo:hi]
        k = 5
        order = torch.argsort(local, dim=1, stable=True)[:, :k]
        vals, ids = torch.gather(local, 1, order), order + lo
        mv, mi = sharding.merge_topk(vals, ids, k, dst=0, merge=_reference_merge)
        if rank == 0:
            want = torch.argsort(full, dim=1, stable=True)[:, :k]
            assert torch.equal(mi, want)
            assert torch.equal(mv, torch.gather(full, 1, want))
        else:
            assert mv is None and mi is None
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_broadcast_and_topk_merge_world_size_2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_row_and_token_shards_cover_everything_once():
    for total in (0, 1, 7, 8192, 10_000_001):
        for world in (1, 2, 4, 8):
            spans = [sharding.row_shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    rng = np.random.default_rng(3)
    counts = rng.integers(64, 301, size=1000)
    offsets = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]))
    for world in (1, 2, 4, 8):
        runs = sharding.token_balanced_shards(offsets, world)
        assert runs[0][0] == 0 and runs[-1][1] == 1000
        assert all(runs[i][1] == runs[i + 1][0] for i in range(world - 1))
        tokens = [int(offsets[e] - offsets[b]) for b, e in runs]
        assert max(tokens) - min(tokens) <= 2 * 300
