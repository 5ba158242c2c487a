"""Synthetic twins of the two search workloads of the packed-contraction path, with device-side timing.

    python -m numkong_b200.workloads nearest --queries 8192 --corpus 65536 --depth 768 --top 10 --dtype f16
    python -m numkong_b200.workloads maxsim  --queries 256 --docs 20000 --depth 128 --top 100
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29500 \
        -m numkong_b200.workloads nearest --queries 65536 --corpus 10000000 --sharded

With --sharded (one process per GPU under torchrun) the corpus rows / the documents are split across the ranks, every rank
searches its own shard and the k best per query are merged on rank 0 with one gather; the time is the slowest rank's, from
"shards packed and resident" to "merged lists on rank 0". Shards are generated per rank, so their content depends on the
number of ranks; sizes and distributions do not.

`nearest`: L2-normalised N(0,1) queries against an L2-normalised corpus, angular top-k per query (the batched
distance kernels + selection). `maxsim`: ColBERT-style late interaction, queries of 32 tokens against documents of
64..300 tokens (uniform), L2-normalised N(0,1) token vectors in bf16, all-pairs MaxSim scores + top-k per query.
Work is counted as 2 * rows * columns * depth (for MaxSim: query tokens x document tokens, unpadded), the
definition the reference's benchmarks use (bench/bench.hpp:257, bench/bench_maxsim.cpp:60). One JSON line per run.
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def _timed(torch, fn, steps: int, warmup: int = 2) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps / 1e3


def _device_rows(torch, rows: int, depth: int, dtype: str, seed: int):
    """L2-normalised N(0,1) rows made on the device (large corpora: the host generator would dominate the run)."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    out = torch.empty((rows, depth), dtype=torch.float16 if dtype == "f16" else torch.bfloat16, device="cuda")
    for r in range(0, rows, 1 << 18):
        n = min(1 << 18, rows - r)
        x = torch.randn((n, depth), generator=gen, device="cuda", dtype=torch.float32)
        out[r:r + n] = (x / x.norm(dim=1, keepdim=True)).to(out.dtype)
    return out


def run_nearest(queries: int, corpus: int, depth: int, top: int, dtype: str = "f16", steps: int = 5, seed: int = 3,
                warmup: int = 2):
    import torch
    import numkong_b200 as nk
    from numkong_b200 import synthetic as syn
    if corpus * depth > (1 << 27):
        tq, tc = _device_rows(torch, queries, depth, dtype, seed), _device_rows(torch, corpus, depth, dtype, seed + 1)
        data = "device generator"
    else:
        q = syn.normal_matrix(queries, depth, dtype, seed, normalize=True)
        c = np.concatenate([syn.normal_matrix(min(65536, corpus - r), depth, dtype, seed + 1 + r, normalize=True)
                            for r in range(0, corpus, 65536)])
        tq, tc = torch.from_numpy(q.view(np.int16)).cuda(), torch.from_numpy(c.view(np.int16)).cuda()
        data = "host generator"
    packed = nk.dots_pack(tc, dtype)
    del tc
    launches0 = nk.launch_count()
    seconds = _timed(torch, lambda: nk.angulars_packed_topk(tq, packed, top, dtype=dtype), steps, warmup)
    launches = (nk.launch_count() - launches0) // (steps + warmup)
    assert nk.synchronize() == 0
    ops = 2.0 * queries * corpus * depth
    return {"workload": f"angular top-{top}: {queries} {dtype} queries x {corpus} corpus rows, depth {depth}", "ms": seconds * 1e3,
            "gso_per_s": ops / seconds / 1e9, "kernels_per_call": int(launches), "steps": steps, "warmup": warmup, "data": data,
            "filter_fallbacks": int(nk.lib.nkb_topk_filter_fallbacks())}


def run_maxsim(queries: int, docs: int, depth: int = 128, top: int = 100, q_tokens: int = 32, steps: int = 3, seed: int = 5,
               warmup: int = 2):
    import torch
    import numkong_b200 as nk
    from numkong_b200 import synthetic as syn
    rng = np.random.default_rng(seed)
    counts = rng.integers(64, 301, size=docs)
    d_off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    q_off = (np.arange(queries + 1) * q_tokens).astype(np.int64)
    total = int(d_off[-1])
    if total * depth > (1 << 27):
        q, d = _device_rows(torch, queries * q_tokens, depth, "bf16", seed + 1), _device_rows(torch, total, depth, "bf16", seed + 2)
    else:
        qh = syn.normal_matrix(queries * q_tokens, depth, "bf16", seed + 1, normalize=True)
        dh = np.concatenate([syn.normal_matrix(min(1 << 20, total - r), depth, "bf16", seed + 2 + r, normalize=True)
                             for r in range(0, total, 1 << 20)])
        q, d = torch.from_numpy(qh.view(np.int16)).cuda(), torch.from_numpy(dh.view(np.int16)).cuda()
    tq = nk.maxsim_pack(q, "bf16")
    td = nk.maxsim_pack(d, "bf16")
    del q, d
    tqo, tdo = torch.from_numpy(q_off).cuda(), torch.from_numpy(d_off).cuda()
    state = {}

    def step():
        state["scores"] = nk.maxsims_packed(tq, tqo, td, tdo)
        state["best"] = nk.topk_smallest(state["scores"], min(top, docs))

    seconds = _timed(torch, step, steps, warmup)
    assert nk.synchronize() == 0
    ops = 2.0 * queries * q_tokens * total * depth
    return {"workload": f"MaxSim top-{top}: {queries} queries x {q_tokens} tokens vs {docs} documents ({total} tokens), depth {depth}, bf16",
            "ms": seconds * 1e3, "gso_per_s": ops / seconds / 1e9, "steps": steps, "warmup": warmup}


def run_dense(rows: int, width: int, depth: int, dtype: str = "f32", op: str = "dots", steps: int = 5, seed: int = 11, warmup: int = 2):
    """One packed product (or distance matrix) of any supported element type and shape, operands resident on the device:
    N(0,1) values generated as f32 and converted with the library's own bulk conversion."""
    import torch
    import numkong_b200 as nk
    torch.manual_seed(seed)
    a32, b32 = torch.randn(rows, depth, device="cuda"), torch.randn(width, depth, device="cuda")
    a = a32 if dtype == "f32" else nk.cast(a32, dtype)
    b = b32 if dtype == "f32" else nk.cast(b32, dtype)
    if dtype in ("i8", "u8"):
        a, b = nk.cast((a32 * 40).contiguous(), dtype), nk.cast((b32 * 40).contiguous(), dtype)
    packed = nk.dots_pack(b, dtype)
    fn = getattr(nk, op + "_packed")
    out = fn(a, packed, dtype=dtype)
    seconds = _timed(torch, lambda: fn(a, packed, out=out, dtype=dtype), steps, warmup)
    assert nk.synchronize() == 0
    return {"workload": f"{op}_packed {dtype} {rows} x {width} x {depth}", "ms": seconds * 1e3,
            "gso_per_s": 2.0 * rows * width * depth / seconds / 1e9, "steps": steps, "warmup": warmup}


def run_quantise(values: int, dtype: str = "e4m3", steps: int = 5, seed: int = 7, warmup: int = 2):
    """The step in front of `pack` when the source is f32: moments of the source (the scale comes from them) and the bulk
    conversion to the storage type. Device-resident; reports both kernels in GB/s of algorithmic traffic."""
    import torch
    import numkong_b200 as nk
    torch.manual_seed(seed)
    x = torch.randn(values, device="cuda")
    out = torch.empty(values * nk.CAST_BITS[dtype] // 8, dtype=torch.uint8, device="cuda")
    stats = nk.moments(x)
    s_moments = _timed(torch, lambda: nk.moments(x), steps, warmup)
    s_cast = _timed(torch, lambda: nk.cast(x, dtype, out=out), steps, warmup)
    return {"workload": "quantise", "values": values, "dtype": dtype, "sum": stats[0], "sumsq": stats[1],
            "moments_ms": s_moments * 1e3, "moments_gbs": values * 4 / s_moments / 1e9,
            "cast_ms": s_cast * 1e3, "cast_gbs": (values * 4 + out.numel()) / s_cast / 1e9}


class _SingleProcess:
    """Stands in for torch.distributed when the script runs as one plain process (one GPU, no launcher)."""
    ReduceOp = type("ReduceOp", (), {"MAX": None})

    @staticmethod
    def barrier():
        pass

    @staticmethod
    def all_reduce(tensor, op=None):
        return tensor


def _distributed(torch):
    """(communication module, rank, world size): torch.distributed under a launcher, a stand-in for a single process."""
    import os
    if "RANK" not in os.environ or int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return _SingleProcess, 0, 1
    import torch.distributed as dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return dist, rank, world


def _timed_all_ranks(torch, dist, fn, steps: int, warmup: int) -> float:
    """Seconds per step of the slowest rank: barrier + synchronize on both sides, CUDA events in between."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    dist.barrier()
    seconds = torch.tensor([start.elapsed_time(stop) / steps / 1e3], device="cuda")
    dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
    return float(seconds.item())


def run_nearest_sharded(queries: int, corpus: int, depth: int, top: int, dtype: str = "f16", steps: int = 2, seed: int = 3,
                        warmup: int = 1):
    import torch
    import numkong_b200 as nk
    from numkong_b200 import search, sharding
    dist, rank, world = _distributed(torch)
    lo, hi = sharding.row_shard(corpus, world, rank)
    tq = _device_rows(torch, queries, depth, dtype, seed)          # the queries live on rank 0 ...
    if rank != 0:
        tq.zero_()
    packed = nk.dots_pack(_device_rows(torch, hi - lo, depth, dtype, seed + 1 + rank), dtype)

    def step():
        if world > 1:
            dist.broadcast(tq, src=0)                              # ... and reach the other ranks inside every timed step
        d, i = search.nearest_in_shard(tq, packed, top, id_base=lo, dtype=dtype)
        sharding.merge_topk(d, i, top)

    seconds = _timed_all_ranks(torch, dist, step, steps, warmup)
    assert nk.synchronize() == 0
    ops = 2.0 * queries * corpus * depth
    out = {"workload": f"angular top-{top}: {queries} {dtype} queries x {corpus} corpus rows over {world} GPUs, depth {depth}",
           "ms": seconds * 1e3, "gso_per_s": ops / seconds / 1e9, "n_gpus": world, "steps": steps, "warmup": warmup,
           "filter_fallbacks": int(nk.lib.nkb_topk_filter_fallbacks())}
    dist.barrier()
    return out if rank == 0 else None


def run_maxsim_sharded(queries: int, docs: int, depth: int = 128, top: int = 100, q_tokens: int = 32, steps: int = 2, seed: int = 5,
                       warmup: int = 1):
    import torch
    import numkong_b200 as nk
    from numkong_b200 import sharding
    dist, rank, world = _distributed(torch)
    counts = np.random.default_rng(seed).integers(64, 301, size=docs)
    d_off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    q_off = torch.from_numpy((np.arange(queries + 1) * q_tokens).astype(np.int64)).cuda()
    d0, d1 = sharding.token_balanced_shards(torch.from_numpy(d_off), world)[rank]
    local_off = torch.from_numpy(d_off[d0:d1 + 1] - d_off[d0]).cuda()
    tq = nk.maxsim_pack(_device_rows(torch, queries * q_tokens, depth, "bf16", seed + 1), "bf16")
    if rank != 0:
        tq.buffer.zero_()                                          # the packed queries live on rank 0 ...
    td = nk.maxsim_pack(_device_rows(torch, int(d_off[d1] - d_off[d0]), depth, "bf16", seed + 2 + rank), "bf16")

    def step():
        if world > 1:
            dist.broadcast(tq.buffer, src=0)                       # ... and are broadcast inside every timed step (position independent)
        scores = nk.maxsims_packed(tq, q_off, td, local_off)
        vals, ids = nk.topk_smallest(scores, min(top, d1 - d0), id_base=d0)
        sharding.merge_topk(vals, ids, min(top, d1 - d0))

    seconds = _timed_all_ranks(torch, dist, step, steps, warmup)
    assert nk.synchronize() == 0
    total = int(d_off[-1])
    ops = 2.0 * queries * q_tokens * total * depth
    out = {"workload": f"MaxSim top-{top}: {queries} queries x {q_tokens} tokens vs {docs} documents ({total} tokens) over {world} GPUs, depth {depth}, bf16",
           "ms": seconds * 1e3, "gso_per_s": ops / seconds / 1e9, "n_gpus": world, "steps": steps, "warmup": warmup}
    dist.barrier()
    return out if rank == 0 else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=["nearest", "maxsim", "quantise", "dense"])
    ap.add_argument("--op", default="dots", choices=["dots", "angulars", "euclideans"])
    ap.add_argument("--values", type=int, default=1 << 26)
    ap.add_argument("--queries", type=int, default=None)
    ap.add_argument("--corpus", type=int, default=65536)
    ap.add_argument("--docs", type=int, default=20000)
    ap.add_argument("--depth", type=int, default=None)
    ap.add_argument("--top", type=int, default=None)
    ap.add_argument("--dtype", default="f16")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--sharded", action="store_true", help="split the corpus / documents over the ranks of a torchrun launch")
    a = ap.parse_args()
    if a.workload == "dense":
        out = run_dense(a.queries or 4096, a.corpus, a.depth or 4096, a.dtype, a.op, a.steps, warmup=a.warmup)
    elif a.workload == "quantise":
        out = run_quantise(a.values, a.dtype if a.dtype != "f16" else "e4m3", a.steps, warmup=a.warmup)
    elif a.workload == "nearest":
        fn = run_nearest_sharded if a.sharded else run_nearest
        out = fn(a.queries or 8192, a.corpus, a.depth or 768, a.top or 10, a.dtype, a.steps, warmup=a.warmup)
    else:
        fn = run_maxsim_sharded if a.sharded else run_maxsim
        out = fn(a.queries or 256, a.docs, a.depth or 128, a.top or 100, steps=a.steps, warmup=a.warmup)
    if out is not None:
        print(json.dumps(out))
    if a.sharded:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
