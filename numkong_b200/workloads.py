"""Synthetic twins of the two search workloads of the packed-contraction path, with device-side timing.

    python -m numkong_b200.workloads nearest --queries 8192 --corpus 65536 --depth 768 --top 10 --dtype f16
    python -m numkong_b200.workloads maxsim  --queries 256 --docs 20000 --depth 128 --top 100

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


def run_nearest(queries: int, corpus: int, depth: int, top: int, dtype: str = "f16", steps: int = 5, seed: int = 3):
    import torch
    import numkong_b200 as nk
    from numkong_b200 import synthetic as syn
    q = syn.normal_matrix(queries, depth, dtype, seed, normalize=True)
    c = np.concatenate([syn.normal_matrix(min(65536, corpus - r), depth, dtype, seed + 1 + r, normalize=True)
                        for r in range(0, corpus, 65536)])
    tq, tc = torch.from_numpy(q.view(np.int16)).cuda(), torch.from_numpy(c.view(np.int16)).cuda()
    packed = nk.dots_pack(tc, dtype)
    launches0 = nk.launch_count()
    seconds = _timed(torch, lambda: nk.angulars_packed_topk(tq, packed, top, dtype=dtype), steps)
    launches = (nk.launch_count() - launches0) // (steps + 2)
    assert nk.synchronize() == 0
    ops = 2.0 * queries * corpus * depth
    return {"workload": f"angular top-{top}: {queries} {dtype} queries x {corpus} corpus rows, depth {depth}", "ms": seconds * 1e3,
            "gso_per_s": ops / seconds / 1e9, "kernels_per_call": int(launches)}


def run_maxsim(queries: int, docs: int, depth: int = 128, top: int = 100, q_tokens: int = 32, steps: int = 3, seed: int = 5):
    import torch
    import numkong_b200 as nk
    from numkong_b200 import synthetic as syn
    rng = np.random.default_rng(seed)
    counts = rng.integers(64, 301, size=docs)
    d_off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    q_off = (np.arange(queries + 1) * q_tokens).astype(np.int64)
    total = int(d_off[-1])
    q = syn.normal_matrix(queries * q_tokens, depth, "bf16", seed + 1, normalize=True)
    d = np.concatenate([syn.normal_matrix(min(1 << 20, total - r), depth, "bf16", seed + 2 + r, normalize=True)
                        for r in range(0, total, 1 << 20)])
    tq = nk.maxsim_pack(torch.from_numpy(q.view(np.int16)).cuda(), "bf16")
    td = nk.maxsim_pack(torch.from_numpy(d.view(np.int16)).cuda(), "bf16")
    tqo, tdo = torch.from_numpy(q_off).cuda(), torch.from_numpy(d_off).cuda()
    state = {}

    def step():
        state["scores"] = nk.maxsims_packed(tq, tqo, td, tdo)
        state["best"] = nk.topk_smallest(state["scores"], min(top, docs))

    seconds = _timed(torch, step, steps)
    score_seconds = _timed(torch, lambda: nk.maxsims_packed(tq, tqo, td, tdo), steps, warmup=1)
    assert nk.synchronize() == 0
    ops = 2.0 * queries * q_tokens * total * depth
    return {"workload": f"MaxSim top-{top}: {queries} queries x {q_tokens} tokens vs {docs} documents ({total} tokens), depth {depth}, bf16",
            "ms": seconds * 1e3, "score_ms": score_seconds * 1e3, "gso_per_s": ops / seconds / 1e9,
            "score_gso_per_s": ops / score_seconds / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=["nearest", "maxsim"])
    ap.add_argument("--queries", type=int, default=None)
    ap.add_argument("--corpus", type=int, default=65536)
    ap.add_argument("--docs", type=int, default=20000)
    ap.add_argument("--depth", type=int, default=None)
    ap.add_argument("--top", type=int, default=None)
    ap.add_argument("--dtype", default="f16")
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    if a.workload == "nearest":
        out = run_nearest(a.queries or 8192, a.corpus, a.depth or 768, a.top or 10, a.dtype, a.steps)
    else:
        out = run_maxsim(a.queries or 256, a.docs, a.depth or 128, a.top or 100, steps=a.steps)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
