"""Sharded nearest-k and MaxSim search: two ranks, each searching its own shard with the CUDA kernels, merged with
one gather. Both ranks share cuda:0 here and the merge travels over gloo, so the test needs one GPU only (the kernels
of the two ranks are independent launches; nothing on the device waits for the other rank)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import numkong_b200 as nk
        import oracle
        from numkong_b200 import search, sharding, synthetic as syn
        torch.cuda.set_device(0)
        # ---- nearest-10 by angular distance over a row-sharded f16 corpus
        n, k, top = 3001, 96, 10
        queries = syn.normal_matrix(40, k, "f16", 11, normalize=True)
        corpus = syn.normal_matrix(n, k, "f16", 12, normalize=True)
        lo, hi = sharding.row_shard(n, world, rank)
        tq = torch.from_numpy(queries.view(np.int16)).cuda()
        shard = torch.from_numpy(corpus[lo:hi].view(np.int16)).cuda()
        dist_m, ids_m = search.nearest_sharded(tq, shard, top, metric="angular", id_base=lo, dtype="f16")
        if rank == 0:
            full = nk.angulars_packed(queries, nk.dots_pack(corpus, "f16"))
            order = np.argsort(full, axis=1, kind="stable")[:, :top]
            assert np.array_equal(ids_m.numpy(), order)
            assert np.array_equal(dist_m.numpy(), np.take_along_axis(full, order, axis=1))
        # ---- MaxSim top-5 over a document-sharded collection
        rng = np.random.default_rng(3)
        counts = rng.integers(20, 90, size=37)
        d_off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        docs = syn.normal_matrix(int(d_off[-1]), 64, "bf16", 13, normalize=True)
        q_counts = [32, 32, 8]
        q_off = np.concatenate([[0], np.cumsum(q_counts)]).astype(np.int64)
        qs = syn.normal_matrix(int(q_off[-1]), 64, "bf16", 14, normalize=True)
        runs = sharding.token_balanced_shards(torch.from_numpy(d_off), world)
        d0, d1 = runs[rank]
        local_off = d_off[d0:d1 + 1] - d_off[d0]
        q_packed = nk.maxsim_pack(torch.from_numpy(qs.view(np.int16)).cuda(), "bf16")
        shard_docs = torch.from_numpy(docs[d_off[d0]:d_off[d1]].view(np.int16)).cuda()
        vals, ids = search.maxsim_search_sharded(q_packed, q_off, shard_docs, local_off, 5, doc_id_base=d0, dtype="bf16")
        if rank == 0:
            want = np.array([[oracle.maxsim(qs[q_off[i]:q_off[i + 1]], docs[d_off[j]:d_off[j + 1]], "bf16") for j in range(len(counts))]
                             for i in range(len(q_counts))])
            order = np.argsort(want, axis=1, kind="stable")[:, :5]
            got_ids = ids.numpy()
            # scores agree to rounding, so compare the score of each returned document with the oracle's ranking
            assert np.allclose(vals.numpy(), np.take_along_axis(want, order, axis=1), rtol=2e-5, atol=2e-5)
            assert np.allclose(np.take_along_axis(want, got_ids, axis=1), vals.numpy(), rtol=2e-5, atol=2e-5)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_search_on_one_gpu(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
