"""Sharded nearest-neighbour and late-interaction search on top of the packed kernels.

One process per GPU. The corpus (or the document collection) is split by rows across ranks - the same
caller-side row partitioning the reference's threading model uses (README.md:199-212 of the reference) -
while the queries are replicated. Every rank searches its own shard with the fused kernels and keeps only
its k best per query; the k-best lists are then merged with a single gather (sharding.merge_topk).
Nothing else crosses GPUs: the data path of a search has no collective.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

from . import angulars_packed_topk, dots_pack, euclideans_packed_topk, maxsim_pack, maxsims_packed, topk_smallest
from . import sharding


def nearest_in_shard(queries: Any, corpus_shard_packed, top: int, *, metric: str = "angular", id_base: int = 0,
                     dtype: Optional[str] = None):
    """k nearest rows of this rank's packed corpus shard for every query: (distances, global ids)."""
    fn = angulars_packed_topk if metric == "angular" else euclideans_packed_topk
    return fn(queries, corpus_shard_packed, top, id_base=id_base, dtype=dtype)


def nearest_sharded(queries: Any, corpus_shard: Any, top: int, *, metric: str = "angular", id_base: int = 0,
                    dtype: Optional[str] = None, group=None, dst: int = 0) -> Tuple[Any, Any]:
    """Packs this rank's corpus shard, searches it, and merges all ranks' results on `dst`.

    `id_base` is the global row index of the shard's first row (sharding.row_shard gives it). Returns
    (distances, ids) on `dst` and (None, None) on the other ranks."""
    packed = dots_pack(corpus_shard, dtype)
    dist, ids = nearest_in_shard(queries, packed, top, metric=metric, id_base=id_base, dtype=dtype)
    return sharding.merge_topk(_as_tensor(dist), _as_tensor(ids), top, group=group, dst=dst)


def maxsim_search_sharded(q_packed, q_offsets, documents_shard: Any, d_offsets_shard, top: int, *, doc_id_base: int = 0,
                          dtype: Optional[str] = None, group=None, dst: int = 0):
    """Late-interaction search: scores every query against every document of this rank's shard with the fused
    MaxSim kernel, keeps the `top` best (smallest summed angular distance) per query and merges across ranks.

    `documents_shard` holds the shard's token vectors back to back, `d_offsets_shard` (length n_docs + 1, starting
    at 0) delimits the documents, `doc_id_base` is the global index of the shard's first document."""
    d_packed = maxsim_pack(documents_shard, dtype)
    scores = maxsims_packed(q_packed, q_offsets, d_packed, d_offsets_shard)
    vals, ids = topk_smallest(scores, top, id_base=doc_id_base)
    return sharding.merge_topk(_as_tensor(vals), _as_tensor(ids), top, group=group, dst=dst)


def _as_tensor(x: Any):
    import torch
    return x if isinstance(x, torch.Tensor) else torch.from_numpy(x)
