"""Size-independent properties at (or near) the sizes the headline numbers are quoted on, where an element-by-element
oracle would take hours:

  * dots at 8192^3: the checksum identity  sum_j C[i, j] = a_i . (sum_j b_j)  - exact for integers, to rounding for floats;
  * nearest-10 over a million-row corpus: ordering, id range / uniqueness, agreement with the stored-matrix path on
    sampled queries, distances reproduced from the returned ids;
  * all-pairs MaxSim: sampled (query, document) cells equal the single-pair entry point, top-100 equals a stable sort.

Inputs are generated on the device (seeded); nothing here reads the oracle beyond exact decoding of small samples."""
import numpy as np
import pytest

import numkong_b200 as nk
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def _device_rows(torch, rows, depth, dtype, seed):
    from numkong_b200.workloads import _device_rows as make
    return make(torch, rows, depth, dtype, seed)


@pytest.mark.parametrize("dtype", ["i8", "u8"])
def test_integer_dots_checksum_is_exact_at_8192_cubed(dtype):
    import torch
    n = 8192
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    lo, hi, tdt = (-128, 128, torch.int8) if dtype == "i8" else (0, 256, torch.uint8)
    a = torch.randint(lo, hi, (n, n), generator=gen, device="cuda", dtype=torch.int16).to(tdt)
    b = torch.randint(lo, hi, (n, n), generator=gen, device="cuda", dtype=torch.int16).to(tdt)
    c = nk.dots_packed(a, nk.dots_pack(b, dtype), dtype=dtype)
    assert nk.synchronize() == 0
    column_sum = b.to(torch.int64).sum(dim=0)                       # sum_j b_j
    # a_i . sum_j b_j: every product and partial sum stays below 2^53, so the f64 matrix-vector product is exact
    want = (a.double() @ column_sum.double()).to(torch.int64)
    got = c.to(torch.int64).sum(dim=1) if dtype == "i8" else (c.to(torch.int64) & 0xffffffff).sum(dim=1)
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype", ["bf16", "f16", "e4m3", "e2m3"])
def test_float_dots_checksum_at_8192_cubed(dtype):
    import torch
    n = 8192
    if dtype in ("bf16", "f16"):
        a, b = _device_rows(torch, n, n, dtype, 21), _device_rows(torch, n, n, dtype, 22)
        fa, fb = a.double(), b.double()
    else:
        ha, hb = syn.normal_matrix(n, n, dtype, 23), syn.normal_matrix(n, n, dtype, 24)
        import oracle
        a, b = torch.from_numpy(ha).cuda(), torch.from_numpy(hb).cuda()
        fa, fb = torch.from_numpy(oracle.decode(ha, dtype)).cuda().double(), torch.from_numpy(oracle.decode(hb, dtype)).cuda().double()
    c = nk.dots_packed(a, nk.dots_pack(b, dtype), dtype=dtype)
    assert nk.synchronize() == 0
    want = fa @ fb.sum(dim=0)
    scale = fa.abs() @ fb.abs().sum(dim=0)                           # sum_j sum_l |a_il||b_jl|
    err = (c.double().sum(dim=1) - want).abs() / scale
    # every cell is within 2.5e-7 of its own scale (tests/_common.py); the row sums are therefore within that bound too
    assert float(err.max()) < 2.5e-7


def test_nearest_ten_over_a_million_corpus_rows():
    import torch
    queries, corpus, depth, top = 4096, 1_000_000, 768, 10
    tq, tc = _device_rows(torch, queries, depth, "f16", 3), _device_rows(torch, corpus, depth, "f16", 4)
    packed = nk.dots_pack(tc, "f16")
    dist, ids = nk.angulars_packed_topk(tq, packed, top, dtype="f16", id_base=7)
    assert nk.synchronize() == 0 and nk.lib.nkb_topk_filter_fallbacks() >= 0
    assert bool((dist[:, 1:] >= dist[:, :-1]).all())                                   # ascending
    assert int(ids.min()) >= 7 and int(ids.max()) < corpus + 7
    assert bool((torch.sort(ids, dim=1).values[:, 1:] != torch.sort(ids, dim=1).values[:, :-1]).all())  # no id twice
    sample = torch.arange(0, queries, queries // 8, device="cuda")[:8]
    full = nk.angulars_packed(tq[sample].contiguous(), packed, dtype="f16")           # 8 x 1e6 stored distances
    assert nk.synchronize() == 0
    order = torch.sort(full, dim=1, stable=True).indices[:, :top]
    assert torch.equal(ids[sample] - 7, order)
    assert torch.equal(dist[sample], torch.gather(full, 1, order))
    # distances reproduced from the ids alone: gather the winners, multiply again
    winners = tc[(ids[sample][:, 0] - 7)]
    again = nk.angulars_packed(tq[sample].contiguous(), nk.dots_pack(winners.contiguous(), "f16"), dtype="f16")
    assert nk.synchronize() == 0
    assert torch.equal(torch.diagonal(again), dist[sample][:, 0])


def test_all_pairs_maxsim_against_single_pairs_and_stable_sort():
    import torch
    queries, docs, depth, q_tokens, top = 256, 20000, 128, 32, 100
    counts = np.random.default_rng(5).integers(64, 301, size=docs)
    d_off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    q_off = (np.arange(queries + 1) * q_tokens).astype(np.int64)
    q = _device_rows(torch, queries * q_tokens, depth, "bf16", 6)
    d = _device_rows(torch, int(d_off[-1]), depth, "bf16", 7)
    scores = nk.maxsims_packed(nk.maxsim_pack(q, "bf16"), q_off, nk.maxsim_pack(d, "bf16"), d_off)
    vals, ids = nk.topk_smallest(scores, top)
    assert nk.synchronize() == 0
    order = torch.sort(scores, dim=1, stable=True).indices[:, :top]
    assert torch.equal(ids, order) and torch.equal(vals, torch.gather(scores, 1, order))
    rng = np.random.default_rng(8)
    for qi, di in zip(rng.integers(0, queries, 12), rng.integers(0, docs, 12)):
        one = nk.maxsim_packed(nk.maxsim_pack(q[q_off[qi]:q_off[qi + 1]].contiguous(), "bf16"),
                               nk.maxsim_pack(d[d_off[di]:d_off[di + 1]].contiguous(), "bf16"))
        assert abs(float(scores[qi, di]) - one) <= 2e-5 * max(1.0, abs(one))
