"""Parity of the fused MaxSim kernel, its all-pairs batch form, and the top-k selection, against the CPU
oracle, through the C ABI."""
import numpy as np
import pytest

import numkong_b200 as nk
import oracle
from tests._common import make_matrix
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu

# The reference's own back ends disagree with each other by more than this on MaxSim (serial vs fused:
# ~0.5 %); against the oracle with the SAME semantics the sum of n_q angulars agrees to f32 rounding.
MAXSIM_RTOL = 2e-5


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("shape", [(32, 180, 128), (8, 64, 64), (5, 3, 17), (1, 1, 1), (130, 257, 96), (256, 128, 1024), (32, 300, 128)])
def test_maxsim_single_pair(dtype, shape):
    nq, nd, k = shape
    q, d = make_matrix(nq, k, dtype, 101), make_matrix(nd, k, dtype, 102)
    got = nk.maxsim(q, d, dtype)
    want = oracle.maxsim(q, d, dtype)
    assert abs(got - want) <= MAXSIM_RTOL * max(1.0, abs(want))
    assert got >= oracle.maxsim_exhaustive(q, d, dtype) - 1e-3


@pytest.mark.parametrize("dist", ["unit", "normal"])
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [(32, 180, 128), (130, 257, 96), (256, 128, 1024), (32, 300, 128)])
def test_maxsim_two_sided_against_the_exhaustive_reference(dtype, shape, dist):
    """The reference's own test compares every back end with the exhaustive sum of minimum angular distances
    (include/numkong/maxsim.hpp:84-110, test/test_maxsim.cpp:51-57). Two gates, both two-sided: on L2-normalised
    vectors (where the largest dot is the smallest angular distance) the device result lies within 6.7e-5 relative of it,
    the distance the reference publishes for its own fused tensor-engine back end; on any input it is no further from it
    than the worst of the reference's back ends on the same inputs (its scalar back end screens in 8 bits and sits at
    up to 1e-2), with a factor of 1.25 and the f32 rounding of the sum on top."""
    nq, nd, k = shape
    normalize = dist == "unit"
    q, d = syn.normal_matrix(nq, k, dtype, 111, normalize=normalize), syn.normal_matrix(nd, k, dtype, 112, normalize=normalize)
    got = nk.maxsim(q, d, dtype)
    exhaustive = oracle.maxsim_exhaustive(q, d, dtype)
    scale = max(1.0, abs(exhaustive))
    if normalize:
        assert abs(got - exhaustive) <= 6.7e-5 * scale
    backends = [r for r in (oracle.ref(), oracle.ref_serial()) if r is not None]
    if not backends:
        pytest.skip("the reference was not compiled into oracle/_ref")
    envelope = max(abs(r.maxsim(q, d, dtype) - exhaustive) for r in backends)
    assert abs(got - exhaustive) <= 1.25 * envelope + 2e-5 * scale, (got, exhaustive, envelope)


def test_all_pairs_batch_is_bit_identical_from_run_to_run():
    """Every (query, document) sum is finished by one warp when the query's tokens sit in one 32-row group (a plain store),
    and by two commuting additions when they straddle two; either way the matrix is the same bits every time."""
    import torch
    rng = np.random.default_rng(17)
    depth = 128
    q_counts = [32] * 6 + [7, 40, 32, 19, 32]          # aligned queries, then queries that straddle 32-row groups and tiles
    d_counts = list(rng.integers(64, 301, size=400))
    q_off = np.concatenate([[0], np.cumsum(q_counts)]).astype(np.int64)
    d_off = np.concatenate([[0], np.cumsum(d_counts)]).astype(np.int64)
    tq = nk.maxsim_pack(torch.from_numpy(syn.normal_matrix(int(q_off[-1]), depth, "bf16", 211, normalize=True).view(np.int16)).cuda(), "bf16")
    td = nk.maxsim_pack(torch.from_numpy(syn.normal_matrix(int(d_off[-1]), depth, "bf16", 212, normalize=True).view(np.int16)).cuda(), "bf16")
    first = nk.maxsims_packed(tq, q_off, td, d_off).clone()
    for _ in range(5):
        assert torch.equal(nk.maxsims_packed(tq, q_off, td, d_off), first)
    assert nk.synchronize() == 0


@pytest.mark.parametrize("depth", [128, 96, 320])
def test_all_pairs_batch_is_the_same_on_the_callers_layout_and_on_32_token_boundaries(depth):
    """The batch form scans a copy of the documents in which every document starts on a multiple of 32 tokens and its last
    token is repeated up to the next one (bit 24 of the tuning word switches the copy off). A repeated token ties with the
    real one and ties go to the lower position, so both layouts must give the same bits - for ragged lengths, one-token
    documents, documents that already are multiples of 32, queries that straddle row groups, and (depth 320) the deep-query
    pipeline."""
    import torch
    rng = np.random.default_rng(23)
    q_counts = [32, 32, 7, 40, 32, 19]
    d_counts = list(rng.integers(1, 301, size=300)) + [1, 32, 64, 31, 33, 256, 255, 257]
    q_off = np.concatenate([[0], np.cumsum(q_counts)]).astype(np.int64)
    d_off = np.concatenate([[0], np.cumsum(d_counts)]).astype(np.int64)
    tq = nk.maxsim_pack(torch.from_numpy(syn.normal_matrix(int(q_off[-1]), depth, "bf16", 221).view(np.int16)).cuda(), "bf16")
    td = nk.maxsim_pack(torch.from_numpy(syn.normal_matrix(int(d_off[-1]), depth, "bf16", 222).view(np.int16)).cuda(), "bf16")
    try:
        nk.lib.nkb_set_gemm_variant(1 << 24)
        plain = nk.maxsims_packed(tq, q_off, td, d_off).clone()
    finally:
        nk.lib.nkb_set_gemm_variant(0)
    padded = nk.maxsims_packed(tq, q_off, td, d_off)
    assert nk.synchronize() == 0
    assert torch.equal(plain, padded)


def test_maxsim_of_identical_sides_is_zero():
    """test/test_maxsim.py:169-175 of the reference."""
    x = np.ones((8, 64), dtype=np.float32)
    assert abs(nk.maxsim(x, x)) < 1e-5
    xb = syn.encode(x, "bf16")
    assert abs(nk.maxsim(xb, xb, "bf16")) < 1e-5


def test_maxsim_ties_go_to_the_first_document_vector():
    """Strict > on the raw dot: maxsim/serial.h:358-361, maxsim/sapphireamx.h:799-805."""
    k = 32
    q = syn.encode(np.ones((1, k), dtype=np.float32), "bf16")
    d = np.ones((3, k), dtype=np.float32)
    d[0, : k // 2] = 2.0        # dot 48, norm larger
    d[1] = 1.5                  # dot 48 as well, but perfectly aligned with q (cosine 1)
    d[2] = 0.5
    db = syn.encode(d, "bf16")
    got = nk.maxsim(q, db, "bf16")
    want, best = oracle.maxsim(q, db, "bf16", want_best=True)
    assert best[0] == 0
    assert abs(got - want) < 1e-6 and got > 1e-3   # the first (worse-aligned) vector was kept


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_all_pairs_batch_matches_pairwise_calls(dtype):
    rng = np.random.default_rng(7)
    depth = 128
    q_counts = [32, 32, 7, 40, 32]
    d_counts = list(rng.integers(64, 301, size=23)) + [1, 256, 255, 257]
    q_off = np.concatenate([[0], np.cumsum(q_counts)]).astype(np.int64)
    d_off = np.concatenate([[0], np.cumsum(d_counts)]).astype(np.int64)
    q_all = syn.normal_matrix(int(q_off[-1]), depth, dtype, 201, normalize=True)
    d_all = syn.normal_matrix(int(d_off[-1]), depth, dtype, 202, normalize=True)
    scores = nk.maxsims_packed(nk.maxsim_pack(q_all, dtype), q_off, nk.maxsim_pack(d_all, dtype), d_off)
    assert scores.shape == (len(q_counts), len(d_counts))
    for qi in range(len(q_counts)):
        for di in range(len(d_counts)):
            want = oracle.maxsim(q_all[q_off[qi]:q_off[qi + 1]], d_all[d_off[di]:d_off[di + 1]], dtype)
            assert abs(scores[qi, di] - want) <= MAXSIM_RTOL * max(1.0, want), (qi, di)
    # device-resident operands give the same matrix
    import torch
    store = np.int16
    tq = nk.maxsim_pack(torch.from_numpy(q_all.view(store)).cuda(), dtype)
    td = nk.maxsim_pack(torch.from_numpy(d_all.view(store)).cuda(), dtype)
    dev = nk.maxsims_packed(tq, q_off, td, d_off)
    assert nk.synchronize() == 0
    assert np.allclose(dev.cpu().numpy(), scores, rtol=1e-6, atol=1e-6)


def test_topk_smallest_matches_a_stable_sort():
    rng = np.random.default_rng(9)
    x = rng.standard_normal((37, 5000)).astype(np.float32)
    x[3, :] = 1.0                      # all ties: lowest columns win
    x[4, 100:200] = x[4, 0]            # ties in the middle
    x[5, :7] = np.inf
    for top in (1, 10, 100, 1000):
        vals, ids = nk.topk_smallest(x, top, id_base=1000)
        order = np.argsort(x, axis=1, kind="stable")[:, :top]
        assert np.array_equal(ids - 1000, order)
        assert np.array_equal(vals, np.take_along_axis(x, order, axis=1))
    vals, ids = nk.topk_smallest(x[:, :5], 8)
    assert np.all(ids[:, 5:] == -1) and np.all(np.isinf(vals[:, 5:]))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("metric", ["angulars", "euclideans"])
def test_distance_topk_equals_full_matrix_then_select(dtype, metric):
    m, n, k, top = 70, 3000, 96, 10
    a = syn.normal_matrix(m, k, dtype, 301, normalize=True)
    b = syn.normal_matrix(n, k, dtype, 302, normalize=True)
    p = nk.dots_pack(b, dtype)
    full = getattr(nk, metric + "_packed")(a, p)
    dist, ids = getattr(nk, metric + "_packed_topk")(a, p, top, id_base=5)
    order = np.argsort(full, axis=1, kind="stable")[:, :top]
    assert np.array_equal(ids - 5, order)
    assert np.array_equal(dist, np.take_along_axis(full, order, axis=1))
    # many narrow panels exercise the running merge
    nk.lib.nkb_set_topk_panel_rows(512)
    try:
        dist2, ids2 = getattr(nk, metric + "_packed_topk")(a, p, top, id_base=5)
    finally:
        nk.lib.nkb_set_topk_panel_rows(0)
    assert np.array_equal(ids2, ids) and np.array_equal(dist2, dist)
    # and the distances themselves agree with the oracle
    ref = getattr(oracle, metric)(a, b, dtype)
    assert np.max(np.abs(dist - np.take_along_axis(ref, order, axis=1))) < 2e-6


def _select_reference(full, top):
    order = np.argsort(full, axis=1, kind="stable")[:, :top]
    return np.take_along_axis(full, order, axis=1), order


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("metric", ["angulars", "euclideans"])
def test_distance_topk_filtered_equals_materialised(dtype, metric):
    """The filter epilogue + refine kernels return exactly what selecting from the stored matrix returns,
    for ragged shapes, duplicated packed rows (ties go to the lower id) and every k the filter serves."""
    m, n, k = 200, 9001, 64
    a = syn.normal_matrix(m, k, dtype, 311, normalize=True)
    b = syn.normal_matrix(n, k, dtype, 312, normalize=True)
    b[5000:8000] = b[:3000]  # exact duplicates in later panels
    p = nk.dots_pack(b, dtype)
    full = getattr(nk, metric + "_packed")(a, p)
    before = nk.lib.nkb_topk_filter_fallbacks()
    try:
        for top in (1, 10, 100, 128):
            want_d, want_i = _select_reference(full, top)
            nk.lib.nkb_set_topk_filter(256)
            dist, ids = getattr(nk, metric + "_packed_topk")(a, p, top, id_base=7)
            assert np.array_equal(ids - 7, want_i), top
            assert np.array_equal(dist, want_d), top
            nk.lib.nkb_set_topk_filter(0)
            dist0, ids0 = getattr(nk, metric + "_packed_topk")(a, p, top, id_base=7)
            assert np.array_equal(ids0, ids) and np.array_equal(dist0, dist)
    finally:
        nk.lib.nkb_set_topk_filter(1)
    assert nk.lib.nkb_topk_filter_fallbacks() == before  # random order never overflows a candidate list
    # default mode picks the filter by itself at this size (>= 8192 packed rows)
    launches = nk.launch_count()
    dist, ids = getattr(nk, metric + "_packed_topk")(a, p, 10)
    want_d, want_i = _select_reference(full, 10)
    assert np.array_equal(ids, want_i) and np.array_equal(dist, want_d)
    # norms, bootstrap GEMM + select, threshold init, one filtered panel (GEMM + refine), possibly a staging kernel
    assert 6 <= nk.launch_count() - launches <= 7


def test_distance_topk_filter_overflow_falls_back():
    """Packed rows ordered from far to near make every later value beat the threshold: the candidate lists
    overflow, the call is redone on the materialising path, and the answer is still exact."""
    dtype, m, n, k, top = "f16", 40, 6000, 64, 10
    rng = np.random.default_rng(5)
    direction = rng.standard_normal(k)
    a = syn.encode((direction + 0.05 * rng.standard_normal((m, k))), dtype)
    mix = np.linspace(-1.0, 1.0, n)[:, None]
    b = syn.encode(mix * direction + 0.3 * rng.standard_normal((n, k)), dtype)
    p = nk.dots_pack(b, dtype)
    full = nk.angulars_packed(a, p)
    want_d, want_i = _select_reference(full, top)
    before = nk.lib.nkb_topk_filter_fallbacks()
    nk.lib.nkb_set_topk_filter(256)
    try:
        dist, ids = nk.angulars_packed_topk(a, p, top)
    finally:
        nk.lib.nkb_set_topk_filter(1)
    assert nk.lib.nkb_topk_filter_fallbacks() == before + 1
    assert np.array_equal(ids, want_i) and np.array_equal(dist, want_d)
