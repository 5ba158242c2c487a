"""Host-side behaviour around the kernels: cross-shard merge, non-finite inputs in the filtered nearest-k, the cache of
host-resident packed blobs, stream switches, and run-to-run determinism of the CTA-pair kernel."""
import numpy as np
import pytest

import numkong_b200 as nk
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def _stable_merge(values, ids, top):
    parts, rows, k = values.shape
    flat_v = np.transpose(values, (1, 0, 2)).reshape(rows, parts * k)
    flat_i = np.transpose(ids, (1, 0, 2)).reshape(rows, parts * k)
    flat_v = np.where(flat_i < 0, np.float32(np.inf), flat_v)
    order = np.lexsort((flat_i, flat_v), axis=1)[:, :top]
    out_v, out_i = np.take_along_axis(flat_v, order, axis=1), np.take_along_axis(flat_i, order, axis=1)
    return out_v, np.where(np.isinf(out_v) & (out_i < 0), -1, out_i)


@pytest.mark.parametrize("parts,rows,top", [(2, 33, 10), (8, 70, 100), (3, 5, 1), (8, 4, 1024), (5, 9, 7)])
def test_merge_topk_matches_a_stable_sort_by_value_then_id(parts, rows, top):
    """nkb_merge_topk against sorting by (value, id): ties go to the lower id wherever they sit, empty slots (id < 0) lose."""
    import torch
    rng = np.random.default_rng(parts * 1000 + top)
    values = rng.standard_normal((parts, rows, top)).astype(np.float32)
    values = (np.round(values * 4) / 4 + np.float32(0.0)) if top > 1 else values   # many exact ties across and inside the lists (no -0: it sorts before +0)
    ids = rng.permutation(parts * rows * top).reshape(parts, rows, top).astype(np.int64)   # tie order unrelated to list order
    values[:, :, -1:] = np.where(rng.random((parts, rows, 1)) < 0.3, np.float32(0.5), values[:, :, -1:])
    empty = rng.random((parts, rows, top)) < 0.1
    ids[empty] = -1
    values[0, 0, :] = np.float32(1.0)                               # one row of nothing but ties
    want_v, want_i = _stable_merge(values, ids, top)
    got_v, got_i = nk.merge_topk(values, ids)                       # host pointers
    assert np.array_equal(got_i, want_i) and np.array_equal(got_v, want_v)
    dv, di = nk.merge_topk(torch.from_numpy(values).cuda(), torch.from_numpy(ids).cuda(), top=max(1, top // 2))   # device pointers
    assert nk.synchronize() == 0
    assert np.array_equal(di.cpu().numpy(), want_i[:, :max(1, top // 2)]) and np.array_equal(dv.cpu().numpy(), want_v[:, :max(1, top // 2)])


@pytest.mark.parametrize("metric", ["angulars", "euclideans"])
def test_filtered_topk_with_non_finite_rows_equals_materialised(metric):
    """Rows holding Inf or values whose squared norm overflows make NaN / Inf dots. The storing epilogue maps those through
    the full formula (a NaN falls out of the clamp as distance 0); the filtered path must select exactly the same entries,
    so tiles whose norms are not finite may not take the sign-bit prefilter."""
    dtype, m, n, k, top = "bf16", 64, 9000, 64, 10
    a = syn.normal_matrix(m, k, dtype, 71, normalize=True)
    b = syn.normal_matrix(n, k, dtype, 72, normalize=True)
    inf, big = np.uint16(0x7F80), np.uint16(0x7F00)   # +Inf and 1.7e38 as bf16 bits
    b[4000, 3] = inf          # a corpus row with an infinite element, in a filtered panel
    b[7000, :] = big          # a corpus row whose squared norm overflows
    b[100, 5] = inf           # one inside the materialised bootstrap panel
    a[7, 0] = inf             # a query row with an infinite element
    a[9, :] = big
    p = nk.dots_pack(b, dtype)
    full = getattr(nk, metric + "_packed")(a, p)
    assert not np.isnan(full).any()
    order = np.argsort(full, axis=1, kind="stable")[:, :top]
    nk.lib.nkb_set_topk_filter(256)
    try:
        dist, ids = getattr(nk, metric + "_packed_topk")(a, p, top)
    finally:
        nk.lib.nkb_set_topk_filter(1)
    assert np.array_equal(ids, order)
    assert np.array_equal(dist, np.take_along_axis(full, order, axis=1))


def test_cache_of_host_blobs_evicts_unpinned_entries_and_stays_correct():
    """Host-resident packed blobs are uploaded once and cached on the device, eight at a time. A ninth evicts the least
    recently used one that no call in flight has pinned; results stay right for old and new blobs alike."""
    nk.lib.nkb_release_caches()
    a = syn.normal_matrix(50, 128, "i8", 1)
    blobs, wants = [], []
    for i in range(11):
        b = syn.normal_matrix(40 + i, 128, "i8", 10 + i)
        blobs.append(nk.dots_pack(b, "i8"))
        wants.append(a.astype(np.int32) @ b.astype(np.int32).T)
        assert nk.lib.nkb_cached_blob_count() <= 8
    assert nk.lib.nkb_cached_blob_count() == 8
    for i in (0, 10, 3, 1, 9, 0, 5):   # evicted ones are uploaded again, cached ones reused
        assert np.array_equal(nk.dots_packed(a, blobs[i]), wants[i])
        assert nk.lib.nkb_cached_blob_count() <= 8
    nk.lib.nkb_release_caches()
    assert nk.lib.nkb_cached_blob_count() == 0
    assert np.array_equal(nk.dots_packed(a, blobs[2]), wants[2])


def test_switching_streams_between_asynchronous_calls_keeps_their_scratch_ordered():
    """Two distance calls of one thread on two different streams share the thread's row-norm scratch. The second stream is
    put behind the first when the thread switches, so the large first call still reads its own norms."""
    import torch
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    big_a = torch.from_numpy(syn.normal_matrix(8192, 256, "bf16", 81).view(np.int16)).cuda()
    small_a = torch.from_numpy(syn.normal_matrix(64, 256, "bf16", 82, scale=37.0).view(np.int16)).cuda()
    packed = nk.dots_pack(torch.from_numpy(syn.normal_matrix(4096, 256, "bf16", 83).view(np.int16)).cuda(), "bf16")
    want_big = nk.angulars_packed(big_a, packed, dtype="bf16")
    want_small = nk.angulars_packed(small_a, packed, dtype="bf16")
    assert nk.synchronize() == 0
    try:
        for _ in range(3):
            nk.set_stream(s1.cuda_stream)
            got_big = nk.angulars_packed(big_a, packed, dtype="bf16")
            nk.set_stream(s2.cuda_stream)
            got_small = nk.angulars_packed(small_a, packed, dtype="bf16")   # rewrites the first 64 norms
            torch.cuda.synchronize()
            assert torch.equal(got_big, want_big) and torch.equal(got_small, want_small)
    finally:
        nk.set_stream(0)


def test_cta_pair_kernel_is_deterministic_and_equals_the_single_cta_kernel():
    """f16 at depth 8192 hands an accumulator from the MMA issuer to the epilogue warps of BOTH CTAs of a pair sixteen times
    per tile. Twenty runs on one input must give one result, and that of the single-CTA kernel."""
    import torch
    m = n = 4096
    depth = 8192
    a = torch.from_numpy(syn.normal_matrix(m, depth, "f16", 91).view(np.int16)).cuda()
    packed = nk.dots_pack(torch.from_numpy(syn.normal_matrix(n, depth, "f16", 92).view(np.int16)).cuda(), "f16")
    try:
        nk.lib.nkb_set_gemm_variant(1)
        single = nk.dots_packed(a, packed, dtype="f16")
        nk.lib.nkb_set_gemm_variant(3)
        first = nk.dots_packed(a, packed, dtype="f16")
        assert torch.equal(first, single)
        out = torch.empty_like(first)
        for _ in range(20):
            nk.dots_packed(a, packed, out=out, dtype="f16")
            assert torch.equal(out, first)
    finally:
        nk.lib.nkb_set_gemm_variant(0)
    assert nk.synchronize() == 0


@pytest.mark.parametrize("dtype", ["bf16", "i8", "f32", "i4"])
def test_column_ranges_of_a_packed_product_tile_the_full_result(dtype):
    """nkb_dots_packed_columns: the product computed in column blocks (as a caller does that receives the packed matrix
    piecewise) equals the product computed at once, bit for bit, and each call writes its own columns only."""
    import torch
    m, n, k = 300, 1000, 512
    a, b = syn.normal_matrix(m, k // (2 if dtype == "i4" else 1), "u8" if dtype == "i4" else dtype, 61), syn.normal_matrix(n, k // (2 if dtype == "i4" else 1), "u8" if dtype == "i4" else dtype, 62)
    packed = nk.dots_pack(b, dtype)
    whole = nk.dots_packed(a, packed, dtype=dtype)
    out = np.full_like(whole, 7)
    for first, count in ((512, 256), (0, 512), (768, n - 768)):
        nk.dots_packed(a, packed, out=out, dtype=dtype, columns=(first, count))
    assert np.array_equal(out, whole)
    ta = torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()
    tp = nk.dots_pack(torch.from_numpy(b.view(np.int16) if b.dtype == np.uint16 else b).cuda(), dtype)
    dev = torch.full((m, n), 7, dtype=torch.from_numpy(whole[:1]).dtype, device="cuda")
    nk.dots_packed(ta, tp, out=dev, dtype=dtype, columns=(256, 512))
    assert nk.synchronize() == 0
    got = dev.cpu().numpy()
    assert np.array_equal(got[:, 256:768], whole[:, 256:768]) and np.all(got[:, :256] == 7) and np.all(got[:, 768:] == 7)
    with pytest.raises(RuntimeError, match="multiple of 256"):
        nk.dots_packed(a, packed, out=out, dtype=dtype, columns=(100, 200))


@pytest.mark.parametrize("dtype,m,n,k", [("bf16", 1024, 8192, 2048), ("i8", 1000, 8100, 1024), ("f16", 2048, 4096, 1536), ("e4m3", 1024, 8192, 4096)])
def test_depth_split_between_cta_pairs_matches_whole_tiles(dtype, m, n, k):
    """nkb_set_gemm_variant(5): the pipeline stages of all 256 x 256 tiles are dealt out to the CTA pairs in equal shares, so a
    tile's depth may be shared by two pairs whose partial results are added in global memory. Integers: bit-identical to the
    whole-tile kernel. Floats: the two halves are rounded once more when they meet, so the result may differ from the
    whole-tile kernel in the last place but not from one run to the next. The mode is opt-in (it measured slower than whole
    tiles, and the default may not make a row's bits depend on how many rows are multiplied with it): the default equals the
    whole-tile kernel bit for bit."""
    import torch
    import oracle
    a, b = syn.normal_matrix(m, k, dtype, 31), syn.normal_matrix(n, k, dtype, 32)
    store = np.int16 if a.dtype == np.uint16 else a.dtype
    ta, tb = torch.from_numpy(a.view(store)).cuda(), torch.from_numpy(b.view(store)).cuda()
    packed = nk.dots_pack(tb, dtype)
    try:
        nk.lib.nkb_set_gemm_variant(3)
        whole = nk.dots_packed(ta, packed, dtype=dtype)
        nk.lib.nkb_set_gemm_variant(5)
        split = nk.dots_packed(ta, packed, dtype=dtype)
        again = torch.empty_like(split)
        for _ in range(5):
            nk.dots_packed(ta, packed, out=again, dtype=dtype)
            assert torch.equal(again, split)
        nk.lib.nkb_set_gemm_variant(0)
        auto = nk.dots_packed(ta, packed, dtype=dtype)
    finally:
        nk.lib.nkb_set_gemm_variant(0)
    assert nk.synchronize() == 0
    assert torch.equal(auto, whole)
    if dtype == "i8":
        assert torch.equal(split, whole)
        rows = np.r_[0:2, m - 2:m]
        assert np.array_equal(split.cpu().numpy()[rows], oracle.dots(a[rows], b, dtype))
    else:
        assert not torch.equal(split, whole) or k <= 1024   # some tile was really shared
        rows = np.r_[0:8, 250:260, m - 8:m]
        exact = oracle.exact_dots_f64(a[rows], b, dtype)
        scale = np.abs(oracle.decode(a[rows], dtype).astype(np.float64)) @ np.abs(oracle.decode(b, dtype).astype(np.float64)).T
        assert np.max(np.abs(split.cpu().numpy()[rows] - exact) / scale) <= 1.5e-7


def test_sm_budget_changes_the_grid_not_the_result():
    """nkb_set_sm_budget caps how many SMs the persistent GEMM kernels occupy (so that a collective on another stream finds
    room); tiles are dealt to fewer CTAs, every tile is computed the same way."""
    import torch
    a = torch.from_numpy(syn.normal_matrix(2048, 1024, "bf16", 51).view(np.int16)).cuda()
    packed = nk.dots_pack(torch.from_numpy(syn.normal_matrix(6144, 1024, "bf16", 52).view(np.int16)).cuda(), "bf16")
    want = nk.dots_packed(a, packed, dtype="bf16")
    want_angular = nk.angulars_packed(a[:300], packed, dtype="bf16")
    try:
        for budget in (132, 64, 3, 2):
            nk.lib.nkb_set_sm_budget(budget)
            assert torch.equal(nk.dots_packed(a, packed, dtype="bf16"), want), budget
            assert torch.equal(nk.angulars_packed(a[:300], packed, dtype="bf16"), want_angular), budget
    finally:
        nk.lib.nkb_set_sm_budget(0)
    assert nk.synchronize() == 0
