"""4-bit packed types (i4 / u4: two values per byte, low nibble first, depth counted in values) through the C ABI:
bit-exact dots against the oracle (itself pinned bit for bit to the reference's scalar kernels), distances within the
tolerance of the 8-bit integer types, odd depths, host and device operands, the symmetric family."""
import numpy as np
import pytest

import numkong_b200 as nk
import oracle

from tests._common import ANGULAR_ATOL, EUCLIDEAN_RTOL

pytestmark = pytest.mark.gpu


def _bytes(rows, depth, seed):
    return np.random.default_rng(seed).integers(0, 256, (rows, (depth + 1) // 2), dtype=np.uint8)


@pytest.mark.parametrize("dtype", ["i4", "u4"])
@pytest.mark.parametrize("shape", [(1, 1, 2), (7, 5, 6), (33, 17, 130), (130, 300, 2000), (64, 257, 4096)])
def test_dots_are_bit_exact(dtype, shape):
    m, n, k = shape
    a, b = _bytes(m, k, 1), _bytes(n, k, 2)
    packed = nk.dots_pack(b, dtype)
    assert packed.depth == k and packed.nbytes == nk.PackedMatrix.packed_size(n, k, dtype)
    c = nk.dots_packed(a, packed, dtype=dtype)
    assert c.dtype == (np.int32 if dtype == "i4" else np.uint32)
    assert np.array_equal(c, oracle.dots(a, b, dtype))


@pytest.mark.parametrize("dtype", ["i4", "u4"])
def test_odd_depth_counts_the_whole_last_byte(dtype):
    """The reference rounds the depth up to a whole byte (include/numkong/dot/serial.h:185-215): the C ABI takes the depth
    in values, so it is exercised directly."""
    import ctypes
    m, n, depth = 9, 11, 77
    a, b = _bytes(m, depth, 3), _bytes(n, depth, 4)
    size = getattr(nk.lib, f"nk_dots_packed_size_{dtype}")(n, depth)
    blob = np.zeros(size, dtype=np.uint8)
    getattr(nk.lib, f"nk_dots_pack_{dtype}")(b.ctypes.data, n, depth, b.strides[0], blob.ctypes.data)
    c = np.zeros((m, n), dtype=np.int32)
    getattr(nk.lib, f"nk_dots_packed_{dtype}")(a.ctypes.data, blob.ctypes.data, c.ctypes.data, m, n, depth, a.strides[0], c.strides[0])
    assert nk.last_error() == ""
    assert np.array_equal(c, oracle.dots(a, b, dtype, depth=depth).astype(np.int32))
    d = np.zeros((m, n), dtype=np.float32)
    getattr(nk.lib, f"nk_angulars_packed_{dtype}")(a.ctypes.data, blob.ctypes.data, d.ctypes.data, m, n, depth, a.strides[0], d.strides[0])
    assert np.max(np.abs(d - oracle.angulars(a, b, dtype, depth=depth))) <= ANGULAR_ATOL


@pytest.mark.parametrize("dtype", ["i4", "u4"])
@pytest.mark.parametrize("op", ["angulars", "euclideans"])
def test_distances(dtype, op):
    m, n, k = 70, 190, 512
    a, b = _bytes(m, k, 5), _bytes(n, k, 6)
    a[3] = 0  # a zero row (both nibble codes of a zero byte are 0): zero-norm rule
    got = getattr(nk, op + "_packed")(a, nk.dots_pack(b, dtype), dtype=dtype)
    want = getattr(oracle, op)(a, b, dtype)
    if op == "angulars":
        assert np.max(np.abs(got - want)) <= ANGULAR_ATOL
    else:
        assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= EUCLIDEAN_RTOL


@pytest.mark.parametrize("dtype", ["i4", "u4"])
def test_device_operands_and_symmetric(dtype):
    import torch
    n, k = 300, 256
    v = _bytes(n, k, 7)
    tv = torch.from_numpy(v).cuda()
    packed = nk.dots_pack(tv, dtype)
    assert packed.is_cuda
    full = nk.dots_packed(tv, packed, dtype=dtype)
    assert nk.synchronize() == 0
    want = oracle.dots(v, v, dtype)
    assert np.array_equal(full.cpu().numpy().view(want.dtype), want)
    out = nk.dots_symmetric(v, dtype=dtype)
    upper = np.triu(np.ones((n, n), dtype=bool))
    assert np.array_equal(out[upper], want[upper]) and np.all(out[~upper] == 0)
    dist = nk.euclideans_symmetric(tv, dtype=dtype, start_row=100, end_row=280)
    assert nk.synchronize() == 0
    ref = oracle.euclideans(v, v, dtype)
    mine = np.zeros((n, n), dtype=bool)
    mine[100:280] = True
    strict = mine & np.triu(np.ones((n, n), dtype=bool), 1)
    got = dist.cpu().numpy()
    assert np.max(np.abs(got[strict] - ref[strict]) / np.maximum(np.abs(ref[strict]), 1e-3)) <= EUCLIDEAN_RTOL
    assert np.all(got[~strict] == 0)


def test_against_the_reference_library_at_a_larger_size():
    ref = oracle.ref()
    if ref is None:
        pytest.skip("reference library was not compiled")
    m, n, k = 256, 512, 8192
    for dtype in ("i4", "u4"):
        a, b = _bytes(m, k, 8), _bytes(n, k, 9)
        ours = nk.dots_packed(a, nk.dots_pack(b, dtype), dtype=dtype)
        theirs = ref.dots(a, b, dtype)
        assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32))
