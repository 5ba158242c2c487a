"""One-bit vectors (u1: eight values per byte, depth counted in bits) through the C ABI: AND-popcount dots, Hamming and
Jaccard distances, packed and symmetric. Everything here is exact: the oracle is pinned bit for bit to the reference's
scalar kernels, and the CUDA path must reproduce the oracle bit for bit (the Jaccard division included)."""
import numpy as np
import pytest

import numkong_b200 as nk
import oracle

pytestmark = pytest.mark.gpu


def _bits(rows, depth, seed, density=0.5):
    rng = np.random.default_rng(seed)
    return np.packbits(rng.random((rows, (depth + 7) // 8 * 8)) < density, axis=1, bitorder="little")


@pytest.mark.parametrize("shape", [(1, 1, 8), (7, 5, 24), (33, 17, 1000), (130, 300, 2048), (64, 257, 16384)])
def test_packed_dots_hamming_jaccard_are_bit_exact(shape):
    m, n, k = shape
    a, b = _bits(m, k, 1), _bits(n, k, 2, density=0.3)
    if m > 3:
        a[3] = 0  # the empty set
    packed = nk.dots_pack(b, "u1")
    assert packed.depth == a.shape[1] * 8
    dots = nk.dots_packed(a, packed, dtype="u1")
    assert dots.dtype == np.uint32 and np.array_equal(dots, oracle.dots(a, b, "u1"))
    ham = nk.hammings_packed(a, packed)
    assert ham.dtype == np.uint32 and np.array_equal(ham, oracle.hammings(a, b))
    jac = nk.jaccards_packed(a, packed)
    assert jac.dtype == np.float32 and np.array_equal(jac.view(np.uint32), oracle.jaccards(a, b).view(np.uint32))


def test_depth_inside_the_last_byte_counts_the_whole_byte():
    m, n, depth = 9, 11, 77
    a, b = _bits(m, depth, 3), _bits(n, depth, 4)
    size = nk.lib.nk_dots_packed_size_u1(n, depth)
    blob = np.zeros(size, dtype=np.uint8)
    nk.lib.nk_dots_pack_u1(b.ctypes.data, n, depth, b.strides[0], blob.ctypes.data)
    c = np.zeros((m, n), dtype=np.uint32)
    nk.lib.nk_hammings_packed_u1(a.ctypes.data, blob.ctypes.data, c.ctypes.data, m, n, depth, a.strides[0], c.strides[0])
    assert nk.last_error() == ""
    assert np.array_equal(c, oracle.hammings(a, b, depth=depth))


def test_symmetric_and_device_operands():
    import torch
    n, k = 300, 1024
    v = _bits(n, k, 5)
    tv = torch.from_numpy(v).cuda()
    upper = np.triu(np.ones((n, n), dtype=bool))
    strict = np.triu(np.ones((n, n), dtype=bool), 1)
    dots = nk.dots_symmetric(tv, dtype="u1")
    ham = nk.hammings_symmetric(tv)
    jac = nk.jaccards_symmetric(v, start_row=40, end_row=290)
    assert nk.synchronize() == 0
    assert np.array_equal(dots.cpu().numpy().view(np.uint32)[upper], oracle.dots(v, v, "u1")[upper])
    got = ham.cpu().numpy().view(np.uint32)
    assert np.array_equal(got[strict], oracle.hammings(v, v)[strict]) and np.all(got[~strict] == 0)
    mine = np.zeros((n, n), dtype=bool)
    mine[40:290] = True
    assert np.array_equal(jac[mine & strict].view(np.uint32), oracle.jaccards(v, v)[mine & strict].view(np.uint32))
    assert np.all(jac[~(mine & strict)] == 0)


def test_against_the_reference_library_at_a_larger_size():
    ref = oracle.ref()
    if ref is None:
        pytest.skip("reference library was not compiled")
    m, n, k = 256, 512, 65536
    a, b = _bits(m, k, 8), _bits(n, k, 9)
    packed = nk.dots_pack(b, "u1")
    assert np.array_equal(nk.dots_packed(a, packed, dtype="u1"), ref.dots(a, b, "u1"))
    assert np.array_equal(nk.hammings_packed(a, packed), ref.hammings(a, b))
    assert np.max(np.abs(nk.jaccards_packed(a, packed) - ref.jaccards(a, b))) < 1e-6  # its SIMD division is approximate
