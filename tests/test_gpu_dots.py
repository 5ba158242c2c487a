"""Parity of the CUDA packed GEMM and batched distances against the CPU oracle, through the C ABI.

Integers must match bit for bit. Floats must stay within DOT_TOLERANCE (tests/_common.py) of the exact
f64 result, the same statistic the reference's own kernels are measured with."""
import ctypes

import numpy as np
import pytest

import numkong_b200 as nk
import oracle
from tests._common import (ALL_DTYPES, ANGULAR_ATOL, DOT_TOLERANCE, EUCLIDEAN_RTOL, MINIFLOATS, SMALL_SHAPES,
                           TENSOR_DTYPES, make_matrix, normalized_error, ones_matrix)

pytestmark = pytest.mark.gpu


def _check_dots(c, a, b, dtype):
    if dtype in ("i8", "u8"):
        assert np.array_equal(c.view(np.int32), oracle.dots(a, b, dtype).view(np.int32))
    else:
        assert not np.any(np.isnan(c))
        assert normalized_error(c, a, b, dtype) <= DOT_TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("shape", SMALL_SHAPES)
def test_dots_packed_host_buffers(dtype, shape):
    m, n, k = shape
    kind = "codes" if dtype in MINIFLOATS and (m + n) % 2 else "normal"
    a, b = make_matrix(m, k, dtype, 11, kind), make_matrix(n, k, dtype, 12, kind)
    packed = nk.dots_pack(b, dtype)
    assert packed.nbytes == nk.PackedMatrix.packed_size(n, k, dtype)
    c = nk.dots_packed(a, packed)
    assert c.dtype == oracle.out_dtype(dtype)
    _check_dots(c, a, b, dtype)
    # out= path equals the allocating path (test/test_cross.py:306-310 of the reference)
    out = np.full_like(c, 7)
    assert nk.dots_packed(a, packed, out=out) is out
    assert np.array_equal(out.view(np.uint8), c.view(np.uint8))


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_all_ones_known_answers(dtype):
    """rust/matrix.rs:4610-4773: every dot equals the depth, every distance is 0."""
    for (h, w, k) in [(1, 1, 1), (1, 8, 3), (3, 1, 7), (7, 5, 3), (33, 17, 65)]:
        a, b = ones_matrix(h, k, dtype), ones_matrix(w, k, dtype)
        p = nk.dots_pack(b, dtype)
        assert np.all(nk.dots_packed(a, p) == k)
        assert np.all(nk.angulars_packed(a, p) <= 5e-7)
        assert np.all(nk.euclideans_packed(a, p) <= 2e-3)


def test_tiny_integer_and_identity_known_answers():
    """golang/unit_test.go:558-652 and test/test.mjs:167-200 of the reference."""
    a = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.int8)
    b = np.array([[7, 8, 9], [10, 11, 12]], dtype=np.int8)
    assert np.array_equal(nk.dots_packed(a, nk.dots_pack(b)), np.array([[50, 68], [122, 167]], dtype=np.int32))
    a = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9], [10, 11, 12]], dtype=np.float32)
    b = np.array([[1, 0, 0], [0, 1, 0], [0, 0, 1], [1, 1, 0], [1, 1, 1]], dtype=np.float32)
    expect = np.array([[1, 2, 3, 3, 6], [4, 5, 6, 9, 15], [7, 8, 9, 15, 24], [10, 11, 12, 21, 33]], dtype=np.float64)
    assert np.array_equal(nk.dots_packed(a, nk.dots_pack(b)), expect)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("shape", [(33, 17, 65), (130, 300, 768), (64, 1000, 96)])
def test_batched_distances(dtype, shape):
    m, n, k = shape
    a, b = make_matrix(m, k, dtype, 21), make_matrix(n, k, dtype, 22)
    p = nk.dots_pack(b, dtype)
    ang, euc = nk.angulars_packed(a, p), nk.euclideans_packed(a, p)
    ref_ang, ref_euc = oracle.angulars(a, b, dtype), oracle.euclideans(a, b, dtype)
    assert ang.dtype == ref_ang.dtype and euc.dtype == ref_euc.dtype
    assert np.all(ang >= 0) and np.all(euc >= 0)
    atol = 1e-12 if dtype == "f32" else ANGULAR_ATOL
    rtol = 1e-12 if dtype == "f32" else EUCLIDEAN_RTOL
    assert np.max(np.abs(ang - ref_ang)) <= atol
    assert np.max(np.abs(euc - ref_euc) / np.maximum(np.abs(ref_euc), 1e-3)) <= rtol


@pytest.mark.parametrize("dtype", ["bf16", "i8", "f32", "e4m3"])
def test_zero_rows_follow_the_batched_zero_norm_rule(dtype):
    """include/numkong/spatial/serial.h:261-267."""
    a, b = make_matrix(5, 40, dtype, 31), make_matrix(6, 40, dtype, 32)
    a[1] = 0
    b[2] = 0
    p = nk.dots_pack(b, dtype)
    ang, euc = nk.angulars_packed(a, p), nk.euclideans_packed(a, p)
    assert np.all(ang[1] == 0) and np.all(ang[:, 2] == 0)
    ref_euc = oracle.euclideans(a, b, dtype)
    assert np.allclose(euc, ref_euc, rtol=1e-5, atol=1e-5)
    assert euc[1, 2] == 0


@pytest.mark.parametrize("dtype", ["i8", "bf16", "e5m2", "e2m3", "f32"])
def test_strided_and_unaligned_inputs_and_outputs(dtype):
    """The reference accepts any byte stride and alignment (CPU loads are unaligned, include/numkong/dots.h:60-72)."""
    import torch
    m, n, k = 37, 45, 77
    eb = nk.DTYPE_BYTES[dtype]
    a_wide, b_wide = make_matrix(m, k + 13, dtype, 41), make_matrix(n, k + 5, dtype, 42)
    a, b = a_wide[:, 3:3 + k], b_wide[:, 1:1 + k]           # odd byte offsets and strides
    assert a.strides[0] != k * eb
    packed = nk.dots_pack(b, dtype)
    ref = oracle.dots(np.ascontiguousarray(a), np.ascontiguousarray(b), dtype)
    out_wide = np.zeros((m, n + 3), dtype=ref.dtype)
    out = out_wide[:, 1:1 + n]
    nk.dots_packed(a, packed, out=out)
    _check_dots(np.ascontiguousarray(out), np.ascontiguousarray(a), np.ascontiguousarray(b), dtype)
    assert np.all(out_wide[:, 0] == 0) and np.all(out_wide[:, -2:] == 0)   # nothing written outside the rows
    # The same through device memory, still strided and misaligned.
    tdt = {1: torch.uint8, 2: torch.int16, 4: torch.float32}[eb]
    ta = torch.from_numpy(a_wide.view({1: np.uint8, 2: np.int16, 4: np.float32}[eb])).cuda()[:, 3:3 + k]
    tb = torch.from_numpy(b_wide.view({1: np.uint8, 2: np.int16, 4: np.float32}[eb])).cuda()[:, 1:1 + k]
    assert ta.dtype == tdt
    tp = nk.dots_pack(tb, dtype)
    tc = nk.dots_packed(ta, tp, dtype=dtype)
    assert nk.synchronize() == 0
    assert np.array_equal(tc.cpu().numpy().view(np.uint8), np.ascontiguousarray(out).view(np.uint8))


@pytest.mark.parametrize("dtype", ["u8", "f16", "e3m2"])
def test_packed_blob_is_relocatable_and_reusable(dtype):
    """Callers memcpy / clone / serialise the blob (rust/matrix.rs:2578-2607, python/matrix.c:743)."""
    import torch
    a, b = make_matrix(20, 100, dtype, 51), make_matrix(30, 100, dtype, 52)
    p = nk.dots_pack(b, dtype)
    first = nk.dots_packed(a, p)
    moved = nk.PackedMatrix(np.frombuffer(bytes(p.buffer.tobytes()), dtype=np.uint8).copy(), dtype, p.width, p.depth)
    assert np.array_equal(nk.dots_packed(a, moved).view(np.uint8), first.view(np.uint8))
    on_device = nk.PackedMatrix(torch.from_numpy(p.buffer.copy()).cuda(), dtype, p.width, p.depth)
    assert np.array_equal(nk.dots_packed(a, on_device).view(np.uint8), first.view(np.uint8))
    # and a blob packed on the device works from host memory
    tb = torch.from_numpy(b.view(np.uint8 if b.itemsize == 1 else np.int16)).cuda()
    dev_packed = nk.dots_pack(tb, dtype)
    nk.synchronize()
    back = nk.PackedMatrix(dev_packed.buffer.cpu().numpy(), dtype, p.width, p.depth)
    assert np.array_equal(nk.dots_packed(a, back).view(np.uint8), first.view(np.uint8))


def test_row_slices_of_a_share_one_packed_matrix():
    """Callers split rows of A over threads against one packed B (README.md:199-212, python/matrix.c:473-482)."""
    a, b = make_matrix(300, 128, "i8", 61), make_matrix(70, 128, "i8", 62)
    p = nk.dots_pack(b)
    whole = nk.dots_packed(a, p)
    out = np.zeros_like(whole)
    for lo in range(0, 300, 64):
        nk.dots_packed(a[lo:lo + 64], p, out=out[lo:lo + 64])
    assert np.array_equal(out, whole)


def test_failure_convention_fills_the_output_with_ff():
    """c/numkong.c:78-81, 209-216: no error codes, the output is filled with 0xFF."""
    a, b = make_matrix(4, 16, "bf16", 71), make_matrix(5, 16, "bf16", 72)
    p = nk.dots_pack(b, "bf16")
    out = np.zeros((4, 5), dtype=np.float32)
    # depth that does not match the blob, straight through the C ABI
    nk.lib.nk_dots_packed_bf16(a.ctypes.data, p.buffer.ctypes.data, out.ctypes.data, 4, 5, 8, 32, 20)
    assert nk.last_error() != ""
    assert np.all(out.view(np.uint8) == 0xFF)
    garbage = np.zeros(p.nbytes, dtype=np.uint8)
    nk.lib.nk_dots_packed_bf16(a.ctypes.data, garbage.ctypes.data, out.ctypes.data, 4, 5, 16, 32, 20)
    assert "pack" in nk.last_error()
    nk.lib.nk_dots_packed_bf16(a.ctypes.data, p.buffer.ctypes.data, out.ctypes.data, 4, 5, 16, 32, 20)
    assert nk.last_error() == ""
    assert not np.any(np.isnan(out))
    # empty problems are no-ops, zero depth gives zeros
    nk.lib.nk_dots_packed_bf16(a.ctypes.data, p.buffer.ctypes.data, out.ctypes.data, 0, 5, 16, 32, 20)
    assert nk.last_error() == ""
    z = nk.dots_pack(np.zeros((5, 0), dtype=np.uint16), "bf16")
    out[:] = 3
    nk.lib.nk_dots_packed_bf16(a.ctypes.data, z.buffer.ctypes.data, out.ctypes.data, 4, 5, 0, 32, 20)
    assert nk.last_error() == "" and np.all(out == 0)


def test_config_1_i8_2048_cubed_is_bit_exact():
    """dots_packed i8 x i8 -> i32, A and B 2048 x 2048, int8 uniform in [-128, 127] from seed 0."""
    rng = np.random.default_rng(0)
    a = rng.integers(-128, 128, size=(2048, 2048), dtype=np.int8)
    b = rng.integers(-128, 128, size=(2048, 2048), dtype=np.int8)
    c = nk.dots_packed(a, nk.dots_pack(b))
    exact = (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.int64)   # every partial sum < 2^53: exact
    assert np.array_equal(c.astype(np.int64), exact)
    assert np.array_equal(c[:16], oracle.dots(a[:16], b, "i8"))


@pytest.mark.parametrize("dtype", TENSOR_DTYPES)
def test_full_size_8192_properties(dtype):
    """At 8192^3 the oracle is too slow for the whole result; check rows against it and size-independent
    properties: the result is independent of how rows of A are grouped, and (for integers) exact."""
    import torch
    n = k = 8192
    m = 1024
    a, b = make_matrix(m, k, dtype, 81), make_matrix(n, k, dtype, 82)
    store = {1: (np.uint8, torch.uint8), 2: (np.int16, torch.int16)}[a.itemsize]
    ta, tb = torch.from_numpy(a.view(store[0])).cuda(), torch.from_numpy(b.view(store[0])).cuda()
    p = nk.dots_pack(tb, dtype)
    c = nk.dots_packed(ta, p, dtype=dtype)
    assert nk.synchronize() == 0
    ch = c.cpu().numpy()
    rows = [0, 1, 127, 128, 640, 1023]
    _check_dots(ch[rows], a[rows], b, dtype)
    # grouping of rows does not change any bit
    c2 = nk.dots_packed(ta[128:640], p, dtype=dtype)
    nk.synchronize()
    assert torch.equal(c2, c[128:640])
    if dtype in ("i8", "u8"):
        exact = (a[:256].astype(np.float64) @ b.astype(np.float64).T).astype(np.int64)
        got = ch[:256].astype(np.int64) if dtype == "i8" else ch[:256].view(np.uint32).astype(np.int64)
        assert np.array_equal(got, exact)
