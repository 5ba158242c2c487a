"""Symmetric products and distance matrices (nk_dots_symmetric_<t>, nk_angulars_symmetric_<t>,
nk_euclideans_symmetric_<t>) through the C ABI, against the packed path, the oracle and - when it was compiled - the
reference's own kernels. The contract under test (include/numkong/dots/serial.h:1958-2440, :2802-2872 of the
reference): only rows [start_row, end_row) are touched, only cells with column >= row; dots keep the squared norm
on the diagonal, distances put 0 there."""
import ctypes

import numpy as np
import pytest

import numkong_b200 as nk
import oracle
from numkong_b200 import synthetic as syn

from tests._common import ANGULAR_ATOL, DOT_TOLERANCE, EUCLIDEAN_RTOL, make_matrix

pytestmark = pytest.mark.gpu

ALL = ["i8", "u8", "bf16", "f16", "e4m3", "e5m2", "e2m3", "e3m2", "f32"]


def _vectors(n, k, dtype, seed):
    if dtype == "i8":
        return np.random.default_rng(seed).integers(-128, 128, (n, k), dtype=np.int8)
    if dtype == "u8":
        return np.random.default_rng(seed).integers(0, 256, (n, k), dtype=np.uint8)
    if dtype == "f32":
        return np.random.default_rng(seed).standard_normal((n, k)).astype(np.float32)
    return make_matrix(n, k, dtype, seed)


def _sentinel(n, dtype, op):
    cell = np.float64 if dtype == "f32" else (np.int32 if dtype == "i8" and op == "dots" else np.uint32 if dtype == "u8" and op == "dots" else np.float32)
    out = np.empty((n, n), dtype=cell)
    out.view(np.uint8)[:] = 0xAB
    return out


@pytest.mark.parametrize("dtype", ALL)
def test_dots_symmetric_matches_packed_path_and_leaves_the_rest_alone(dtype):
    n, k = 300, 96
    v = _vectors(n, k, dtype, 41)
    full = nk.dots_packed(v, nk.dots_pack(v, dtype), dtype=dtype)
    upper = np.triu(np.ones((n, n), dtype=bool))
    out = _sentinel(n, dtype, "dots")
    before = out.copy()
    got = nk.dots_symmetric(v, dtype=dtype, out=out)
    assert got is out
    assert np.array_equal(out[upper], full[upper])                                   # same kernel, same bits
    assert np.array_equal(out[~upper].view(np.uint8), before[~upper].view(np.uint8))  # below the diagonal: untouched
    want = oracle.dots(v, v, dtype)
    if dtype in ("i8", "u8"):
        assert np.array_equal(out[upper], want[upper])
    else:
        scale = np.abs(oracle.decode(v, dtype).astype(np.float64)) @ np.abs(oracle.decode(v, dtype).astype(np.float64)).T
        exact = oracle.exact_dots_f64(v, v, dtype)
        err = np.abs(out.astype(np.float64) - exact) / np.maximum(scale, 1e-30)
        assert err[np.triu(upper, 1)].max() <= DOT_TOLERANCE[dtype]
        # The diagonal is a sum of squares: no cancellation, and the tensor cores truncate towards zero every time a
        # 32-byte slice of depth is added to the accumulator, so those errors all point the same way - at most one
        # f32 ulp (2^-24 relative to the sum) per slice.
        slices = -(-k * v.itemsize // 32)
        assert np.diag(err).max() <= (1e-15 if dtype == "f32" else (slices + 1) * 2.0 ** -24)


@pytest.mark.parametrize("dtype", ["bf16", "i8", "f32", "e2m3"])
@pytest.mark.parametrize("rows", [(100, 280), (260, 300), (0, 1), (299, 300), (32, 64)])
def test_row_slices_touch_only_their_rows(dtype, rows):
    n, k = 300, 80
    v = _vectors(n, k, dtype, 43)
    whole = nk.dots_symmetric(v, dtype=dtype)
    out = _sentinel(n, dtype, "dots")
    before = out.copy()
    nk.dots_symmetric(v, dtype=dtype, out=out, start_row=rows[0], end_row=rows[1])
    mine = np.zeros((n, n), dtype=bool)
    mine[rows[0]:rows[1]] = True
    mine &= np.triu(np.ones((n, n), dtype=bool))
    assert np.array_equal(out[mine], whole[mine])
    assert np.array_equal(out[~mine].view(np.uint8), before[~mine].view(np.uint8))


@pytest.mark.parametrize("dtype", ALL)
@pytest.mark.parametrize("op", ["angulars", "euclideans"])
def test_distance_matrices(dtype, op):
    n, k = 270, 64
    v = _vectors(n, k, dtype, 47)
    v[5] = 0  # a zero vector exercises the zero-norm rule
    full = getattr(nk, op + "_packed")(v, nk.dots_pack(v, dtype), dtype=dtype)
    strict = np.triu(np.ones((n, n), dtype=bool), 1)
    out = _sentinel(n, dtype, op)
    before = out.copy()
    getattr(nk, op + "_symmetric")(v, dtype=dtype, out=out)
    assert np.array_equal(out[strict], full[strict])
    assert np.all(np.diag(out) == 0)
    lower = np.tril(np.ones((n, n), dtype=bool), -1)
    assert np.array_equal(out[lower].view(np.uint8), before[lower].view(np.uint8))
    want = getattr(oracle, op)(v, v, dtype)
    if op == "angulars":
        assert np.max(np.abs(out[strict].astype(np.float64) - want[strict])) <= (1e-12 if dtype == "f32" else ANGULAR_ATOL)
    else:
        rel = np.abs(out[strict].astype(np.float64) - want[strict]) / np.maximum(np.abs(want[strict]), 1e-3)
        assert rel.max() <= (1e-12 if dtype == "f32" else 2 * EUCLIDEAN_RTOL)


@pytest.mark.parametrize("n,k", [(1500, 256), (2400, 2048)])
def test_device_resident_and_large_enough_for_tile_skipping(n, k):
    """Many tiles (and, at depth 2048, the CTA-pair kernel): tiles below the diagonal are skipped, the result stays
    identical to the rectangular product."""
    import torch
    v = syn.normal_matrix(n, k, "bf16", 53)
    tv = torch.from_numpy(v.view(np.int16)).cuda()
    full = nk.dots_packed(tv, nk.dots_pack(tv, "bf16"), dtype="bf16")
    out = torch.full((n, n), -7.0, dtype=torch.float32, device="cuda")
    nk.dots_symmetric(tv, dtype="bf16", out=out)
    assert nk.synchronize() == 0
    upper = torch.triu(torch.ones((n, n), dtype=torch.bool, device="cuda"))
    assert torch.equal(out[upper], full[upper])
    assert bool((out[~upper] == -7.0).all())
    # sliced, starting inside a 256-row block
    out2 = torch.full((n, n), -7.0, dtype=torch.float32, device="cuda")
    nk.angulars_symmetric(tv, dtype="bf16", out=out2, start_row=700, end_row=1333)
    dist = nk.angulars_packed(tv, nk.dots_pack(tv, "bf16"), dtype="bf16")
    assert nk.synchronize() == 0
    mine = torch.zeros((n, n), dtype=torch.bool, device="cuda")
    mine[700:1333] = True
    strict = mine & torch.triu(torch.ones((n, n), dtype=torch.bool, device="cuda"), 1)
    assert torch.equal(out2[strict], dist[strict])
    assert bool((torch.diagonal(out2)[700:1333] == 0).all())
    untouched = ~(mine & upper)
    assert bool((out2[untouched] == -7.0).all())


@pytest.mark.parametrize("dtype,op", [("i8", "dots"), ("u8", "dots"), ("bf16", "dots"), ("f16", "angulars"), ("f32", "euclideans")])
def test_against_the_reference_library(dtype, op):
    """Same call on the reference's dispatched kernels: integers bit for bit, floats within the tolerances of the
    packed tests."""
    ref = oracle.ref()
    if ref is None:
        pytest.skip("reference library was not compiled")
    n, k = 192, 128
    v = _vectors(n, k, dtype, 59)
    ours = _sentinel(n, dtype, op)
    theirs = ours.copy()
    getattr(nk, op + "_symmetric")(v, dtype=dtype, out=ours, start_row=32, end_row=160)
    u64, vp = ctypes.c_uint64, ctypes.c_void_p
    fn = getattr(ref.lib, f"nk_{op}_symmetric_{dtype}")
    fn.restype, fn.argtypes = None, [vp, u64, u64, u64, vp, u64, u64, u64]
    raw = np.ascontiguousarray(v)
    fn(raw.ctypes.data, n, k, raw.strides[0], theirs.ctypes.data, theirs.strides[0], 32, 128)
    mine = np.zeros((n, n), dtype=bool)
    mine[32:160] = True
    mine &= np.triu(np.ones((n, n), dtype=bool))
    # Cells outside the contract: this library leaves them alone (like the reference's scalar kernels); the reference's
    # SIMD back ends also fill the mirrored cells of the rows they own, so those are not compared.
    sentinel = _sentinel(n, dtype, op)
    assert np.array_equal(ours[~mine].view(np.uint8), sentinel[~mine].view(np.uint8))
    if dtype in ("i8", "u8"):
        assert np.array_equal(ours[mine], theirs[mine])
        return
    a, b = ours[mine].astype(np.float64), theirs[mine].astype(np.float64)
    if op == "dots":
        x = np.abs(oracle.decode(v, dtype).astype(np.float64))
        err = np.abs(ours.astype(np.float64) - theirs.astype(np.float64)) / np.maximum(x @ x.T, 1e-30)
        assert err[mine & np.triu(np.ones((n, n), dtype=bool), 1)].max() <= 2 * DOT_TOLERANCE[dtype]
        slices = -(-k * v.itemsize // 32)  # truncating accumulation: up to one ulp per 32-byte slice on the diagonal
        assert np.diag(err)[32:160].max() <= (slices + 2) * 2.0 ** -24
    elif op == "angulars":
        assert np.max(np.abs(a - b)) <= 2 * ANGULAR_ATOL
    else:
        assert np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3)) <= 1e-9


def test_lookup_by_kind_returns_the_symmetric_entry_points():
    for kind, name in (("y", "nk_dots_symmetric_bf16"), ("n", "nk_angulars_symmetric_bf16"), ("D", "nk_euclideans_symmetric_bf16")):
        fn, cap = ctypes.c_void_p(), ctypes.c_uint64()
        nk.lib.nk_find_kernel_punned(ord(kind), nk.DTYPE_CODES["bf16"], ctypes.c_uint64(~0 & (2**64 - 1)), ctypes.byref(fn), ctypes.byref(cap))
        assert cap.value != 0
        assert fn.value == ctypes.cast(getattr(nk.lib, name), ctypes.c_void_p).value
