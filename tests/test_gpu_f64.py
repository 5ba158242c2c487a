"""f64 packed family through the C ABI. The dots must equal the oracle - and with it the reference's scalar kernels, to
which the oracle is pinned - BIT FOR BIT: the CUDA kernel performs the same two-lane Dot2 operations in the same order.
Distances use plain f64 norms (the reference's are Neumaier-compensated), so they agree to a few ulp."""
import numpy as np
import pytest

import numkong_b200 as nk
import oracle

pytestmark = pytest.mark.gpu


def _wide(rows, cols, seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((rows, cols)) * np.exp2(rng.integers(-20, 21, (rows, cols)))


@pytest.mark.parametrize("shape", [(1, 1, 1), (7, 5, 3), (33, 17, 65), (130, 300, 1000), (64, 257, 2049)])
def test_dots_are_bit_identical_to_the_oracle(shape):
    m, n, k = shape
    a, b = _wide(m, k, 1), _wide(n, k, 2)
    c = nk.dots_packed(a, nk.dots_pack(b))
    assert c.dtype == np.float64
    assert np.array_equal(c.view(np.uint64), oracle.dots(a, b, "f64").view(np.uint64))


@pytest.mark.parametrize("op", ["angulars", "euclideans"])
def test_distances(op):
    m, n, k = 70, 190, 300
    a, b = _wide(m, k, 3), _wide(n, k, 4)
    a[3] = 0
    got = getattr(nk, op + "_packed")(a, nk.dots_pack(b))
    want = getattr(oracle, op)(a, b, "f64")
    if op == "angulars":
        assert np.max(np.abs(got - want)) <= 1e-14
    else:
        assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-300)) <= 1e-12


def test_device_operands_strides_and_symmetric():
    import torch
    n, k = 260, 129
    v = _wide(n, k + 3, 5)[:, :k]  # a row stride that is not the row length
    tv = torch.from_numpy(np.ascontiguousarray(v)).cuda()
    full = nk.dots_packed(tv, nk.dots_pack(tv))
    assert nk.synchronize() == 0
    want = oracle.dots(np.ascontiguousarray(v), np.ascontiguousarray(v), "f64")
    assert np.array_equal(full.cpu().numpy().view(np.uint64), want.view(np.uint64))
    host = nk.dots_packed(v, nk.dots_pack(v))  # strided host input
    assert np.array_equal(host.view(np.uint64), want.view(np.uint64))
    out = np.full((n, n), -7.0)
    nk.dots_symmetric(v, out=out, start_row=30, end_row=200)
    mine = np.zeros((n, n), dtype=bool)
    mine[30:200] = True
    mine &= np.triu(np.ones((n, n), dtype=bool))
    assert np.array_equal(out[mine].view(np.uint64), want[mine].view(np.uint64)) and np.all(out[~mine] == -7.0)


def test_against_the_reference_library():
    ref = oracle.ref()
    if ref is None:
        pytest.skip("reference library was not compiled")
    a, b = _wide(64, 777, 6), _wide(96, 777, 7)
    assert np.array_equal(nk.dots_packed(a, nk.dots_pack(b)).view(np.uint64), ref.dots(a, b, "f64").view(np.uint64))
