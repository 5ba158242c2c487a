"""Edge cases of the later additions: padded result matrices and tiny inputs of the symmetric family, sub-byte operands on
the row-pipelined host path, wide-store (short depth) products with ragged shapes and strides."""
import numpy as np
import pytest

import numkong_b200 as nk
import oracle
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 2, 31, 257])
def test_symmetric_tiny_and_padded_result(n):
    v = np.random.default_rng(n).integers(-128, 128, (n, 40), dtype=np.int8)
    wide = np.full((n, n + 5), -3, dtype=np.int32)           # result rows are longer than the matrix
    out = wide[:, :n]
    nk.dots_symmetric(v, out=out)
    want = oracle.dots(v, v, "i8")
    upper = np.triu(np.ones((n, n), dtype=bool))
    assert np.array_equal(out[upper], want[upper])
    assert np.all(out[~upper] == -3) and np.all(wide[:, n:] == -3)


@pytest.mark.parametrize("dtype,per", [("i4", 2), ("u4", 2), ("u1", 8)])
def test_sub_byte_operands_on_the_pipelined_host_path(dtype, per):
    m, n, k = 4500, 300, 1024                                  # m >= 2048 host rows: uploaded and multiplied block by block
    rng = np.random.default_rng(3)
    a = rng.integers(0, 256, (m, k // per), dtype=np.uint8)
    b = rng.integers(0, 256, (n, k // per), dtype=np.uint8)
    c = nk.dots_packed(a, nk.dots_pack(b, dtype), dtype=dtype)
    rows = rng.integers(0, m, 64)
    assert np.array_equal(c[rows], oracle.dots(a[rows], b, dtype))
    assert np.array_equal(c[-3:], oracle.dots(a[-3:], b, dtype))


@pytest.mark.parametrize("dtype", ["bf16", "i8", "e5m2"])
@pytest.mark.parametrize("k", [1, 64, 200, 256])
def test_short_depth_products_with_ragged_shapes(dtype, k):
    """Depths of at most 512 bytes per row take the three-stage kernel with 64-column staged stores."""
    m, n = 300, 1000
    a, b = syn.normal_matrix(m, k, dtype, 5), syn.normal_matrix(n, k, dtype, 6)
    wide = np.zeros((m, n + 3), dtype=np.int32 if dtype == "i8" else np.float32)
    out = wide[:, 1:n + 1]                                     # rows start 4 bytes off a 16-byte boundary
    nk.dots_packed(a, nk.dots_pack(b, dtype), out=out, dtype=dtype)
    want = oracle.dots(a, b, dtype)
    if dtype == "i8":
        assert np.array_equal(out, want)
    else:
        exact = oracle.exact_dots_f64(a, b, dtype)
        scale = np.abs(oracle.decode(a, dtype).astype(np.float64)) @ np.abs(oracle.decode(b, dtype).astype(np.float64)).T
        assert np.max(np.abs(out - exact) / np.maximum(scale, 1e-30)) <= 2.5e-7
    assert np.all(wide[:, 0] == 0) and np.all(wide[:, n + 1:] == 0)
    import torch
    ta, tb = torch.from_numpy(a.view(np.int16) if dtype == "bf16" else a).cuda(), torch.from_numpy(b.view(np.int16) if dtype == "bf16" else b).cuda()
    for op in ("angulars", "euclideans"):
        got = getattr(nk, op + "_packed")(ta, nk.dots_pack(tb, dtype), dtype=dtype)
        assert nk.synchronize() == 0
        ref = getattr(oracle, op)(a, b, dtype)
        if op == "angulars":
            assert np.max(np.abs(got.cpu().numpy() - ref)) <= 5e-7
        else:
            assert np.max(np.abs(got.cpu().numpy() - ref) / np.maximum(np.abs(ref), 1e-3)) <= 4e-6


def test_accumulation_span_trades_speed_for_accuracy():
    """Same-sign bf16 data at depth 4096 (the worst case of the truncating tensor-core accumulate): shorter spans bring the
    error down, and the default span (4 stages at this depth) sits at the level of the reference's own scalar kernel
    (1.85 units in the last place on these inputs)."""
    a, b = syn.lognormal_matrix(256, 4096, "bf16", 1), syn.lognormal_matrix(512, 4096, "bf16", 2)
    exact = oracle.exact_dots_f64(a, b, "bf16")
    nearest = exact.astype(np.float32)
    ulp = np.spacing(np.abs(nearest)).astype(np.float64)
    packed = nk.dots_pack(b, "bf16")
    errors = {}
    try:
        for stages in (0, 16, 8, 4):
            nk.set_accumulation_span(stages)
            c = nk.dots_packed(a, packed, dtype="bf16")
            errors[stages] = float(np.mean(np.abs(c.astype(np.float64) - nearest.astype(np.float64)) / ulp))
    finally:
        nk.set_accumulation_span(0)
    assert errors[4] < errors[8] < errors[16]
    assert errors[0] == errors[4]            # sqrt(4096) / 16 = 4 stages is the default for bf16 at this depth
    assert errors[4] <= 2.3 and errors[16] <= 25.0


@pytest.mark.parametrize("dtype,limit", [("f16", 32), ("bf16", 256), ("e4m3", 4), ("e5m2", 4), ("e2m3", 4), ("e3m2", 4)])
def test_reference_acceptance_thresholds_at_its_default_test_shape(dtype, limit):
    """The reference's own test harness accepts a dots kernel when, on all-positive log-normal inputs at 1024 x 128 x 1536, no
    cell is further than 32 (f16), 256 (bf16) or 4 (everything else) units in the last place from the exactly computed result
    rounded to f32 (test/test.hpp:192-230, :207-219, :478-486). The same gate, applied to this library."""
    a, b = syn.lognormal_matrix(1024, 1536, dtype, 42), syn.lognormal_matrix(128, 1536, dtype, 43)
    c = nk.dots_packed(a, nk.dots_pack(b, dtype), dtype=dtype)
    nearest = oracle.exact_dots_f64(a, b, dtype).astype(np.float32)
    ulps = np.abs(c.view(np.int32).astype(np.int64) - nearest.view(np.int32).astype(np.int64))   # same sign: bit patterns are ordered
    assert int(ulps.max()) <= limit, (dtype, int(ulps.max()), float(ulps.mean()))


@pytest.mark.parametrize("dtype", ["bf16", "f16", "i8", "e4m3", "e2m3"])
def test_cta_pair_kernel_at_mid_depth_with_ragged_edges(dtype):
    """4000 x 5100 x 1000: enough 256 x 256 tiles for the CTA-pair kernel (chosen from 8 stages of depth on), none of the
    three extents a multiple of its tile. Sampled rows (the last, partial row tile included) against the oracle."""
    m, n, k = 4000, 5100, 1000
    a, b = syn.normal_matrix(m, k, dtype, 21), syn.normal_matrix(n, k, dtype, 22)
    ta, tb = (torch_from(a), torch_from(b))
    packed = nk.dots_pack(tb, dtype)
    rows = np.r_[0:3, 127:130, 2047:2050, m - 40:m]
    for op in ("dots", "angulars", "euclideans"):
        got = getattr(nk, op + "_packed")(ta, packed, dtype=dtype)
        assert nk.synchronize() == 0
        got = got.cpu().numpy()[rows]
        want = getattr(oracle, op)(a[rows], b, dtype)
        if op == "dots" and dtype == "i8":
            assert np.array_equal(got, want)
        elif op == "dots":
            exact = oracle.exact_dots_f64(a[rows], b, dtype)
            scale = np.abs(oracle.decode(a[rows], dtype).astype(np.float64)) @ np.abs(oracle.decode(b, dtype).astype(np.float64)).T
            assert np.max(np.abs(got - exact) / scale) <= 2.5e-7
        elif op == "angulars":
            assert np.max(np.abs(got - want)) <= 5e-7
        else:
            assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= 4e-6


def torch_from(x):
    import torch
    return torch.from_numpy(x.view(np.int16) if x.dtype == np.uint16 else x).cuda()
