"""Pins the CPU oracle (oracle/nk_oracle.c) to the reference: against golden vectors produced by the
reference's own kernels (tests/golden/packed_path.npz, generator committed beside it), against the
known-answer tests of the reference's binding suites, and - when the reference has been compiled into
oracle/_ref/ - against the reference itself on fresh seeded inputs. No GPU involved."""
import os

import numpy as np
import pytest

import oracle
from numkong_b200 import synthetic as syn
from tests._common import ALL_DTYPES, MINIFLOATS, make_matrix, ones_matrix

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "packed_path.npz"))
GOLDEN_SHAPES = [(7, 5, 3), (33, 17, 65), (16, 24, 128), (5, 9, 1031)]


def _bits_equal(x, y):
    return x.shape == y.shape and np.array_equal(np.ascontiguousarray(x).view(np.uint8), np.ascontiguousarray(y).view(np.uint8))


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("shape", GOLDEN_SHAPES)
def test_oracle_matches_reference_serial_golden_bit_for_bit(dtype, shape):
    m, n, k = shape
    key = f"{dtype}_{m}x{n}x{k}"
    a, b = GOLDEN[key + "_a"], GOLDEN[key + "_b"]
    assert _bits_equal(oracle.dots(a, b, dtype), GOLDEN[key + "_dots_serial"])
    assert _bits_equal(oracle.angulars(a, b, dtype), GOLDEN[key + "_angulars_serial"])
    assert _bits_equal(oracle.euclideans(a, b, dtype), GOLDEN[key + "_euclideans_serial"])


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_oracle_within_envelope_of_reference_dispatched_backend(dtype):
    """The reference's SIMD/AMX back ends differ from its scalar one only by summation order."""
    for (m, n, k) in GOLDEN_SHAPES:
        key = f"{dtype}_{m}x{n}x{k}"
        a, b = GOLDEN[key + "_a"], GOLDEN[key + "_b"]
        got, ref = oracle.dots(a, b, dtype).astype(np.float64), GOLDEN[key + "_dots_dispatch"].astype(np.float64)
        if dtype in ("i8", "u8"):
            assert np.array_equal(got, ref)
        else:
            scale = np.abs(oracle.decode(a, dtype)).astype(np.float64) @ np.abs(oracle.decode(b, dtype)).astype(np.float64).T
            assert np.max(np.abs(got - ref) / np.maximum(scale, 1e-30)) < 5e-7  # the spread between the reference's own back ends
        assert np.nanmax(np.abs(oracle.angulars(a, b, dtype) - GOLDEN[key + "_angulars_dispatch"])) < 1e-6


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_maxsim_oracles_against_golden(dtype):
    for (nq, nd, k) in [(32, 180, 128), (8, 64, 64), (5, 3, 17)]:
        key = f"maxsim_{dtype}_{nq}x{nd}x{k}"
        q, d = GOLDEN[key + "_q"], GOLDEN[key + "_d"]
        serial, dispatch = float(GOLDEN[key + "_serial"]), float(GOLDEN[key + "_dispatch"])
        # The scalar back end (i8 screening): winners are reproduced exactly, the sum to f32 rounding noise
        # (the reference refines with a run-time dispatched dot).
        assert abs(oracle.maxsim_coarse_i8(q, d, dtype) - serial) <= 2e-6 * max(1.0, abs(serial))
        # Fused semantics (first argmax of the raw dot): never better than the exhaustive minimum beyond rounding.
        fused, exhaustive = oracle.maxsim(q, d, dtype), oracle.maxsim_exhaustive(q, d, dtype)
        assert fused >= exhaustive - 1e-4
        if dtype == "bf16":
            # The fixture was generated on a CPU whose dispatched bf16 MaxSim is the reference's fused
            # tensor-engine back end (maxsim/sapphireamx.h:716-861): same winners, sum within f32 rounding.
            assert abs(fused - dispatch) <= 2e-5 * max(1.0, abs(dispatch))


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 8, 3), (3, 1, 7), (7, 5, 3), (33, 17, 65)])
def test_all_ones_known_answers(dtype, shape):
    """rust/matrix.rs:4610-4773 of the reference: all-ones inputs give dots == depth, distances == 0."""
    h, w, k = shape
    a, b = ones_matrix(h, k, dtype), ones_matrix(w, k, dtype)
    assert np.all(oracle.dots(a, b, dtype) == k)
    assert np.all(oracle.angulars(a, b, dtype) <= 2e-7)
    assert np.all(oracle.euclideans(a, b, dtype) <= 1e-3 * np.sqrt(k) * 1e-3 + 1e-6)


def test_tiny_integer_and_identity_known_answers():
    """golang/unit_test.go:558-652 (2x3 integer matrices) and test/test.mjs:167-200 (identity-row B)."""
    a = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.int8)
    b = np.array([[7, 8, 9], [10, 11, 12]], dtype=np.int8)
    assert np.array_equal(oracle.dots(a, b, "i8"), np.array([[50, 68], [122, 167]], dtype=np.int32))
    a = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9], [10, 11, 12]], dtype=np.float32)
    b = np.array([[1, 0, 0], [0, 1, 0], [0, 0, 1], [1, 1, 0], [1, 1, 1]], dtype=np.float32)
    expect = np.array([[1, 2, 3, 3, 6], [4, 5, 6, 9, 15], [7, 8, 9, 15, 24], [10, 11, 12, 21, 33]], dtype=np.float64)
    assert np.array_equal(oracle.dots(a, b, "f32"), expect)


def test_maxsim_of_identical_sides_is_zero():
    """test/test_maxsim.py:169-175 of the reference."""
    x = np.ones((8, 64), dtype=np.float32)
    assert abs(oracle.maxsim(x, x, "f32")) < 1e-6
    assert abs(oracle.maxsim_coarse_i8(x, x, "f32")) < 1e-6


def test_zero_norm_rule_and_clamps():
    """include/numkong/spatial/serial.h:261-267: zero norm product -> 0 if the dot is 0 else 1; results >= 0."""
    a = np.zeros((2, 8), dtype=np.float32)
    b = np.zeros((3, 8), dtype=np.float32)
    b[1, 0] = 2.0
    assert np.array_equal(oracle.angulars(a, b, "f32"), np.zeros((2, 3)))
    assert np.array_equal(oracle.euclideans(a, b, "f32")[:, 1], np.array([2.0, 2.0]))
    x = syn.normal_matrix(9, 33, "bf16", 3)
    assert np.all(oracle.angulars(x, x, "bf16") >= 0)
    assert np.all(np.diag(oracle.euclideans(x, x, "bf16")) < 1e-2)


needs_ref = pytest.mark.skipif(oracle.ref_serial() is None or oracle.ref() is None,
                               reason="reference not compiled (make -C oracle ref)")


@needs_ref
@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_oracle_against_live_reference_on_fresh_inputs(dtype):
    serial = oracle.ref_serial()
    for seed, (m, n, k) in enumerate([(9, 11, 40), (4, 6, 515), (31, 8, 96)]):
        kind = "codes" if dtype in MINIFLOATS and seed % 2 else "normal"
        a, b = make_matrix(m, k, dtype, 7000 + seed, kind), make_matrix(n, k, dtype, 7100 + seed, kind)
        assert _bits_equal(oracle.dots(a, b, dtype), serial.dots(a, b, dtype))
        assert _bits_equal(oracle.angulars(a, b, dtype), serial.angulars(a, b, dtype))
        assert _bits_equal(oracle.euclideans(a, b, dtype), serial.euclideans(a, b, dtype))


@needs_ref
def test_decoders_and_encoders_against_reference_cast():
    import ctypes
    ref = oracle.ref()
    ref.lib.nk_cast.restype = None
    ref.lib.nk_cast.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int]
    x = (np.random.default_rng(0).standard_normal(20000) * 4).astype(np.float32)
    for dt in MINIFLOATS:
        codes = np.arange(64 if dt in ("e2m3", "e3m2") else 256, dtype=np.uint8)
        out = np.zeros(len(codes), dtype=np.float32)
        ref.lib.nk_cast(codes.ctypes.data, oracle.CODES[dt], len(codes), out.ctypes.data, oracle.CODES["f32"])
        mine = oracle.decode(codes.reshape(1, -1), dt).ravel()
        assert np.array_equal(np.isnan(out), np.isnan(mine))
        assert np.array_equal(out[~np.isnan(out)], mine[~np.isnan(mine)])
        table = syn.minifloat_values(dt)[:len(codes)].astype(np.float32)
        assert np.array_equal(np.nan_to_num(table, nan=-1.0), np.nan_to_num(out, nan=-1.0))
        enc = np.zeros(len(x), dtype=np.uint8)
        ref.lib.nk_cast(x.ctypes.data, oracle.CODES["f32"], len(x), enc.ctypes.data, oracle.CODES[dt])
        assert np.array_equal(enc, syn.encode(x, dt))
    for dt in ("bf16", "f16"):
        enc = np.zeros(len(x), dtype=np.uint16)
        ref.lib.nk_cast(x.ctypes.data, oracle.CODES["f32"], len(x), enc.ctypes.data, oracle.CODES[dt])
        assert np.array_equal(enc, syn.encode(x, dt))


NIBBLE_GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "nibble_path.npz"))


@pytest.mark.parametrize("dtype", ["i4", "u4"])
@pytest.mark.parametrize("shape", GOLDEN_SHAPES)
def test_four_bit_oracle_matches_reference_golden(dtype, shape):
    """4-bit types (two values per byte, depth counted in values, odd depths included): bit for bit against the
    reference's scalar kernels; its dispatched back end agrees exactly on the dots and to an ulp on the distances."""
    m, n, k = shape
    key = f"{dtype}_{m}x{n}x{k}"
    a, b = NIBBLE_GOLDEN[key + "_a"], NIBBLE_GOLDEN[key + "_b"]
    for op in ("dots", "angulars", "euclideans"):
        assert _bits_equal(getattr(oracle, op)(a, b, dtype, depth=k), NIBBLE_GOLDEN[f"{key}_{op}_serial"])
    assert _bits_equal(oracle.dots(a, b, dtype, depth=k), NIBBLE_GOLDEN[key + "_dots_dispatch"])
    if k % 2 == 0 and dtype == "u4":
        # Signed nibbles: the reference's dispatched back end on this CPU returns distances that do not follow from its own
        # dots and scalar norms (e.g. 0.929 where dot 757 and squared norms 2457, 2422 give 0.690), so i4 distances are
        # pinned to the scalar kernels only. At odd depths the reference's back ends disagree with each other about the second nibble of the last byte in the
        # NORMS (its SIMD moments stop at `depth`, its dots and its scalar moments take the whole byte); the oracle and the
        # CUDA path follow the scalar kernels, so only even depths are compared with the dispatched distances.
        assert np.max(np.abs(oracle.angulars(a, b, dtype, depth=k) - NIBBLE_GOLDEN[key + "_angulars_dispatch"])) < 1e-6


@pytest.mark.parametrize("dtype", ["i4", "u4"])
def test_four_bit_oracle_against_live_reference(dtype):
    serial = oracle.ref_serial()
    if serial is None:
        pytest.skip("reference library was not compiled")
    rng = np.random.default_rng(77)
    for depth in (1, 2, 15, 64, 333):
        a = rng.integers(0, 256, (6, (depth + 1) // 2), dtype=np.uint8)
        b = rng.integers(0, 256, (9, (depth + 1) // 2), dtype=np.uint8)
        for op in ("dots", "angulars", "euclideans"):
            assert _bits_equal(getattr(oracle, op)(a, b, dtype, depth=depth), getattr(serial, op)(a, b, dtype, depth=depth))
    # an all-sevens row against itself: the dot is depth * 49 (both nibbles of the last byte count, so odd depths round up)
    ones = np.full((1, 4), 0x77, dtype=np.uint8)
    assert oracle.dots(ones, ones, dtype, depth=7)[0, 0] == 8 * 49


@pytest.mark.parametrize("shape", GOLDEN_SHAPES)
def test_one_bit_oracle_matches_reference_golden(shape):
    """Bit vectors: AND-popcount dots, Hamming and Jaccard distances, bit for bit against the reference's scalar kernels;
    its dispatched back end agrees exactly on the integer results and to rounding on the Jaccard division."""
    m, n, k = shape
    key = f"u1_{m}x{n}x{k}"
    a, b = NIBBLE_GOLDEN[key + "_a"], NIBBLE_GOLDEN[key + "_b"]
    for op in ("dots", "hammings", "jaccards"):
        assert _bits_equal(getattr(oracle, op)(a, b, "u1", depth=k), NIBBLE_GOLDEN[f"{key}_{op}_serial"])
    assert _bits_equal(oracle.dots(a, b, "u1", depth=k), NIBBLE_GOLDEN[key + "_dots_dispatch"])
    assert _bits_equal(oracle.hammings(a, b, depth=k), NIBBLE_GOLDEN[key + "_hammings_dispatch"])
    assert np.max(np.abs(oracle.jaccards(a, b, depth=k) - NIBBLE_GOLDEN[key + "_jaccards_dispatch"])) < 1e-6


def test_one_bit_known_answers():
    a = np.array([[0b10110000, 0b00000001]], dtype=np.uint8)   # 4 bits set
    b = np.array([[0b10010000, 0b00000001], [0, 0]], dtype=np.uint8)  # 3 bits set, all shared; the empty set
    assert oracle.dots(a, b, "u1").tolist() == [[3, 0]]
    assert oracle.hammings(a, b).tolist() == [[1, 4]]
    assert np.allclose(oracle.jaccards(a, b), [[1 - 3 / 4, 1.0]])
    assert oracle.jaccards(b[1:], b[1:])[0, 0] == 0.0  # two empty sets


@pytest.mark.parametrize("shape", GOLDEN_SHAPES)
def test_f64_oracle_matches_reference_golden(shape):
    """f64: two-lane Dot2 accumulation restated operation by operation - bit for bit against the reference's scalar kernels
    (dots, angular, Euclidean) and against its dispatched back end on the dots."""
    m, n, k = shape
    key = f"f64_{m}x{n}x{k}"
    a, b = NIBBLE_GOLDEN[key + "_a"], NIBBLE_GOLDEN[key + "_b"]
    for op in ("dots", "angulars", "euclideans"):
        assert _bits_equal(getattr(oracle, op)(a, b, "f64"), NIBBLE_GOLDEN[f"{key}_{op}_serial"])
    assert _bits_equal(oracle.dots(a, b, "f64"), NIBBLE_GOLDEN[key + "_dots_dispatch"])
    # Dot2 is worth having: on these inputs a plain f64 loop is measurably further from the exact value
    exact = np.array([[float(sum(__import__("fractions").Fraction(x) * __import__("fractions").Fraction(y) for x, y in zip(r, c)))
                       for c in b[:3]] for r in a[:3]])
    assert np.max(np.abs(oracle.dots(a, b, "f64")[:3, :3] - exact)) <= np.max(np.abs((a @ b.T)[:3, :3] - exact))


COMPACT_GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "compact_path.npz"))


@pytest.mark.parametrize("shape", GOLDEN_SHAPES)
def test_compact_oracle_matches_reference_golden(shape):
    """In-place down-casts of a dots matrix (f32 -> bf16, i32 -> i8 rescaled by the norms): bit for bit against the
    reference's scalar helpers, padded rows, zero vectors, a cosine-1 pair and a rounding tie included."""
    m, n, k = shape
    for dt in ("i8", "bf16"):
        key = f"{dt}_{m}x{n}x{k}"
        c = COMPACT_GOLDEN[key + "_c"][:, :n]
        assert c.strides[0] == (n + int(COMPACT_GOLDEN[key + "_pad"])) * 4
        got = oracle.dots_compact(c, COMPACT_GOLDEN[key + "_an"], COMPACT_GOLDEN[key + "_bn"]) if dt == "i8" else oracle.dots_compact(c)
        assert np.array_equal(got, COMPACT_GOLDEN[key + "_compact_serial"])
    # the cosine-1 pair: 127, or 126 where the approximate reciprocal square roots leave the product just below 127
    assert COMPACT_GOLDEN[f"i8_{m}x{n}x{k}_compact_serial"][0, 0] in (126, 127)


def test_compact_oracle_against_live_reference():
    serial = oracle.ref_serial()
    if serial is None:
        pytest.skip("reference not compiled here")
    rng = np.random.default_rng(11)
    a, b = rng.integers(-128, 128, (40, 96), dtype=np.int8), rng.integers(-128, 128, (70, 96), dtype=np.int8)
    c = a.astype(np.int32) @ b.astype(np.int32).T
    an, bn = (a.astype(np.int32) ** 2).sum(1).astype(np.int32), (b.astype(np.int32) ** 2).sum(1).astype(np.int32)
    assert np.array_equal(oracle.dots_compact(c, an, bn), serial.dots_compact(c, an, bn))
    f = (rng.standard_normal((40, 70)) * 1e4).astype(np.float32)
    assert np.array_equal(oracle.dots_compact(f), serial.dots_compact(f))


CAST_GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "cast_path.npz"))
CAST_TYPES = ["f64", "f32", "f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2", "i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "i4", "u4", "u1"]


def cast_pair_defined(a, b):
    signed = ("i8", "i16", "i32", "i64", "i4")
    return not ((a == "u1" and b in signed) or (a in signed and b in ("u4", "u1")))


@pytest.mark.parametrize("source", CAST_TYPES)
def test_cast_oracle_matches_reference_golden(source):
    """Bulk conversion from `source` to every other type: byte for byte against the reference's scalar back end."""
    x = CAST_GOLDEN["from_" + source]
    for target in CAST_TYPES:
        if target == source or not cast_pair_defined(source, target):
            continue
        got = oracle.cast(x, source, target, 136)
        assert np.array_equal(got.view(np.uint8), CAST_GOLDEN[f"{source}_to_{target}"].view(np.uint8)), (source, target)


def test_cast_oracle_against_live_reference():
    """Fresh samples, tails included, against the scalar back end; the dispatched back end agrees except where it breaks its
    own scalar rules (f32/f16/bf16 -> e5m2 overflow gives NaN codes there, negative integers -> u64 wrap around)."""
    serial, dispatch = oracle.ref_serial(), oracle.ref()
    if serial is None or dispatch is None:
        pytest.skip("reference not compiled here")
    for si, a in enumerate(CAST_TYPES):
        for n in (1000, 1003):
            if n % 8 and oracle.CAST_BITS[a] < 8:
                continue                                     # the reference reads and writes whole sub-byte batches
            x = syn.cast_samples(a, n, 7000 + si)
            for b in CAST_TYPES:
                if a == b or not cast_pair_defined(a, b) or (n % 8 and oracle.CAST_BITS[b] < 8):
                    continue
                if b in ("i64", "u64") and a in ("f64", "f32", "bf16"):
                    continue                                 # |x| >= 2^63: the reference leaves the result to the C cast
                got = oracle.cast(x, a, b, n).view(np.uint8)
                assert np.array_equal(got, serial.cast(x, a, b, n).view(np.uint8)), (a, b, n)
                if b == "e5m2" or (b == "u64" and a in ("i8", "i16", "i32", "i64")):
                    continue
                assert np.array_equal(got, dispatch.cast(x, a, b, n).view(np.uint8)), (a, b, n, "dispatch")


MOMENTS_GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "moments_path.npz"))


def _same_bits(pair, key):
    return all(np.array(v).tobytes() == MOMENTS_GOLDEN[f"{key}_{name}"].tobytes() for v, name in zip(pair, ("sum", "sumsq")))


@pytest.mark.parametrize("dtype", CAST_TYPES)
def test_moments_oracle_matches_reference_golden(dtype):
    """Sum and sum of squares: bit for bit against the reference's scalar reductions (compensated serial sums for the
    floats, exact and saturating integer rules), contiguous and strided."""
    x = MOMENTS_GOLDEN["from_" + dtype]
    per_unit = 8 // oracle.CAST_BITS[dtype] if oracle.CAST_BITS[dtype] < 8 else 1
    assert _same_bits(oracle.moments(x, dtype, 1000 if per_unit > 1 else None), dtype + "_all")
    strided = oracle.moments(x, dtype, 333 if per_unit == 1 else 40 * per_unit, 3 * max(oracle.CAST_BITS[dtype] // 8, 1))
    assert _same_bits(strided, dtype + "_strided")


def test_moments_oracle_saturation_cases():
    for key in ("i32", "u32", "i64", "u64", "i64_negative"):
        assert _same_bits(oracle.moments(MOMENTS_GOLDEN["big_" + key], key.split("_")[0]), "big_" + key), key


def test_moments_oracle_against_live_reference():
    serial = oracle.ref_serial()
    if serial is None:
        pytest.skip("reference not compiled here")
    for si, t in enumerate(CAST_TYPES):
        for n in (1, 9, 2500):
            x = syn.moments_samples(t, n, 9500 + si)
            count = n if oracle.CAST_BITS[t] < 8 else None
            mine, theirs = oracle.moments(x, t, count), serial.moments(x, t, count)
            assert all(np.array(a).tobytes() == np.array(b).tobytes() for a, b in zip(mine, theirs)), (t, n)
