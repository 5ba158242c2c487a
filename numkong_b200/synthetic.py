"""Seeded synthetic inputs in NumKong's storage formats (NumPy only).

The reference's own tests and benchmarks are fully synthetic (bench/bench.hpp:237-246,
test/test_base.py:437-493); these generators reproduce their shapes and value distributions:
normal or uniform draws rounded to nearest-even into the storage type, or uniform draws over the
finite byte codes of the 8- and 6-bit floats.

Storage conventions: bf16 / f16 as uint16 words, e4m3 / e5m2 as uint8, e2m3 / e3m2 as uint8 holding
0b00SEEMMM / 0b00SEEEMM, i8 as int8, u8 as uint8, f32 as float32.
"""
from __future__ import annotations

import numpy as np

STORAGE = {"i8": np.int8, "u8": np.uint8, "f32": np.float32, "f16": np.uint16, "bf16": np.uint16,
           "e4m3": np.uint8, "e5m2": np.uint8, "e2m3": np.uint8, "e3m2": np.uint8}


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even truncation of f32 to its upper 16 bits (NaN kept quiet)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    return np.where(nan, (u >> np.uint32(16)) | np.uint32(0x40), rounded).astype(np.uint16)


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def _minifloat_table(exp_bits: int, man_bits: int, bias: int, ieee_specials: bool, fn_nan: bool) -> np.ndarray:
    """Non-negative values of every magnitude code (NaN/inf as np.nan/np.inf)."""
    n = 1 << (exp_bits + man_bits)
    vals = np.empty(n, dtype=np.float64)
    for code in range(n):
        e, m = code >> man_bits, code & ((1 << man_bits) - 1)
        if e == 0:
            vals[code] = m / (1 << man_bits) * 2.0 ** (1 - bias)
        else:
            vals[code] = (1 + m / (1 << man_bits)) * 2.0 ** (e - bias)
        if ieee_specials and e == (1 << exp_bits) - 1:
            vals[code] = np.inf if m == 0 else np.nan
        if fn_nan and code == n - 1:
            vals[code] = np.nan
    return vals


_FORMATS = {
    # name: (exp bits, mantissa bits, bias, IEEE inf/NaN, single NaN code, sign bit position)
    "e4m3": (4, 3, 7, False, True, 7),
    "e5m2": (5, 2, 15, True, False, 7),
    "e2m3": (2, 3, 1, False, False, 5),
    "e3m2": (3, 2, 3, False, False, 5),
}


def minifloat_values(name: str) -> np.ndarray:
    """Value of every byte code 0..255 of an 8/6-bit float (codes outside the format's bits alias inside it)."""
    e, m, bias, ieee, fn, sign_bit = _FORMATS[name]
    mags = _minifloat_table(e, m, bias, ieee, fn)
    out = np.empty(256, dtype=np.float64)
    mask = (1 << (e + m)) - 1
    for code in range(256):
        v = mags[code & mask]
        out[code] = -v if (code >> sign_bit) & 1 else v
    return out


def f32_to_minifloat(x: np.ndarray, name: str) -> np.ndarray:
    """Round-to-nearest-even (ties to the even code), saturating to the largest finite value."""
    e, m, bias, ieee, fn, sign_bit = _FORMATS[name]
    mags = _minifloat_table(e, m, bias, ieee, fn)
    finite = np.flatnonzero(np.isfinite(mags))
    grid = mags[finite]                       # ascending, starts at 0
    x = np.asarray(x, dtype=np.float64)
    ax = np.minimum(np.abs(x), grid[-1])
    hi = np.clip(np.searchsorted(grid, ax, side="left"), 0, len(grid) - 1)
    lo = np.clip(hi - 1, 0, len(grid) - 1)
    d_hi, d_lo = np.abs(grid[hi] - ax), np.abs(ax - grid[lo])
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & ((finite[hi] & 1) == 0))
    code = np.where(pick_hi, finite[hi], finite[lo]).astype(np.uint8)
    sign = (np.signbit(x)).astype(np.uint8) << np.uint8(sign_bit)
    return (code | sign).astype(np.uint8)


def encode(x: np.ndarray, dtype: str) -> np.ndarray:
    """f32 values -> storage of `dtype` with round-to-nearest-even (saturating for the mini-floats and integers)."""
    if dtype == "f32":
        return np.ascontiguousarray(x, dtype=np.float32)
    if dtype == "bf16":
        return f32_to_bf16(x)
    if dtype == "f16":
        return f32_to_f16(x)
    if dtype in _FORMATS:
        return f32_to_minifloat(x, dtype)
    if dtype == "i8":
        return np.clip(np.rint(x), -128, 127).astype(np.int8)
    if dtype == "u8":
        return np.clip(np.rint(x), 0, 255).astype(np.uint8)
    raise KeyError(dtype)


def normal_matrix(rows: int, cols: int, dtype: str, seed: int, scale: float = 1.0, normalize: bool = False) -> np.ndarray:
    """N(0, scale^2) entries (optionally L2-normalised rows) rounded into `dtype`. Integers: full-range uniform."""
    rng = np.random.default_rng(seed)
    if dtype == "i8":
        return rng.integers(-128, 128, size=(rows, cols), dtype=np.int8)
    if dtype == "u8":
        return rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(scale)
    if normalize:
        x /= np.maximum(np.linalg.norm(x, axis=1, keepdims=True), 1e-30).astype(np.float32)
    return encode(x, dtype)


def finite_codes_matrix(rows: int, cols: int, dtype: str, seed: int, max_abs: float = 458.0) -> np.ndarray:
    """Uniform draws over the finite byte codes of an 8/6-bit float whose magnitude is at most `max_abs`
    (the reference's Python tests draw fp8/fp6 inputs this way, test/test_base.py:463-465)."""
    vals = minifloat_values(dtype)
    e, m, *_rest, sign_bit = _FORMATS[dtype]
    valid_bits = (1 << (e + m)) - 1 | (1 << sign_bit)
    codes = np.array([c for c in range(256) if (c & ~valid_bits) == 0 and np.isfinite(vals[c]) and abs(vals[c]) <= max_abs],
                     dtype=np.uint8)
    rng = np.random.default_rng(seed)
    return codes[rng.integers(0, len(codes), size=(rows, cols))]


def lognormal_matrix(rows: int, cols: int, dtype: str, seed: int, signed: bool = False) -> np.ndarray:
    """Log-normal(0, 0.5) entries. `signed=True` gives each a random sign, which is what the reference's C++ precision
    tests draw for signed element types (include/numkong/random.hpp:130-146, default of test/test.hpp:536-549); the
    all-positive form is the harder case for a truncating accumulator and is kept as the default."""
    rng = np.random.default_rng(seed)
    x = rng.lognormal(0.0, 0.5, size=(rows, cols)).astype(np.float32)
    if signed and dtype != "u8":
        x *= rng.choice(np.array([1.0, -1.0], dtype=np.float32), size=(rows, cols))
    if dtype in ("i8", "u8"):
        x = np.clip(x * 16, -127, 127)
    return encode(x, dtype)


# Values every float source of a conversion test starts with: zeros, rounding ties of the integer targets, the largest
# values and rounding ties of the small float formats, a binary16 underflow tie, an f32 subnormal, large magnitudes.
_CAST_SPECIALS = [0.0, -0.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.5, -128.5, 254.5, 255.5, 448.0, 464.0, 480.0, -464.0,
                  57344.0, 61440.0, 61439.0, 7.5, 7.75, 7.25, 28.0, 30.0, 26.0, 65504.0, 65520.0, 65519.0, 2.0 ** -25, 2.0 ** -24 * 1.5,
                  1e-40, 0.0009765625, 0.001953125 * 1.5, 3e9, -3e9, 1e30, -1e30, 32767.5, -32768.5, 65535.5, 15.9, -8.9, 0.9]


def cast_samples(dtype: str, n: int, seed: int) -> np.ndarray:
    """Storage of `n` finite values of `dtype` for conversion tests: floats spread over forty binades behind the list of
    special cases above, 16-bit and smaller floats as uniformly random finite codes, integers half full-range and half
    small, sub-byte types as random bytes."""
    rng = np.random.default_rng(seed)
    if dtype in ("f64", "f32"):
        v = rng.standard_normal(n) * np.exp2(rng.integers(-20, 20, n))
        k = min(n, len(_CAST_SPECIALS))
        v[:k] = _CAST_SPECIALS[:k]
        return v if dtype == "f64" else v.astype(np.float32)
    if dtype in ("f16", "bf16"):
        v = rng.integers(0, 65536, n).astype(np.uint16)
        all_ones = 0x7C00 if dtype == "f16" else 0x7F80
        v[(v & all_ones) == all_ones] &= np.uint16(0xBFFF)   # clear one exponent bit of infinities and NaN
        return v
    if dtype in ("e4m3", "e5m2", "e2m3", "e3m2"):
        return finite_codes_matrix(1, n, dtype, seed, max_abs=1e9).ravel()
    if dtype in ("i4", "u4", "u1"):
        return rng.integers(0, 256, (n * (1 if dtype == "u1" else 4) + 7) // 8).astype(np.uint8)
    storage = {"i8": np.int8, "u8": np.uint8, "i16": np.int16, "u16": np.uint16, "i32": np.int32, "u32": np.uint32,
               "i64": np.int64, "u64": np.uint64}[dtype]
    info = np.iinfo(storage)
    v = rng.integers(info.min, info.max, n, dtype=storage, endpoint=True)
    v[: n // 2] = rng.integers(max(info.min, -300), min(info.max, 300), n // 2).astype(storage)
    return v


def moments_samples(dtype: str, n: int, seed: int) -> np.ndarray:
    """`cast_samples` with magnitudes bounded so that sums of squares stay finite in the result type: f32 / f64 clipped to
    +-1e6, bf16 kept below 2 (top exponent bit cleared)."""
    x = cast_samples(dtype, n, seed)
    if dtype in ("f64", "f32"):
        return np.clip(x, -1e6, 1e6).astype(x.dtype)
    if dtype == "bf16":
        return x & np.uint16(0xBFFF)
    return x
