"""Generates the fixtures under tests/golden/ (packed_path, nibble_path, compact_path, cast_path, moments_path) from the
REFERENCE ITSELF.

Run in a container that has the NumKong source tree (where `make -C oracle ref` looks for it; REF=... overrides):

    make -C oracle ref            # compiles the reference's own sources into oracle/_ref/
    python tests/golden/make_golden.py

For every dtype of the packed-contraction path it draws seeded inputs (numkong_b200.synthetic), runs the
reference's scalar back end (nk_*_serial, bit-reproducible) and its dispatched best back end on this CPU,
and stores inputs and outputs. tests/test_oracle_pins.py then checks oracle/nk_oracle.c against these
vectors anywhere, without the reference tree.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from numkong_b200 import synthetic as syn  # noqa: E402

SHAPES = [(7, 5, 3), (33, 17, 65), (16, 24, 128), (5, 9, 1031)]
DTYPES = ["i8", "u8", "bf16", "f16", "e4m3", "e5m2", "e2m3", "e3m2", "f32"]


def main():
    serial, dispatch = oracle.ref_serial(), oracle.ref()
    if serial is None or dispatch is None:
        raise SystemExit("compile the reference first: make -C oracle ref")
    out = {}
    for dt in DTYPES:
        for si, (m, n, k) in enumerate(SHAPES):
            kind_seed = 100 * DTYPES.index(dt) + si
            if dt in ("e4m3", "e5m2", "e2m3", "e3m2") and si % 2:
                a, b = syn.finite_codes_matrix(m, k, dt, kind_seed), syn.finite_codes_matrix(n, k, dt, kind_seed + 50)
            else:
                a, b = syn.normal_matrix(m, k, dt, kind_seed), syn.normal_matrix(n, k, dt, kind_seed + 50)
            key = f"{dt}_{m}x{n}x{k}"
            out[key + "_a"], out[key + "_b"] = a, b
            for op in ("dots", "angulars", "euclideans"):
                out[f"{key}_{op}_serial"] = getattr(serial, op)(a, b, dt)
                out[f"{key}_{op}_dispatch"] = getattr(dispatch, op)(a, b, dt)
    for dt in ("bf16", "f16", "f32"):
        for si, (nq, nd, k) in enumerate([(32, 180, 128), (8, 64, 64), (5, 3, 17)]):
            q, d = syn.normal_matrix(nq, k, dt, 900 + si), syn.normal_matrix(nd, k, dt, 950 + si)
            key = f"maxsim_{dt}_{nq}x{nd}x{k}"
            out[key + "_q"], out[key + "_d"] = q, d
            out[key + "_serial"] = np.float64(serial.maxsim(q, d, dt))
            out[key + "_dispatch"] = np.float64(dispatch.maxsim(q, d, dt))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "packed_path.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")
    # Types added after the first nine (file nibble_path.npz): sub-byte integers, bit vectors, f64. 4-bit types: uniformly random bytes (every nibble value), depths counted in values - odd ones included, where the
    # reference lets the second nibble of the last byte take part.
    out = {}
    for dt in ("i4", "u4"):
        for si, (m, n, k) in enumerate(SHAPES):
            rng = np.random.default_rng(2000 + 10 * ("i4", "u4").index(dt) + si)
            a = rng.integers(0, 256, (m, (k + 1) // 2), dtype=np.uint8)
            b = rng.integers(0, 256, (n, (k + 1) // 2), dtype=np.uint8)
            key = f"{dt}_{m}x{n}x{k}"
            out[key + "_a"], out[key + "_b"] = a, b
            for op in ("dots", "angulars", "euclideans"):
                out[f"{key}_{op}_serial"] = getattr(serial, op)(a, b, dt, depth=k)
                out[f"{key}_{op}_dispatch"] = getattr(dispatch, op)(a, b, dt, depth=k)
    # One-bit vectors: depth counted in bits (every bit of the last byte takes part), AND-popcount dots and set distances.
    for si, (m, n, k) in enumerate(SHAPES):
        rng = np.random.default_rng(3000 + si)
        a = rng.integers(0, 256, (m, (k + 7) // 8), dtype=np.uint8)
        b = rng.integers(0, 256, (n, (k + 7) // 8), dtype=np.uint8)
        key = f"u1_{m}x{n}x{k}"
        out[key + "_a"], out[key + "_b"] = a, b
        for op in ("dots", "hammings", "jaccards"):
            out[f"{key}_{op}_serial"] = getattr(serial, op)(a, b, "u1", depth=k)
            out[f"{key}_{op}_dispatch"] = getattr(dispatch, op)(a, b, "u1", depth=k)
    # f64: N(0,1) values spread over forty binades, so that the compensated (Dot2) accumulation matters.
    for si, (m, n, k) in enumerate(SHAPES):
        rng = np.random.default_rng(4000 + si)
        a = rng.standard_normal((m, k)) * np.exp2(rng.integers(-20, 21, (m, k)))
        b = rng.standard_normal((n, k)) * np.exp2(rng.integers(-20, 21, (n, k)))
        key = f"f64_{m}x{n}x{k}"
        out[key + "_a"], out[key + "_b"] = a, b
        for op in ("dots", "angulars", "euclideans"):
            out[f"{key}_{op}_serial"] = getattr(serial, op)(a, b, "f64")
            out[f"{key}_{op}_dispatch"] = getattr(dispatch, op)(a, b, "f64")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nibble_path.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")
    make_compact(serial)
    make_cast(serial)
    make_moments(serial)


def make_compact(serial):
    """compact_path.npz: the in-place down-casts of a dots matrix (f32 -> bf16, i32 -> i8 rescaled by the norms), from the
    reference's scalar helpers. Matrices with padded rows included; an all-zero vector on each side of the i8 case."""
    out = {}
    for si, (m, n, k) in enumerate(SHAPES):
        rng = np.random.default_rng(5000 + si)
        a, b = rng.integers(-128, 128, (m, k), dtype=np.int8), rng.integers(-128, 128, (n, k), dtype=np.int8)
        a[m // 2], b[n // 3] = 0, 0
        b[0] = a[0]                                              # a pair with cosine 1: the rescaled cell sits at the clamp
        c = np.zeros((m, n + si), dtype=np.int32)                # rows padded by `si` cells
        c[:, :n] = a.astype(np.int32) @ b.astype(np.int32).T
        an, bn = (a.astype(np.int32) ** 2).sum(1).astype(np.int32), (b.astype(np.int32) ** 2).sum(1).astype(np.int32)
        key = f"i8_{m}x{n}x{k}"
        out[key + "_c"], out[key + "_pad"], out[key + "_an"], out[key + "_bn"] = c, np.int64(si), an, bn
        out[key + "_compact_serial"] = serial.dots_compact(c[:, :n], an, bn)
        f = np.zeros((m, n + si), dtype=np.float32)
        f[:, :n] = (rng.standard_normal((m, n)) * np.exp2(rng.integers(-30, 31, (m, n)))).astype(np.float32)
        f[0, 0], f[m - 1, n - 1] = np.float32(np.inf), np.float32(-0.0)
        f.view(np.uint32)[0, 1 % n] = 0x3F808000                 # exactly half way between two bf16 values: ties to even
        key = f"bf16_{m}x{n}x{k}"
        out[key + "_c"], out[key + "_pad"] = f, np.int64(si)
        out[key + "_compact_serial"] = serial.dots_compact(f[:, :n])
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "compact_path.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


CAST_TYPES = ["f64", "f32", "f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2", "i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "i4", "u4", "u1"]


def cast_pair_defined(a: str, b: str) -> bool:
    """Pairs of the bulk conversion the reference defines (its integer hub has no u1 source and no u4 / u1 target)."""
    signed = ("i8", "i16", "i32", "i64", "i4")
    return not ((a == "u1" and b in signed) or (a in signed and b in ("u4", "u1")))


def make_cast(serial):
    """cast_path.npz: nk_cast_serial on 136 values (seventeen whole batches) of every source type to every target type."""
    out = {}
    for si, a in enumerate(CAST_TYPES):
        x = syn.cast_samples(a, 136, 6000 + si)
        out["from_" + a] = x
        for b in CAST_TYPES:
            if a != b and cast_pair_defined(a, b):
                out[f"{a}_to_{b}"] = serial.cast(x, a, b, 136)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cast_path.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


def make_moments(serial):
    """moments_path.npz: nk_reduce_moments_<t>_serial on 1000 contiguous values and on every third of 999, all nineteen types;
    plus the saturating cases of the 32 / 64-bit integers. Results are stored in their own types (`_sum`, `_sumsq`)."""
    out = {}

    def keep(key, pair):
        out[key + "_sum"], out[key + "_sumsq"] = np.array([pair[0]]), np.array([pair[1]])

    for si, t in enumerate(CAST_TYPES):
        x = syn.moments_samples(t, 1000, 9000 + si)
        out["from_" + t] = x
        per_unit = 8 // oracle.CAST_BITS[t] if oracle.CAST_BITS[t] < 8 else 1
        keep(t + "_all", serial.moments(x, t, 1000 if per_unit > 1 else None))
        keep(t + "_strided", serial.moments(x, t, 333 * per_unit if per_unit == 1 else 40 * per_unit, 3 * max(oracle.CAST_BITS[t] // 8, 1)))
    big = {"i32": np.full(5, -2 ** 31, dtype=np.int32), "u32": np.full(5, 2 ** 32 - 1, dtype=np.uint32),
           "i64": np.array([2 ** 63 - 1, 2 ** 63 - 1, 5, -7], dtype=np.int64), "u64": np.array([2 ** 64 - 1, 2 ** 64 - 1, 3], dtype=np.uint64),
           "i64_negative": np.array([-2 ** 63, -2 ** 63, -1], dtype=np.int64)}
    for key, x in big.items():
        out["big_" + key] = x
        keep("big_" + key, serial.moments(x, key.split("_")[0]))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moments_path.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    if "--only-moments" in sys.argv:
        make_moments(oracle.ref_serial())
    elif "--only-compact" in sys.argv:
        make_compact(oracle.ref_serial())
    elif "--only-cast" in sys.argv:
        make_cast(oracle.ref_serial())
    else:
        main()
