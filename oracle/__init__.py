"""TEST INFRASTRUCTURE ONLY: Python face of the CPU oracle.

`oracle.*` wraps oracle/nk_oracle.c (our scalar restatement of NumKong's packed-contraction path);
`oracle.ref` / `oracle.ref_serial` wrap the reference itself when it has been compiled from its own
sources into oracle/_ref/ (see oracle/Makefile). Only tests/, __graft_entry__.smoke() and bench.py's
CPU-baseline leg may import this package; the product never does.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path
from typing import Optional

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "liboracle.so"
REF_SO = _HERE / "_ref" / "libnumkong.so"
REF_SERIAL_SO = _HERE / "_ref" / "libnkref_serial.so"
REF_BACKENDS_SO = _HERE / "_ref" / "libnkref_backends.so"

CODES = {"i8": 1 << 2, "u8": 1 << 6, "f32": 1 << 11, "f16": 1 << 12, "bf16": 1 << 13,
         "e4m3": 1 << 14, "e5m2": 1 << 15, "e2m3": 1 << 18, "e3m2": 1 << 19, "i4": 1 << 16, "u4": 1 << 17, "u1": 1 << 1, "f64": 1 << 10}
BYTES = {"i8": 1, "u8": 1, "f32": 4, "f16": 2, "bf16": 2, "e4m3": 1, "e5m2": 1, "e2m3": 1, "e3m2": 1, "i4": 1, "u4": 1, "u1": 1, "f64": 8}
STORAGE = {"i8": np.int8, "u8": np.uint8, "f32": np.float32, "f16": np.uint16, "bf16": np.uint16,
           "e4m3": np.uint8, "e5m2": np.uint8, "e2m3": np.uint8, "e3m2": np.uint8, "i4": np.uint8, "u4": np.uint8, "u1": np.uint8, "f64": np.float64}


# Every real type nk_cast converts (numerically nk_dtype_t), bits per value, NumPy storage of a buffer of them.
CAST_CODES = dict(CODES, i16=1 << 3, i32=1 << 4, i64=1 << 5, u16=1 << 7, u32=1 << 8, u64=1 << 9)
CAST_BITS = {"u1": 1, "i4": 4, "u4": 4, "i8": 8, "u8": 8, "e4m3": 8, "e5m2": 8, "e2m3": 8, "e3m2": 8, "i16": 16, "u16": 16, "f16": 16,
             "bf16": 16, "i32": 32, "u32": 32, "f32": 32, "i64": 64, "u64": 64, "f64": 64}
CAST_STORAGE = dict(STORAGE, i16=np.int16, i32=np.int32, i64=np.int64, u16=np.uint16, u32=np.uint32, u64=np.uint64)


def _cast_with(fn, x: np.ndarray, from_dtype: str, to_dtype: str, n: Optional[int]) -> np.ndarray:
    x = np.ascontiguousarray(x)
    n = int(n) if n is not None else x.nbytes * 8 // CAST_BITS[from_dtype]
    out = np.zeros(max((n * CAST_BITS[to_dtype] + 7) // 8, 1) + 8, dtype=np.uint8)   # slack: the reference writes whole batches
    fn(x.ctypes.data, CAST_CODES[from_dtype], n, out.ctypes.data, CAST_CODES[to_dtype])
    return out[:(n * CAST_BITS[to_dtype] + 7) // 8].view(CAST_STORAGE[to_dtype]).copy()


def cast(x: np.ndarray, from_dtype: str, to_dtype: str, n: Optional[int] = None) -> np.ndarray:
    """Bulk conversion of `n` values (default: all of `x`) with the reference's rules; returns the result's storage."""
    return _cast_with(_lib.orc_cast, x, from_dtype, to_dtype, n)


def moments_result_dtype(dtype: str):
    """(sum, sum of squares) types of nk_reduce_moments_<dtype> (include/numkong/reduce.h:120-279)."""
    if dtype in ("f64", "f32"):
        return np.float64, np.float64
    if dtype in ("f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2"):
        return np.float32, np.float32
    return (np.int64 if dtype in ("i8", "i16", "i32", "i64", "i4") else np.uint64), np.uint64


def _moments_with(fn, x: np.ndarray, dtype: str, count: Optional[int], stride: Optional[int]):
    x = np.ascontiguousarray(x)
    unit = max(CAST_BITS[dtype] // 8, 1)
    stride = int(stride) if stride is not None else unit
    count = int(count) if count is not None else (x.nbytes // stride) * (8 // CAST_BITS[dtype] if CAST_BITS[dtype] < 8 else 1)
    s, q = np.zeros(1, dtype=np.uint64), np.zeros(1, dtype=np.uint64)
    fn(x.ctypes.data, count, stride, s.ctypes.data, q.ctypes.data)
    st, qt = moments_result_dtype(dtype)
    return s.view(np.uint8)[:np.dtype(st).itemsize].view(st)[0], q.view(np.uint8)[:np.dtype(qt).itemsize].view(qt)[0]


def moments(x: np.ndarray, dtype: str, count: Optional[int] = None, stride: Optional[int] = None):
    """Sum and sum of squares of `count` values of `dtype` taken `stride` bytes apart, with the reference's scalar rules."""
    code = CAST_CODES[dtype]
    return _moments_with(lambda p, n, st, s, q: _lib.orc_moments(code, p, n, st, s, q), x, dtype, count, stride)


def _depth(x: np.ndarray, dtype: str, depth: Optional[int]) -> int:
    """Logical dimensions of a row: 4-bit types hold two per byte (an explicit `depth` may be odd)."""
    return int(depth) if depth is not None else x.shape[1] * {"i4": 2, "u4": 2, "u1": 8}.get(dtype, 1)


def build(force: bool = False) -> Path:
    """Compiles oracle/nk_oracle.c into liboracle.so (gcc, a second or two)."""
    if force or not _SO.exists() or _SO.stat().st_mtime < (_HERE / "nk_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-s", "-C", str(_HERE), "all"], check=True)
    return _SO


def reference_root() -> Optional[Path]:
    """Where the NumKong source tree lies: $NUMKONG_REFERENCE, else a `reference` directory beside this repository."""
    import os
    for candidate in (os.environ.get("NUMKONG_REFERENCE"), _HERE.parent.parent / "reference"):
        if candidate and Path(candidate, "c", "numkong.c").exists():
            return Path(candidate)
    return None


def build_ref(root: Optional[str] = None) -> bool:
    """Compiles the reference from its own sources into oracle/_ref/ when the source tree is present."""
    root = Path(root) if root else reference_root()
    if root is None or not Path(root, "c", "numkong.c").exists():
        return False
    subprocess.run(["make", "-s", "-C", str(_HERE), "ref", f"REF={root}", "-j8"], check=True)
    return True


def _load() -> ctypes.CDLL:
    build()
    lib = ctypes.CDLL(str(_SO))
    u64, vp, i32 = ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int
    lib.orc_decode.restype, lib.orc_decode.argtypes = None, [i32, vp, u64, vp]
    lib.orc_dots.restype, lib.orc_dots.argtypes = None, [i32, vp, u64, vp, u64, vp, u64, u64, u64, u64]
    lib.orc_spatials.restype, lib.orc_spatials.argtypes = None, [i32, i32, vp, u64, vp, u64, vp, u64, u64, u64, u64]
    lib.orc_sumsq.restype, lib.orc_sumsq.argtypes = ctypes.c_double, [i32, vp, u64]
    lib.orc_sets.restype, lib.orc_sets.argtypes = None, [i32, vp, u64, vp, u64, vp, u64, u64, u64, u64]
    lib.orc_rsqrt_f32.restype, lib.orc_rsqrt_f32.argtypes = ctypes.c_float, [ctypes.c_float]
    lib.orc_cast.restype, lib.orc_cast.argtypes = ctypes.c_int, [vp, i32, u64, vp, i32]
    lib.orc_moments.restype, lib.orc_moments.argtypes = ctypes.c_int, [i32, vp, u64, u64, vp, vp]
    lib.orc_compact_bf16.restype, lib.orc_compact_bf16.argtypes = None, [vp, u64, u64, u64]
    lib.orc_compact_i8.restype, lib.orc_compact_i8.argtypes = None, [vp, u64, u64, u64, vp, vp]
    for name in ("orc_maxsim_argmax_dot", "orc_maxsim_coarse_i8"):
        f = getattr(lib, name)
        f.restype, f.argtypes = ctypes.c_double, [i32, vp, u64, u64, vp, u64, u64, u64, vp]
    lib.orc_maxsim_exhaustive.restype = ctypes.c_double
    lib.orc_maxsim_exhaustive.argtypes = [i32, vp, u64, u64, vp, u64, u64, u64]
    return lib


_lib = _load()


def _as_storage(x: np.ndarray, dtype: str) -> np.ndarray:
    x = np.asarray(x)
    if x.ndim != 2:
        raise ValueError("expected a 2-D matrix")
    if x.itemsize != BYTES[dtype]:
        raise TypeError(f"{dtype} needs {BYTES[dtype]}-byte elements")
    if x.shape[1] > 1 and x.strides[1] != x.itemsize:
        x = np.ascontiguousarray(x)
    return x


def _stride(x: np.ndarray) -> int:
    return x.strides[0] if x.shape[0] > 1 else x.shape[1] * x.itemsize


def decode(x: np.ndarray, dtype: str) -> np.ndarray:
    """Exact f32 values of a storage array."""
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, dtype=np.float32)
    _lib.orc_decode(CODES[dtype], x.ctypes.data, x.size, out.ctypes.data)
    return out


def out_dtype(dtype: str, op: str = "dots"):
    if dtype in ("f32", "f64"):
        return np.float64
    if op == "dots" and dtype in ("i8", "i4"):
        return np.int32
    if (op == "dots" and dtype in ("u8", "u4", "u1")) or op == "hammings":
        return np.uint32
    return np.float32


def dots(a: np.ndarray, b: np.ndarray, dtype: str, depth: Optional[int] = None) -> np.ndarray:
    a, b = _as_storage(a, dtype), _as_storage(b, dtype)
    c = np.empty((a.shape[0], b.shape[0]), dtype=out_dtype(dtype))
    _lib.orc_dots(CODES[dtype], a.ctypes.data, _stride(a), b.ctypes.data, _stride(b), c.ctypes.data,
                  c.shape[1] * c.itemsize, a.shape[0], b.shape[0], _depth(a, dtype, depth))
    return c


def _spatials(kind: int, a, b, dtype, depth=None):
    a, b = _as_storage(a, dtype), _as_storage(b, dtype)
    c = np.empty((a.shape[0], b.shape[0]), dtype=out_dtype(dtype, "spatial"))
    _lib.orc_spatials(kind, CODES[dtype], a.ctypes.data, _stride(a), b.ctypes.data, _stride(b), c.ctypes.data,
                      c.shape[1] * c.itemsize, a.shape[0], b.shape[0], _depth(a, dtype, depth))
    return c


def angulars(a, b, dtype, depth: Optional[int] = None):
    return _spatials(0, a, b, dtype, depth)


def euclideans(a, b, dtype, depth: Optional[int] = None):
    return _spatials(1, a, b, dtype, depth)


def _sets(kind: int, a, b, depth=None):
    a, b = _as_storage(a, "u1"), _as_storage(b, "u1")
    c = np.empty((a.shape[0], b.shape[0]), dtype=np.uint32 if kind == 0 else np.float32)
    _lib.orc_sets(kind, a.ctypes.data, _stride(a), b.ctypes.data, _stride(b), c.ctypes.data, c.shape[1] * c.itemsize,
                  a.shape[0], b.shape[0], _depth(a, "u1", depth))
    return c


def hammings(a, b, dtype: str = "u1", depth: Optional[int] = None):
    """Hamming distances between bit vectors (u32)."""
    return _sets(0, a, b, depth)


def jaccards(a, b, dtype: str = "u1", depth: Optional[int] = None):
    """Jaccard distances between bit vectors (f32)."""
    return _sets(1, a, b, depth)


def _compact(lib_fn_bf16, lib_fn_i8, c: np.ndarray, a_norms, b_norms) -> np.ndarray:
    """Runs an in-place compaction on a copy of `c` (f32 -> bf16 bits, or i32 -> i8 with the two squared-norm vectors)."""
    assert c.ndim == 2 and c.strides[1] == 4 and c.dtype in (np.float32, np.int32)
    rows, cols = c.shape
    stride = c.strides[0]
    work = np.zeros(max((rows - 1) * stride + cols * 4, 4), dtype=np.uint8)
    for i in range(rows):
        work[i * stride:i * stride + cols * 4] = np.ascontiguousarray(c[i]).view(np.uint8)
    if c.dtype == np.float32:
        lib_fn_bf16(work.ctypes.data, rows, cols, stride)
        return work[:rows * cols * 2].view(np.uint16).reshape(rows, cols).copy()
    an, bn = np.ascontiguousarray(a_norms, dtype=np.int32), np.ascontiguousarray(b_norms, dtype=np.int32)
    lib_fn_i8(work.ctypes.data, rows, cols, stride, an.ctypes.data, bn.ctypes.data)
    return work[:rows * cols].view(np.int8).reshape(rows, cols).copy()


def dots_compact(c: np.ndarray, a_norms=None, b_norms=None) -> np.ndarray:
    """Down-cast of a dots matrix: f32 -> bf16 storage (uint16), or i32 -> i8 rescaled by 127 / (|a| |b|)."""
    return _compact(_lib.orc_compact_bf16, _lib.orc_compact_i8, c, a_norms, b_norms)


def sumsq(x: np.ndarray, dtype: str, depth: Optional[int] = None) -> np.ndarray:
    x = _as_storage(x, dtype)
    return np.array([_lib.orc_sumsq(CODES[dtype], x[i:i + 1].ctypes.data, _depth(x, dtype, depth)) for i in range(x.shape[0])])


def _maxsim(fn, q, d, dtype, want_best):
    q, d = _as_storage(q, dtype), _as_storage(d, dtype)
    best = np.zeros(q.shape[0], dtype=np.uint32)
    total = fn(CODES[dtype], q.ctypes.data, _stride(q), q.shape[0], d.ctypes.data, _stride(d), d.shape[0], q.shape[1],
               best.ctypes.data)
    value = float(total) if dtype == "f32" else float(np.float32(total))
    return (value, best) if want_best else value


def maxsim(q, d, dtype, want_best: bool = False):
    """Fused semantics (argmax of the raw dot, winner normalised) - what the CUDA kernel implements."""
    return _maxsim(_lib.orc_maxsim_argmax_dot, q, d, dtype, want_best)


def maxsim_coarse_i8(q, d, dtype, want_best: bool = False):
    """The reference's serial back end (i8 screening, full-precision refinement)."""
    return _maxsim(_lib.orc_maxsim_coarse_i8, q, d, dtype, want_best)


def maxsim_exhaustive(q, d, dtype) -> float:
    q, d = _as_storage(q, dtype), _as_storage(d, dtype)
    return float(_lib.orc_maxsim_exhaustive(CODES[dtype], q.ctypes.data, _stride(q), q.shape[0], d.ctypes.data,
                                            _stride(d), d.shape[0], q.shape[1]))


def exact_dots_f64(a: np.ndarray, b: np.ndarray, dtype: str) -> np.ndarray:
    """Ground truth the reference's tests use: exactly decoded inputs, f64 accumulation."""
    return decode(a, dtype).astype(np.float64) @ decode(b, dtype).astype(np.float64).T


# ---------------------------------------------------------------- the reference itself, when compiled
class _Ref:
    """ctypes view of a reference build: `prefix` is 'nk_' (dispatch library) or 'ref_' (scalar shim)."""

    def __init__(self, path: Path, prefix: str):
        self.lib = ctypes.CDLL(str(path))
        self.prefix = prefix
        if prefix == "nk_":
            self.lib.nk_capabilities.restype = ctypes.c_uint64
            self.lib.nk_configure_thread.argtypes = [ctypes.c_uint64]
            self.configure_thread()

    def configure_thread(self):
        if self.prefix == "nk_":
            self.lib.nk_configure_thread(self.lib.nk_capabilities())

    def _fn(self, name, restype, argtypes):
        f = getattr(self.lib, self.prefix + name)
        f.restype, f.argtypes = restype, argtypes
        return f

    def pack(self, b: np.ndarray, dtype: str, family: str = "dots", depth: Optional[int] = None) -> np.ndarray:
        b = _as_storage(b, dtype)
        u64, vp = ctypes.c_uint64, ctypes.c_void_p
        k = _depth(b, dtype, depth)
        size = self._fn(f"{family}_packed_size_{dtype}", u64, [u64, u64])(b.shape[0], k)
        blob = np.zeros(size + 64, dtype=np.uint8)
        self._fn(f"{family}_pack_{dtype}", None, [vp, u64, u64, u64, vp])(b.ctypes.data, b.shape[0], k, _stride(b), blob.ctypes.data)
        return blob

    def packed(self, op: str, a: np.ndarray, blob: np.ndarray, n: int, dtype: str, out: Optional[np.ndarray] = None,
               rows: Optional[slice] = None, depth: Optional[int] = None) -> np.ndarray:
        a = _as_storage(a, dtype)
        u64, vp = ctypes.c_uint64, ctypes.c_void_p
        c = out if out is not None else np.empty((a.shape[0], n), dtype=out_dtype(dtype, op))
        f = self._fn(f"{op}_packed_{dtype}", None, [vp, vp, vp, u64, u64, u64, u64, u64])
        lo, hi = (0, a.shape[0]) if rows is None else (rows.start, rows.stop)
        f(a[lo:hi].ctypes.data, blob.ctypes.data, c[lo:hi].ctypes.data, hi - lo, n, _depth(a, dtype, depth), _stride(a), c.strides[0])
        return c

    def dots(self, a, b, dtype, depth=None):
        return self.packed("dots", a, self.pack(b, dtype, depth=depth), np.asarray(b).shape[0], dtype, depth=depth)

    def angulars(self, a, b, dtype, depth=None):
        return self.packed("angulars", a, self.pack(b, dtype, depth=depth), np.asarray(b).shape[0], dtype, depth=depth)

    def euclideans(self, a, b, dtype, depth=None):
        return self.packed("euclideans", a, self.pack(b, dtype, depth=depth), np.asarray(b).shape[0], dtype, depth=depth)

    def hammings(self, a, b, dtype="u1", depth=None):
        return self.packed("hammings", a, self.pack(b, "u1", depth=depth), np.asarray(b).shape[0], "u1", depth=depth)

    def jaccards(self, a, b, dtype="u1", depth=None):
        return self.packed("jaccards", a, self.pack(b, "u1", depth=depth), np.asarray(b).shape[0], "u1", depth=depth)

    def dots_compact(self, c, a_norms=None, b_norms=None):
        u64, vp = ctypes.c_uint64, ctypes.c_void_p
        return _compact(self._fn("dots_compact_bf16", None, [vp, u64, u64, u64]),
                        self._fn("dots_compact_i8", None, [vp, u64, u64, u64, vp, vp]), c, a_norms, b_norms)

    def cast(self, x, from_dtype, to_dtype, n=None):
        u64, vp = ctypes.c_uint64, ctypes.c_void_p
        return _cast_with(self._fn("cast", None, [vp, ctypes.c_int, u64, vp, ctypes.c_int]), x, from_dtype, to_dtype, n)

    def moments(self, x, dtype, count=None, stride=None):
        u64, vp = ctypes.c_uint64, ctypes.c_void_p
        return _moments_with(self._fn(f"reduce_moments_{dtype}", None, [vp, u64, u64, vp, vp]), x, dtype, count, stride)

    def maxsim(self, q, d, dtype) -> float:
        q, d = _as_storage(q, dtype), _as_storage(d, dtype)
        u64, vp = ctypes.c_uint64, ctypes.c_void_p
        qp, dp = self.pack(q, dtype, "maxsim"), self.pack(d, dtype, "maxsim")
        res = (ctypes.c_double if dtype == "f32" else ctypes.c_float)()
        self._fn(f"maxsim_packed_{dtype}", None, [vp, vp, u64, u64, u64, vp])(qp.ctypes.data, dp.ctypes.data, q.shape[0], d.shape[0], q.shape[1], ctypes.addressof(res))
        return float(res.value)


def ref() -> Optional[_Ref]:
    """The reference's dispatch library (best SIMD back end of this CPU), or None when it was not compiled."""
    return _Ref(REF_SO, "nk_") if REF_SO.exists() else None


def ref_serial() -> Optional[_Ref]:
    """The reference's scalar back end, or None when it was not compiled."""
    return _Ref(REF_SERIAL_SO, "ref_") if REF_SERIAL_SO.exists() else None


# ---------------------------------------------------------------- every x86 back end of the 16-bit float kernels
# Capability bits of the reference (include/numkong/capabilities.h:261-304) each back end needs.
_BACKEND_CAPS = {"serial": 1 << 0, "haswell": 1 << 2, "skylake": 1 << 3, "genoa": 1 << 8, "sapphireamx": 1 << 18}
_BACKENDS = {"bf16": ("serial", "haswell", "skylake", "genoa", "sapphireamx"), "f16": ("serial", "haswell", "skylake")}


class _RefBackends:
    """The reference's packed bf16 / f16 kernels, one back end at a time (oracle/ref_backends_shim.c): the error of the
    WORST of them on given inputs is the envelope the device kernels are held to."""

    def __init__(self, path: Path):
        self.lib = ctypes.CDLL(str(path))
        self.lib.refb_capabilities.restype = ctypes.c_uint64
        self.lib.refb_configure_thread.argtypes = [ctypes.c_uint64]
        self.caps = int(self.lib.refb_capabilities())
        self.lib.refb_configure_thread(self.caps)  # AMX needs the kernel's permission per thread

    def available(self, dtype: str):
        return [b for b in _BACKENDS[dtype] if self.caps & _BACKEND_CAPS[b]]

    def packed(self, backend: str, op: str, a: np.ndarray, b: np.ndarray, dtype: str) -> np.ndarray:
        a, b = _as_storage(a, dtype), _as_storage(b, dtype)
        u64, vp = ctypes.c_uint64, ctypes.c_void_p
        self.lib.refb_configure_thread(self.caps)
        n, k = b.shape
        size = getattr(self.lib, f"refb_{backend}_dots_packed_size_{dtype}")
        size.restype, size.argtypes = u64, [u64, u64]
        blob = np.zeros(size(n, k) + 64, dtype=np.uint8)
        pack = getattr(self.lib, f"refb_{backend}_dots_pack_{dtype}")
        pack.restype, pack.argtypes = None, [vp, u64, u64, u64, vp]
        pack(b.ctypes.data, n, k, _stride(b), blob.ctypes.data)
        fn = getattr(self.lib, f"refb_{backend}_{op}_packed_{dtype}")
        fn.restype, fn.argtypes = None, [vp, vp, vp, u64, u64, u64, u64, u64]
        c = np.empty((a.shape[0], n), dtype=np.float32)
        fn(a.ctypes.data, blob.ctypes.data, c.ctypes.data, a.shape[0], n, k, _stride(a), c.strides[0])
        return c


def ref_backends() -> Optional[_RefBackends]:
    """Per-back-end view of the reference, or None when it was not compiled."""
    return _RefBackends(REF_BACKENDS_SO) if REF_BACKENDS_SO.exists() else None
