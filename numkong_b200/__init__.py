"""Host-side mirror of NumKong's Python interface for the packed-contraction path, running on a B200.

Same names and argument meaning as the reference's module (python/numkong.c:1135-1146,
python/numkong/__init__.pyi:999-1074):

    dots_pack(b, dtype=None) -> PackedMatrix
    dots_packed / angulars_packed / euclideans_packed(a, packed, *, out=None) -> matrix
    maxsim_pack(vectors, dtype=None) -> MaxSimPackedMatrix
    maxsim_packed(q_packed, d_packed) -> float ;  maxsim(q, d, dtype=None) -> float

Every call goes through the C ABI of libnumkong_b200.so with plain pointers. Inputs may be
NumPy arrays (host memory: the library stages them) or torch tensors (host or CUDA: CUDA
tensors are used in place and the result is a CUDA tensor). Element types NumPy cannot name
(bf16, e4m3, e5m2, e2m3, e3m2) are passed as uint16 / uint8 storage with `dtype="bf16"` etc.,
or as ml_dtypes / torch low-precision dtypes.
"""
from __future__ import annotations

import ctypes
from typing import Any, Optional, Tuple

import numpy as np

from . import _lib
from ._lib import DIMENSIONS_PER_VALUE, DTYPE_BYTES, DTYPE_CODES, MAXSIM_DTYPES, PACKED_DTYPES, check, last_error, lib

__all__ = [
    "PackedMatrix", "MaxSimPackedMatrix", "dots_pack", "dots_packed", "angulars_packed", "euclideans_packed",
    "dots_symmetric", "angulars_symmetric", "euclideans_symmetric",
    "hammings_packed", "jaccards_packed", "hammings_symmetric", "jaccards_symmetric",
    "maxsim_pack", "maxsim_packed", "maxsim", "maxsims_packed", "angulars_packed_topk", "euclideans_packed_topk",
    "topk_smallest", "merge_topk", "synchronize", "set_wait_limit_ns", "set_stream", "launch_count", "last_error", "dots_compact", "cast", "moments", "set_accumulation_span",
]

_NUMPY_NAMES = {
    "int8": "i8", "uint8": "u8", "float32": "f32", "float64": "f64", "float16": "f16", "bfloat16": "bf16",
    "float8_e4m3fn": "e4m3", "float8_e5m2": "e5m2", "float6_e2m3fn": "e2m3", "float6_e3m2fn": "e3m2",
}
_TORCH_NAMES = {
    "torch.int8": "i8", "torch.uint8": "u8", "torch.float32": "f32", "torch.float64": "f64", "torch.float16": "f16",
    "torch.bfloat16": "bf16", "torch.float8_e4m3fn": "e4m3", "torch.float8_e5m2": "e5m2",
}
_OUT_NUMPY = {"i8": np.int32, "u8": np.uint32, "i4": np.int32, "u4": np.uint32, "u1": np.uint32, "f32": np.float64, "f64": np.float64}


def _integer_cells(dtype: str, op: str) -> bool:
    """Integer result cells: dots of the integer types, and Hamming distances."""
    return (op == "dots" and dtype in ("i8", "u8", "i4", "u4", "u1")) or op == "hammings"


def _is_torch(x: Any) -> bool:
    return type(x).__module__.startswith("torch")


_CAI_TYPES = {"<f2": "f16", "<f4": "f32", "<f8": "f64", "|i1": "i8", "|u1": "u8"}  # other element types need dtype=...


def _adopt_device_array(x: Any) -> Any:
    """Zero-copy handle on a foreign CUDA array: a torch tensor sharing the memory when the object speaks DLPack for a
    CUDA device, a pointer/shape/stride record when it only has __cuda_array_interface__. Anything else is returned
    unchanged and handled as a host array."""
    dl_device = getattr(x, "__dlpack_device__", None)
    if dl_device is not None and hasattr(x, "__dlpack__"):
        kind = int(dl_device()[0])
        if kind in (2, 13):  # kDLCUDA, kDLCUDAManaged
            import torch
            return torch.from_dlpack(x)
        return x
    cai = getattr(x, "__cuda_array_interface__", None)
    return _ForeignCuda(x, cai) if cai is not None else x


class _ForeignCuda:
    """A 2-D CUDA array described by __cuda_array_interface__ (pointer, shape, byte strides); used in place."""

    def __init__(self, owner: Any, cai: dict):
        if len(cai["shape"]) != 2:
            raise ValueError("expected a 2-D matrix")
        self.owner = owner  # keeps the exporter's memory alive
        self.rows, self.cols = (int(s) for s in cai["shape"])
        self.itemsize = int(cai["typestr"][2:])
        strides = cai.get("strides") or (self.cols * self.itemsize, self.itemsize)
        if self.cols > 1 and int(strides[1]) != self.itemsize:
            raise ValueError("rows must be contiguous (column-major inputs are not supported)")
        self.stride = int(strides[0])
        self.ptr = int(cai["data"][0])
        self.name = _CAI_TYPES.get(cai["typestr"])

    @property
    def device(self):
        import torch
        return torch.device("cuda", torch.cuda.current_device())


class _View:
    """Pointer, shape and byte strides of a 2-D matrix, plus where it lives."""

    def __init__(self, x: Any, dtype: Optional[str]):
        # Device arrays of other libraries (CuPy, Numba, ...) come in without a copy: through DLPack when the object
        # offers it for a CUDA device, else through __cuda_array_interface__. The reference's binding rejects CUDA
        # capsules (python/dlpack_interop.c:97-99); here they are the fast path.
        if not _is_torch(x) and not isinstance(x, np.ndarray):
            x = _adopt_device_array(x)
        self.obj = x
        if isinstance(x, _ForeignCuda):
            name = dtype or x.name
            if name is None:
                raise TypeError("pass dtype='bf16' etc. for storage words that have no element type of their own")
            self.is_cuda, self.ptr, self.rows, self.cols = True, x.ptr, x.rows, x.cols
            self.stride = x.stride if x.rows > 1 else x.cols * x.itemsize
            item = x.itemsize
        elif _is_torch(x):
            if x.dim() != 2:
                raise ValueError("expected a 2-D matrix")
            if x.stride(1) != 1 and x.shape[1] > 1:
                raise ValueError("rows must be contiguous (column-major inputs are not supported)")
            name = dtype or _TORCH_NAMES.get(str(x.dtype))
            if name is None:
                raise TypeError(f"unsupported torch dtype {x.dtype}")
            self.is_cuda = x.is_cuda
            self.ptr = x.data_ptr()
            self.rows, self.cols = int(x.shape[0]), int(x.shape[1])
            self.stride = int(x.stride(0)) * x.element_size() if self.rows > 1 else self.cols * x.element_size()
            item = x.element_size()
        else:
            x = np.asarray(x)
            self.obj = x
            if x.ndim != 2:
                raise ValueError("expected a 2-D matrix")
            if x.shape[1] > 1 and x.strides[1] != x.itemsize:
                raise ValueError("rows must be contiguous (column-major inputs are not supported)")
            name = dtype or _NUMPY_NAMES.get(x.dtype.name)
            if name is None:
                raise TypeError(f"unsupported numpy dtype {x.dtype}; pass dtype='bf16' etc. with uint16/uint8 storage")
            self.is_cuda = False
            self.ptr = x.ctypes.data
            self.rows, self.cols = int(x.shape[0]), int(x.shape[1])
            self.stride = int(x.strides[0]) if self.rows > 1 else self.cols * x.itemsize
            item = x.itemsize
        if name not in DTYPE_CODES:
            raise TypeError(f"unknown dtype name {name!r}")
        if item != DTYPE_BYTES[name]:
            raise TypeError(f"dtype {name!r} needs {DTYPE_BYTES[name]}-byte elements, got {item}-byte storage")
        self.dtype = name
        self.depth = self.cols * DIMENSIONS_PER_VALUE.get(name, 1)  # logical dimensions of a row


def _view_like(x: Any, dtype: Optional[str], packed_dtype: str) -> _View:
    """View of `x` for use against a matrix packed as `packed_dtype`. Unsigned storage words (uint8 /
    uint16 / int16) stand for the 8/6-bit and 16-bit float types NumPy and torch cannot name."""
    if dtype is None:
        name = (_TORCH_NAMES.get(str(x.dtype)) if _is_torch(x) else _NUMPY_NAMES.get(np.asarray(x).dtype.name))
        container = (name in (None, "u8") and packed_dtype not in ("i8", "u8", "f32", "f64")) or \
                    (name == "i8" and packed_dtype in ("i4", "u4")) or (name == "u8" and packed_dtype == "u1")
        dtype = packed_dtype if container else name
    v = _View(x, dtype)
    if v.dtype != packed_dtype:
        raise TypeError(f"dtype mismatch: matrix is {v.dtype}, packed matrix is {packed_dtype}")
    return v


def _alloc_bytes(nbytes: int, cuda: bool):
    if cuda:
        import torch
        return torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    return np.empty(nbytes, dtype=np.uint8)


def _ptr(buf: Any) -> int:
    return buf.data_ptr() if _is_torch(buf) else buf.ctypes.data


class PackedMatrix:
    """Opaque pre-packed B matrix (the counterpart of the reference's PackedMatrix object,
    python/matrix.h): the blob lives where the source matrix lived (host or CUDA)."""

    kind = "dots"

    def __init__(self, buffer: Any, dtype: str, width: int, depth: int):
        self.buffer, self.dtype, self.width, self.depth = buffer, dtype, width, depth

    @property
    def nbytes(self) -> int:
        return int(self.buffer.numel()) if _is_torch(self.buffer) else int(self.buffer.nbytes)

    @property
    def is_cuda(self) -> bool:
        return _is_torch(self.buffer) and self.buffer.is_cuda

    @staticmethod
    def packed_size(width: int, depth: int, dtype: str) -> int:
        if dtype not in PACKED_DTYPES:
            raise LookupError(f"no packed kernels for dtype {dtype!r}")
        return int(getattr(lib, f"nk_dots_packed_size_{dtype}")(width, depth))

    def __repr__(self) -> str:
        return f"PackedMatrix(dtype={self.dtype}, width={self.width}, depth={self.depth}, nbytes={self.nbytes})"


class MaxSimPackedMatrix(PackedMatrix):
    """Packed token vectors of one query or one document (python/maxsim.h of the reference)."""

    kind = "maxsim"

    @staticmethod
    def packed_size(count: int, depth: int, dtype: str) -> int:
        if dtype not in MAXSIM_DTYPES:
            raise LookupError(f"MaxSim supports {MAXSIM_DTYPES}, not {dtype!r}")
        return int(getattr(lib, f"nk_maxsim_packed_size_{dtype}")(count, depth))


def dots_pack(b: Any, dtype: Optional[str] = None) -> PackedMatrix:
    """Packs B (width x depth, row-major) once for repeated multiplication. Mirrors nk.dots_pack."""
    v = _View(b, dtype)
    if v.dtype not in PACKED_DTYPES:
        raise LookupError(f"no packed kernels for dtype {v.dtype!r}")
    size = PackedMatrix.packed_size(v.rows, v.depth, v.dtype)
    buf = _alloc_bytes(size, v.is_cuda)
    getattr(lib, f"nk_dots_pack_{v.dtype}")(v.ptr, v.rows, v.depth, v.stride, _ptr(buf))
    check("dots_pack")
    return PackedMatrix(buf, v.dtype, v.rows, v.depth)


def _out_matrix(v: _View, width: int, out: Any, dtype_name: str):
    """Allocates (or validates) the result matrix; returns (object, ptr, stride)."""
    if out is not None:
        if _is_torch(out):
            if tuple(out.shape) != (v.rows, width) or out.element_size() != (8 if dtype_name in ("f32", "f64") else 4):
                raise ValueError("out has the wrong shape or cell size")
            return out, out.data_ptr(), (int(out.stride(0)) * out.element_size() if v.rows > 1 else width * out.element_size())
        if out.shape != (v.rows, width) or out.itemsize != (8 if dtype_name in ("f32", "f64") else 4):
            raise ValueError("out has the wrong shape or cell size")
        return out, out.ctypes.data, (int(out.strides[0]) if v.rows > 1 else width * out.itemsize)
    return None, 0, 0


def _packed_call(op: str, a: Any, packed: PackedMatrix, out: Any, dtype: Optional[str], columns: Optional[Tuple[int, int]] = None):
    if not isinstance(packed, PackedMatrix) or packed.kind != "dots":
        raise TypeError("second argument must be a PackedMatrix produced by dots_pack")
    v = _view_like(a, dtype, packed.dtype)
    if v.depth != packed.depth:
        raise ValueError(f"depth mismatch: a has {v.depth} dimensions, packed matrix has depth {packed.depth}")
    t = v.dtype
    obj, ptr, stride = _out_matrix(v, packed.width, out, t)
    if obj is None:
        if v.is_cuda:
            import torch
            tdt = torch.float64 if t in ("f32", "f64") else (torch.int32 if _integer_cells(t, op) else torch.float32)
            obj = torch.empty((v.rows, packed.width), dtype=tdt, device=v.obj.device)
            ptr, stride = obj.data_ptr(), packed.width * obj.element_size()
        else:
            ndt = np.float64 if t in ("f32", "f64") else (_OUT_NUMPY.get(t, np.float32) if _integer_cells(t, op) else np.float32)
            obj = np.empty((v.rows, packed.width), dtype=ndt)
            ptr, stride = obj.ctypes.data, packed.width * obj.itemsize
    if columns is not None:
        if op != "dots":
            raise ValueError("a column range is available for dots_packed only")
        lib.nkb_dots_packed_columns(DTYPE_CODES[t], v.ptr, _ptr(packed.buffer), ptr, v.rows, packed.width, v.depth, v.stride, stride,
                                    int(columns[0]), int(columns[1]))
    else:
        getattr(lib, f"nk_{op}_packed_{t}")(v.ptr, _ptr(packed.buffer), ptr, v.rows, packed.width, v.depth, v.stride, stride)
    check(f"{op}_packed")
    return obj


def dots_packed(a: Any, packed: PackedMatrix, *, out: Any = None, dtype: Optional[str] = None, columns: Optional[Tuple[int, int]] = None):
    """C = A . B^T with widening accumulation (i8->i32, u8->u32, f32->f64, else f32). Mirrors nk.dots_packed.
    `columns=(first, count)` (an addition; first a multiple of 256) computes only that range of columns of C and leaves
    the rest of `out` untouched (nkb_dots_packed_columns)."""
    return _packed_call("dots", a, packed, out, dtype, columns)


def angulars_packed(a: Any, packed: PackedMatrix, *, out: Any = None, dtype: Optional[str] = None):
    """Batched angular (cosine) distances. Mirrors nk.angulars_packed."""
    return _packed_call("angulars", a, packed, out, dtype)


def euclideans_packed(a: Any, packed: PackedMatrix, *, out: Any = None, dtype: Optional[str] = None):
    """Batched Euclidean distances. Mirrors nk.euclideans_packed."""
    return _packed_call("euclideans", a, packed, out, dtype)


def _symmetric_call(op: str, vectors: Any, out: Any, dtype: Optional[str], start_row: Optional[int], end_row: Optional[int]):
    v = _View(vectors, dtype)
    t = v.dtype
    if t not in PACKED_DTYPES:
        raise LookupError(f"no symmetric kernels for dtype {t!r}")
    n = v.rows
    cell = 8 if t in ("f32", "f64") else 4
    if out is None:
        # Cells below the diagonal are not written by the call; a fresh result starts as zeros (as the reference's does).
        if v.is_cuda:
            import torch
            tdt = torch.float64 if t in ("f32", "f64") else (torch.int32 if _integer_cells(t, op) else torch.float32)
            out = torch.zeros((n, n), dtype=tdt, device=v.obj.device)
        else:
            ndt = np.float64 if t in ("f32", "f64") else (_OUT_NUMPY.get(t, np.float32) if _integer_cells(t, op) else np.float32)
            out = np.zeros((n, n), dtype=ndt)
    if _is_torch(out):
        if tuple(out.shape) != (n, n) or out.element_size() != cell:
            raise ValueError("out has the wrong shape or cell size")
        ptr, stride = out.data_ptr(), (int(out.stride(0)) * cell if n > 1 else n * cell)
    else:
        if out.shape != (n, n) or out.itemsize != cell:
            raise ValueError("out has the wrong shape or cell size")
        ptr, stride = out.ctypes.data, (int(out.strides[0]) if n > 1 else n * cell)
    first = 0 if start_row is None else int(start_row)
    last = n if end_row is None else min(int(end_row), n)
    if last > first:
        getattr(lib, f"nk_{op}_symmetric_{t}")(v.ptr, n, v.depth, v.stride, ptr, stride, first, last - first)
        check(f"{op}_symmetric")
    return out


def dots_symmetric(vectors: Any, *, dtype: Optional[str] = None, out: Any = None, start_row: Optional[int] = None,
                   end_row: Optional[int] = None):
    """Upper triangle (diagonal included) of A . A^T for rows [start_row, end_row). Mirrors nk.dots_symmetric."""
    return _symmetric_call("dots", vectors, out, dtype, start_row, end_row)


def angulars_symmetric(vectors: Any, *, dtype: Optional[str] = None, out: Any = None, start_row: Optional[int] = None,
                       end_row: Optional[int] = None):
    """Upper triangle of the pairwise angular distances (diagonal 0). Mirrors nk.angulars_symmetric."""
    return _symmetric_call("angulars", vectors, out, dtype, start_row, end_row)


def euclideans_symmetric(vectors: Any, *, dtype: Optional[str] = None, out: Any = None, start_row: Optional[int] = None,
                         end_row: Optional[int] = None):
    """Upper triangle of the pairwise Euclidean distances (diagonal 0). Mirrors nk.euclideans_symmetric."""
    return _symmetric_call("euclideans", vectors, out, dtype, start_row, end_row)


def hammings_packed(a: Any, packed: PackedMatrix, *, out: Any = None, dtype: Optional[str] = "u1"):
    """Hamming distances between bit vectors (u32 cells). Mirrors nk.hammings_packed."""
    return _packed_call("hammings", a, packed, out, dtype)


def jaccards_packed(a: Any, packed: PackedMatrix, *, out: Any = None, dtype: Optional[str] = "u1"):
    """Jaccard distances between bit vectors (f32 cells). Mirrors nk.jaccards_packed."""
    return _packed_call("jaccards", a, packed, out, dtype)


def hammings_symmetric(vectors: Any, *, dtype: Optional[str] = "u1", out: Any = None, start_row: Optional[int] = None,
                       end_row: Optional[int] = None):
    """Upper triangle of the pairwise Hamming distances (diagonal 0). Mirrors nk.hammings_symmetric."""
    return _symmetric_call("hammings", vectors, out, dtype, start_row, end_row)


def jaccards_symmetric(vectors: Any, *, dtype: Optional[str] = "u1", out: Any = None, start_row: Optional[int] = None,
                       end_row: Optional[int] = None):
    """Upper triangle of the pairwise Jaccard distances (diagonal 0). Mirrors nk.jaccards_symmetric."""
    return _symmetric_call("jaccards", vectors, out, dtype, start_row, end_row)


def dots_compact(c: Any, a_squared_norms: Any = None, b_squared_norms: Any = None):
    """Down-casts a finished dots matrix IN PLACE and returns the tightly packed result as a view of `c`'s memory:
    f32 cells become bf16 (round to nearest even; returned as torch.bfloat16 or uint16 storage), i32 cells become i8
    rescaled by 127 / (|a_i| |b_j|) from the two squared-norm vectors (int32). Mirrors nk_dots_compact_bf16_serial /
    nk_dots_compact_i8_serial (include/numkong/dots/serial.h:2707-2754). `c` is overwritten from its first byte."""
    cells = str(c.dtype).replace("torch.", "") if hasattr(c, "dtype") else ""
    if cells not in ("float32", "int32"):
        raise TypeError("dots_compact takes the f32 result of a bf16 product or the i32 result of an i8 product")
    to_i8 = cells == "int32"
    v = _View(c, "f32")  # four-byte cells either way
    if to_i8:
        norms = []
        for vec, count in ((a_squared_norms, v.rows), (b_squared_norms, v.cols)):
            if vec is None:
                raise ValueError("the i8 form needs the squared norms of both operands")
            if _is_torch(vec):
                if str(vec.dtype) != "torch.int32" or vec.numel() != count or not vec.is_contiguous():
                    raise ValueError("squared norms must be contiguous int32 vectors, one entry per row / column")
            else:
                vec = np.ascontiguousarray(vec, dtype=np.int32)
                if vec.size != count:
                    raise ValueError("squared norms must hold one entry per row / column")
            norms.append(vec)
        lib.nk_dots_compact_i8(v.ptr, v.rows, v.cols, v.stride, _ptr(norms[0]), _ptr(norms[1]))
    else:
        lib.nk_dots_compact_bf16(v.ptr, v.rows, v.cols, v.stride)
    check("dots_compact")
    if _is_torch(v.obj):
        import torch
        flat = v.obj.view(torch.int8 if to_i8 else torch.bfloat16)
        return torch.as_strided(flat, (v.rows, v.cols), (v.cols, 1), flat.storage_offset())
    if isinstance(v.obj, np.ndarray):
        flat = v.obj.view(np.int8 if to_i8 else np.uint16)
        return np.lib.stride_tricks.as_strided(flat, shape=(v.rows, v.cols), strides=(v.cols * flat.itemsize, flat.itemsize))
    return None


# ---- bulk type conversion -------------------------------------------------------------------------------------------
CAST_CODES = dict(DTYPE_CODES, i16=1 << 3, i32=1 << 4, i64=1 << 5, u16=1 << 7, u32=1 << 8, u64=1 << 9)
CAST_BITS = {"u1": 1, "i4": 4, "u4": 4, "i8": 8, "u8": 8, "e4m3": 8, "e5m2": 8, "e2m3": 8, "e3m2": 8, "i16": 16, "u16": 16,
             "f16": 16, "bf16": 16, "i32": 32, "u32": 32, "f32": 32, "i64": 64, "u64": 64, "f64": 64}
_CAST_NUMPY = {"i8": np.int8, "u8": np.uint8, "i16": np.int16, "u16": np.uint16, "i32": np.int32, "u32": np.uint32, "i64": np.int64,
               "u64": np.uint64, "f16": np.float16, "f32": np.float32, "f64": np.float64, "bf16": np.uint16}
_CAST_TORCH = {"i8": "int8", "u8": "uint8", "i16": "int16", "u16": "uint16", "i32": "int32", "u32": "uint32", "i64": "int64",
               "u64": "uint64", "f16": "float16", "f32": "float32", "f64": "float64", "bf16": "bfloat16", "e4m3": "float8_e4m3fn",
               "e5m2": "float8_e5m2"}
_CAST_NAMES = {"int16": "i16", "uint16": "u16", "int32": "i32", "uint32": "u32", "int64": "i64", "uint64": "u64"}


def cast(x: Any, to_dtype: str, *, dtype: Optional[str] = None, count: Optional[int] = None, out: Any = None):
    """Converts the values of a contiguous array to another element type with the rules of the reference's nk_cast
    (include/numkong/cast.h:55, scalar back end include/numkong/cast/serial.h:2250-2311). `dtype` names the source type
    where the storage cannot (bf16 / fp8 / fp6 words, packed i4 / u4 / u1 bytes); `count` is the number of VALUES
    (default: all the storage holds). NumPy in, NumPy out; CUDA tensor in, CUDA tensor out. Types NumPy or torch cannot
    name come back as uint8 / uint16 storage."""
    is_torch = _is_torch(x)
    if not is_torch:
        x = np.asarray(x)
    name = dtype or (_TORCH_NAMES.get(str(x.dtype)) or _CAST_NAMES.get(str(x.dtype).replace("torch.", "")) if is_torch
                     else _NUMPY_NAMES.get(x.dtype.name) or _CAST_NAMES.get(x.dtype.name))
    if name not in CAST_CODES or to_dtype not in CAST_CODES:
        raise TypeError(f"cannot cast {name!r} to {to_dtype!r}")
    contiguous = x.is_contiguous() if is_torch else x.flags.c_contiguous
    if not contiguous:
        raise ValueError("cast needs a contiguous array")
    nbytes = x.numel() * x.element_size() if is_torch else x.nbytes
    n = int(count) if count is not None else nbytes * 8 // CAST_BITS[name]
    if n * CAST_BITS[name] > nbytes * 8:
        raise ValueError("count exceeds what the array holds")
    out_bytes = (n * CAST_BITS[to_dtype] + 7) // 8
    if out is None:
        if is_torch:
            import torch
            tdt = getattr(torch, _CAST_TORCH.get(to_dtype, "uint8"))
            shape = tuple(x.shape) if (CAST_BITS[to_dtype] >= 8 and count is None and CAST_BITS[name] >= 8) else (out_bytes * 8 // max(CAST_BITS[to_dtype], 8),)
            out = torch.empty(shape, dtype=tdt, device=x.device)
        else:
            ndt = _CAST_NUMPY.get(to_dtype, np.uint8)
            shape = x.shape if (CAST_BITS[to_dtype] >= 8 and count is None and CAST_BITS[name] >= 8) else (out_bytes * 8 // max(CAST_BITS[to_dtype], 8),)
            out = np.empty(shape, dtype=ndt)
    else:
        have = out.numel() * out.element_size() if _is_torch(out) else out.nbytes
        if have < out_bytes or not (out.is_contiguous() if _is_torch(out) else out.flags.c_contiguous):
            raise ValueError("out is too small or not contiguous")
    lib.nk_cast(_ptr(x), CAST_CODES[name], n, _ptr(out), CAST_CODES[to_dtype])
    check("cast")
    return out


def moments(x: Any, *, dtype: Optional[str] = None, count: Optional[int] = None, stride: Optional[int] = None) -> Tuple[Any, Any]:
    """(sum, sum of squares) of the values of a flat array - nk_reduce_moments_<dtype> (include/numkong/reduce.h:120-279).
    `count` values `stride` bytes apart (default: all of `x`, contiguous; sub-byte types count whole bytes). Python ints
    for integer types, floats otherwise (f32 precision for the 16-bit and smaller floats, as in the reference)."""
    is_torch = _is_torch(x)
    if not is_torch:
        x = np.asarray(x)
    name = dtype or (_TORCH_NAMES.get(str(x.dtype)) or _CAST_NAMES.get(str(x.dtype).replace("torch.", "")) if is_torch
                     else _NUMPY_NAMES.get(x.dtype.name) or _CAST_NAMES.get(x.dtype.name))
    if name not in CAST_CODES:
        raise TypeError(f"no moments kernel for {name!r}")
    if not (x.is_contiguous() if is_torch else x.flags.c_contiguous):
        raise ValueError("moments needs a contiguous array (use `stride` to skip values)")
    nbytes = x.numel() * x.element_size() if is_torch else x.nbytes
    unit = max(CAST_BITS[name] // 8, 1)
    step = int(stride) if stride is not None else unit
    per_unit = 8 // CAST_BITS[name] if CAST_BITS[name] < 8 else 1
    n = int(count) if count is not None else (nbytes // step) * per_unit
    units = (n + per_unit - 1) // per_unit
    if units and (units - 1) * step + unit > nbytes:
        raise ValueError("count and stride reach beyond the array")
    floats = name in ("f64", "f32", "f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2")
    narrow = floats and name not in ("f64", "f32")
    signed = name in ("i8", "i16", "i32", "i64", "i4")
    total = (ctypes.c_float if narrow else ctypes.c_double if floats else ctypes.c_int64 if signed else ctypes.c_uint64)()
    squares = (ctypes.c_float if narrow else ctypes.c_double if floats else ctypes.c_uint64)()
    getattr(lib, f"nk_reduce_moments_{name}")(_ptr(x), n, step, ctypes.byref(total), ctypes.byref(squares))
    check("moments")
    return total.value, squares.value


def maxsim_pack(vectors: Any, dtype: Optional[str] = None) -> MaxSimPackedMatrix:
    """Packs the token vectors of a query or a document. Mirrors nk.maxsim_pack."""
    v = _View(vectors, dtype)
    if v.dtype not in MAXSIM_DTYPES:
        raise TypeError(f"MaxSim supports {MAXSIM_DTYPES}, not {v.dtype!r}")
    size = MaxSimPackedMatrix.packed_size(v.rows, v.cols, v.dtype)
    buf = _alloc_bytes(size, v.is_cuda)
    getattr(lib, f"nk_maxsim_pack_{v.dtype}")(v.ptr, v.rows, v.cols, v.stride, _ptr(buf))
    check("maxsim_pack")
    return MaxSimPackedMatrix(buf, v.dtype, v.rows, v.cols)


def maxsim_packed(q: MaxSimPackedMatrix, d: MaxSimPackedMatrix) -> float:
    """sum_i min_j angular(q_i, d_j) with the argmax taken on the raw dot. Mirrors nk.maxsim_packed."""
    if not isinstance(q, MaxSimPackedMatrix) or not isinstance(d, MaxSimPackedMatrix):
        raise TypeError("both arguments must be MaxSimPackedMatrix objects")
    if q.dtype != d.dtype:
        raise TypeError("query and document were packed with different dtypes")
    if q.depth != d.depth:
        raise ValueError("query and document depths differ")
    res = (ctypes.c_double if q.dtype == "f32" else ctypes.c_float)()
    getattr(lib, f"nk_maxsim_packed_{q.dtype}")(_ptr(q.buffer), _ptr(d.buffer), q.width, d.width, q.depth, ctypes.addressof(res))
    check("maxsim_packed")
    return float(res.value)


def maxsim(q: Any, d: Any, dtype: Optional[str] = None) -> float:
    """Packs both sides and scores them. Mirrors nk.maxsim."""
    return maxsim_packed(maxsim_pack(q, dtype), maxsim_pack(d, dtype))


# ---- additions that the reference API cannot express (results too large to materialise) ----

def _topk_call(op: str, a: Any, packed: PackedMatrix, top: int, id_base: int, dtype: Optional[str]):
    v = _view_like(a, dtype, packed.dtype)
    if v.dtype not in ("f16", "bf16"):
        raise TypeError("top-k distances are available for f16 and bf16")
    if v.cols != packed.depth:
        raise ValueError("depth mismatch")
    if v.is_cuda:
        import torch
        dist = torch.empty((v.rows, top), dtype=torch.float32, device=v.obj.device)
        ids = torch.empty((v.rows, top), dtype=torch.int64, device=v.obj.device)
    else:
        dist = np.empty((v.rows, top), dtype=np.float32)
        ids = np.empty((v.rows, top), dtype=np.int64)
    getattr(lib, f"nkb_{op}_packed_topk_{v.dtype}")(v.ptr, _ptr(packed.buffer), v.rows, packed.width, v.cols, v.stride,
                                                    top, _ptr(dist), _ptr(ids), id_base)
    check(f"{op}_packed_topk")
    return dist, ids


def angulars_packed_topk(a: Any, packed: PackedMatrix, top: int, *, id_base: int = 0, dtype: Optional[str] = None):
    """The `top` nearest packed rows per row of `a` by angular distance, ascending: (distances, ids)."""
    return _topk_call("angulars", a, packed, top, id_base, dtype)


def euclideans_packed_topk(a: Any, packed: PackedMatrix, top: int, *, id_base: int = 0, dtype: Optional[str] = None):
    """The `top` nearest packed rows per row of `a` by Euclidean distance, ascending: (distances, ids)."""
    return _topk_call("euclideans", a, packed, top, id_base, dtype)


def maxsims_packed(q: MaxSimPackedMatrix, q_offsets: Any, d: MaxSimPackedMatrix, d_offsets: Any):
    """All-pairs MaxSim between many queries and many documents whose token vectors were packed
    together: `q_offsets` / `d_offsets` (int64, length count+1) delimit each query's / document's
    tokens. Returns the (queries x documents) matrix of the values maxsim_packed would return."""
    if q.dtype != d.dtype or q.dtype not in ("bf16", "f16"):
        raise TypeError("batched MaxSim is available for bf16 and f16")
    if q.depth != d.depth:
        raise ValueError("query and document depths differ")
    nq, nd = len(q_offsets) - 1, len(d_offsets) - 1
    cuda = d.is_cuda
    if cuda:
        import torch
        qo = torch.as_tensor(q_offsets, dtype=torch.int64, device="cuda").contiguous()
        do = torch.as_tensor(d_offsets, dtype=torch.int64, device="cuda").contiguous()
        scores = torch.empty((nq, nd), dtype=torch.float32, device="cuda")
    else:
        qo = np.ascontiguousarray(q_offsets, dtype=np.int64)
        do = np.ascontiguousarray(d_offsets, dtype=np.int64)
        scores = np.empty((nq, nd), dtype=np.float32)
    getattr(lib, f"nkb_maxsims_packed_{q.dtype}")(_ptr(q.buffer), _ptr(qo), nq, _ptr(d.buffer), _ptr(do), nd, q.depth,
                                                  _ptr(scores), nd * 4)
    check("maxsims_packed")
    return scores


def topk_smallest(scores: Any, top: int, *, id_base: int = 0):
    """Per row, the `top` smallest values (ascending, ties by lower column) and their columns + id_base."""
    if _is_torch(scores):
        import torch
        rows, cols = scores.shape
        vals = torch.empty((rows, top), dtype=torch.float32, device=scores.device)
        ids = torch.empty((rows, top), dtype=torch.int64, device=scores.device)
        stride = scores.stride(0) * 4
    else:
        scores = np.ascontiguousarray(scores, dtype=np.float32)
        rows, cols = scores.shape
        vals = np.empty((rows, top), dtype=np.float32)
        ids = np.empty((rows, top), dtype=np.int64)
        stride = scores.strides[0]
    lib.nkb_topk_smallest_f32(_ptr(scores), rows, cols, stride, top, id_base, _ptr(vals), _ptr(ids))
    check("topk_smallest")
    return vals, ids


def merge_topk(values: Any, ids: Any, top: Optional[int] = None):
    """Merges nearest-k lists of several shards: `values` (f32) and `ids` (i64) shaped [parts, rows, k], slots with id < 0
    empty. Returns ([rows, top], [rows, top]) ordered by (value, id) - the cross-shard step of a sharded search, on the device."""
    parts, rows, k = values.shape
    top = k if top is None else int(top)
    if top > k:
        raise ValueError("top may not exceed the length of the lists being merged")
    if _is_torch(values):
        import torch
        values, ids = values.to(torch.float32).contiguous(), ids.to(torch.int64).contiguous()
        out_v = torch.empty((rows, k), dtype=torch.float32, device=values.device)
        out_i = torch.empty((rows, k), dtype=torch.int64, device=values.device)
    else:
        values, ids = np.ascontiguousarray(values, dtype=np.float32), np.ascontiguousarray(ids, dtype=np.int64)
        out_v, out_i = np.empty((rows, k), dtype=np.float32), np.empty((rows, k), dtype=np.int64)
    lib.nkb_merge_topk(_ptr(values), _ptr(ids), parts, rows, k, _ptr(out_v), _ptr(out_i))
    check("merge_topk")
    return out_v[:, :top], out_i[:, :top]


def synchronize() -> int:
    """Waits for this thread's stream; returns the device error word (0 = healthy) and clears what it reports."""
    return int(lib.nkb_synchronize())


def set_wait_limit_ns(site: int, nanoseconds: int) -> None:
    """Limit of the kernels' bounded pipeline waits (nkb_set_wait_limit_ns): site 0 = all, nanoseconds 0 = the default 2 s."""
    lib.nkb_set_wait_limit_ns(int(site), int(nanoseconds))


def set_stream(cuda_stream: int) -> None:
    lib.nkb_set_stream(ctypes.c_void_p(cuda_stream))


def set_accumulation_span(stages: int) -> None:
    """Stages (128 bytes of depth each) the tensor cores accumulate before the partial sums are added with round-to-nearest;
    0 = automatic. Shorter spans are slower and more accurate for bf16 / f16 products (nkb_set_accumulation_span)."""
    lib.nkb_set_accumulation_span(int(stages))


def launch_count() -> int:
    return int(lib.nkb_launch_count())
