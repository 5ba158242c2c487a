"""ctypes binding of libnumkong_b200.so (the C ABI declared in include/numkong_b200.h).

The library is the product; there is no fallback. If it has not been built, or cannot be
loaded, importing this module raises with the build command to run.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libnumkong_b200.so"

# name -> numerically nk_dtype_t (include/numkong/types.h:923-953 of the reference)
DTYPE_CODES = {
    "i8": 1 << 2, "u8": 1 << 6, "f32": 1 << 11, "f16": 1 << 12, "bf16": 1 << 13,
    "e4m3": 1 << 14, "e5m2": 1 << 15, "e2m3": 1 << 18, "e3m2": 1 << 19, "i4": 1 << 16, "u4": 1 << 17, "u1": 1 << 1, "f64": 1 << 10,
}
DTYPE_BYTES = {"i8": 1, "u8": 1, "f32": 4, "f16": 2, "bf16": 2, "e4m3": 1, "e5m2": 1, "e2m3": 1, "e3m2": 1, "i4": 1, "u4": 1, "u1": 1, "f64": 8}
# Logical dimensions per storage element: 4-bit types hold two values per byte and `depth` counts values, as in the
# reference's binding (python/matrix.c:400-401 multiplies the byte width by nk_dimensions_per_value).
DIMENSIONS_PER_VALUE = {"i4": 2, "u4": 2, "u1": 8}
SET_DTYPES = ("u1",)  # dots (AND-popcount), Hamming and Jaccard instead of angular / Euclidean
PACKED_DTYPES = tuple(DTYPE_CODES)
MAXSIM_DTYPES = ("bf16", "f16", "f32")


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python numkong_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_LOCAL)
    sz, vp = ctypes.c_uint64, ctypes.c_void_p
    for t in PACKED_DTYPES:
        f = getattr(lib, f"nk_dots_packed_size_{t}")
        f.restype, f.argtypes = sz, [sz, sz]
        f = getattr(lib, f"nk_dots_pack_{t}")
        f.restype, f.argtypes = None, [vp, sz, sz, sz, vp]
        for op in (("dots", "hammings", "jaccards") if t in SET_DTYPES else ("dots", "angulars", "euclideans")):
            f = getattr(lib, f"nk_{op}_packed_{t}")
            f.restype, f.argtypes = None, [vp, vp, vp, sz, sz, sz, sz, sz]
            f = getattr(lib, f"nk_{op}_symmetric_{t}")
            f.restype, f.argtypes = None, [vp, sz, sz, sz, vp, sz, sz, sz]
    for t in MAXSIM_DTYPES:
        f = getattr(lib, f"nk_maxsim_packed_size_{t}")
        f.restype, f.argtypes = sz, [sz, sz]
        f = getattr(lib, f"nk_maxsim_pack_{t}")
        f.restype, f.argtypes = None, [vp, sz, sz, sz, vp]
        f = getattr(lib, f"nk_maxsim_packed_{t}")
        f.restype, f.argtypes = None, [vp, vp, sz, sz, sz, vp]
    lib.nk_find_kernel_punned.restype = None
    lib.nk_find_kernel_punned.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_uint64,
                                          ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_uint64)]
    lib.nk_capabilities.restype, lib.nk_capabilities.argtypes = ctypes.c_uint64, []
    lib.nk_configure_thread.restype, lib.nk_configure_thread.argtypes = ctypes.c_int, [ctypes.c_uint64]
    lib.nkb_last_error.restype, lib.nkb_last_error.argtypes = ctypes.c_char_p, []
    lib.nkb_set_stream.restype, lib.nkb_set_stream.argtypes = None, [vp]
    lib.nkb_synchronize.restype, lib.nkb_synchronize.argtypes = ctypes.c_uint32, []
    lib.nkb_launch_count.restype, lib.nkb_launch_count.argtypes = ctypes.c_uint64, []
    lib.nkb_set_gemm_variant.restype, lib.nkb_set_gemm_variant.argtypes = None, [ctypes.c_int]
    lib.nkb_set_accumulation_span.restype, lib.nkb_set_accumulation_span.argtypes = None, [ctypes.c_int]
    lib.nkb_release_caches.restype, lib.nkb_release_caches.argtypes = None, []
    lib.nkb_set_fp6_native.restype, lib.nkb_set_fp6_native.argtypes = None, [ctypes.c_int]
    lib.nkb_set_topk_panel_rows.restype, lib.nkb_set_topk_panel_rows.argtypes = None, [sz]
    lib.nkb_set_topk_filter.restype, lib.nkb_set_topk_filter.argtypes = None, [ctypes.c_int]
    lib.nkb_topk_filter_fallbacks.restype, lib.nkb_topk_filter_fallbacks.argtypes = sz, []
    for t in ("f16", "bf16"):
        for op in ("angulars", "euclideans"):
            f = getattr(lib, f"nkb_{op}_packed_topk_{t}")
            f.restype, f.argtypes = None, [vp, vp, sz, sz, sz, sz, sz, vp, vp, sz]
    for t in ("bf16", "f16"):
        f = getattr(lib, f"nkb_maxsims_packed_{t}")
        f.restype, f.argtypes = None, [vp, vp, sz, vp, vp, sz, sz, vp, sz]
    lib.nk_cast.restype, lib.nk_cast.argtypes = None, [vp, ctypes.c_uint32, sz, vp, ctypes.c_uint32]
    for t in ("f64", "f32", "f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2", "i8", "u8", "i16", "u16", "i32", "u32", "i64", "u64", "i4", "u4", "u1"):
        f = getattr(lib, f"nk_reduce_moments_{t}")
        f.restype, f.argtypes = None, [vp, sz, sz, vp, vp]
    lib.nk_dots_compact_bf16.restype, lib.nk_dots_compact_bf16.argtypes = None, [vp, sz, sz, sz]
    lib.nk_dots_compact_i8.restype, lib.nk_dots_compact_i8.argtypes = None, [vp, sz, sz, sz, vp, vp]
    lib.nkb_topk_smallest_f32.restype = None
    lib.nkb_topk_smallest_f32.argtypes = [vp, sz, sz, sz, sz, sz, vp, vp]
    lib.nkb_merge_topk.restype, lib.nkb_merge_topk.argtypes = None, [vp, vp, sz, sz, sz, vp, vp]
    lib.nkb_dots_packed_columns.restype = None
    lib.nkb_dots_packed_columns.argtypes = [ctypes.c_uint32, vp, vp, vp, sz, sz, sz, sz, sz, sz, sz]
    lib.nkb_angulars_packed_noalloc.restype = ctypes.c_int
    lib.nkb_angulars_packed_noalloc.argtypes = [ctypes.c_uint32, vp, vp, vp, sz, sz, sz, sz, sz]
    lib.nkb_set_wait_limit_ns.restype, lib.nkb_set_wait_limit_ns.argtypes = None, [ctypes.c_int, sz]
    lib.nkb_test_set_error_word.restype, lib.nkb_test_set_error_word.argtypes = ctypes.c_int, [ctypes.c_int, ctypes.c_uint32]
    lib.nkb_cached_blob_count.restype, lib.nkb_cached_blob_count.argtypes = sz, []
    lib.nkb_set_sm_budget.restype, lib.nkb_set_sm_budget.argtypes = None, [ctypes.c_int]
    lib.nkb_multicast_store.restype, lib.nkb_multicast_store.argtypes = ctypes.c_int, [vp, vp, sz, ctypes.c_int]
    lib.nkb_peer_barrier.restype = ctypes.c_int
    lib.nkb_peer_barrier.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_uint32]
    return lib


lib = _load()


def last_error() -> str:
    return lib.nkb_last_error().decode()


def check(what: str) -> None:
    """Raises if the last call of this thread recorded an error."""
    msg = last_error()
    if msg:
        raise RuntimeError(f"{what}: {msg}")
