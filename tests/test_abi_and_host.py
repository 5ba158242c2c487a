"""CPU-only checks of the drop-in boundary: the shared library loads, exports every symbol the header
declares, answers the pure (no-GPU) entry points, and the Python mirror rejects bad arguments the way
the reference's binding does. No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

import numkong_b200 as nk
from numkong_b200 import _lib, synthetic as syn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "numkong_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    names = set(re.findall(r"NKB_API[^;(]*?\b(nkb?_[a-z0-9_]+)\s*\(", text))
    for macro, pattern in (("NKB_DECLARE_PACKED_FAMILY", ["nk_dots_packed_size_{}", "nk_dots_pack_{}", "nk_dots_packed_{}",
                                                          "nk_angulars_packed_{}", "nk_euclideans_packed_{}"]),
                           ("NKB_DECLARE_SYMMETRIC_FAMILY", ["nk_dots_symmetric_{}", "nk_angulars_symmetric_{}", "nk_euclideans_symmetric_{}"]),
                           ("NKB_DECLARE_MAXSIM_FAMILY", ["nk_maxsim_packed_size_{}", "nk_maxsim_pack_{}", "nk_maxsim_packed_{}"]),
                           ("NKB_DECLARE_TOPK_FAMILY", ["nkb_angulars_packed_topk_{}", "nkb_euclideans_packed_topk_{}"]),
                           ("NKB_DECLARE_MAXSIMS_FAMILY", ["nkb_maxsims_packed_{}"])):
        for t in re.findall(macro + r"\((\w+)\)", text):
            if t != "T":
                names.update(p.format(t) for p in pattern)
    return sorted(n for n in names if "##" not in n)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    names = declared_symbols()
    assert len(names) >= 11 * 8 + 8 + 3 * 3 + 8
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_packed_size_is_pure_and_bounds_the_payload():
    for dt in nk.PACKED_DTYPES:
        eb = nk.DTYPE_BYTES[dt]
        for (n, k) in [(1, 1), (5, 3), (256, 128), (257, 129), (2048, 2048), (10_000_000, 768)]:
            size = nk.PackedMatrix.packed_size(n, k, dt)
            assert size == nk.PackedMatrix.packed_size(n, k, dt)
            assert size >= 128 + n * k * eb + n * 4
            assert size % 128 == 0
    assert nk.PackedMatrix.packed_size(2048, 2048, "i8") == 128 + 2048 * 2048 + 2048 * 4
    for dt in nk.MAXSIM_DTYPES:
        assert nk.MaxSimPackedMatrix.packed_size(180, 128, dt) >= 180 * 128 * nk.DTYPE_BYTES[dt]
    with pytest.raises(LookupError):
        nk.PackedMatrix.packed_size(4, 4, "f64c")


def test_find_kernel_punned_contract():
    """c/numkong.c:848-913: known (kind, dtype) -> entry point + non-zero capability; unknown -> NULL + 0."""
    fn, cap = ctypes.c_void_p(), ctypes.c_uint64()
    lib = _lib.lib
    for dt in nk.PACKED_DTYPES:
        # bit vectors have set distances (Hamming 'M'/'Y', Jaccard 'p'/'Z') where the others have angular / Euclidean
        for kind in ("PQGyMYpZ" if dt == "u1" else "PQGNEynD"):
            lib.nk_find_kernel_punned(ord(kind), nk.DTYPE_CODES[dt], (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))
            assert fn.value and cap.value == 1 << 40, (kind, dt)
    lib.nk_find_kernel_punned(ord("N"), nk.DTYPE_CODES["u1"], (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))
    assert not fn.value and cap.value == 0  # no angular distance between bit vectors
    lib.nk_find_kernel_punned(ord("G"), nk.DTYPE_CODES["i8"], (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))
    direct = ctypes.cast(lib.nk_dots_packed_i8, ctypes.c_void_p).value
    assert fn.value == direct
    for kind in "LlT":
        for dt in nk.MAXSIM_DTYPES:
            lib.nk_find_kernel_punned(ord(kind), nk.DTYPE_CODES[dt], 1 << 40, ctypes.byref(fn), ctypes.byref(cap))
            assert fn.value and cap.value
    lib.nk_find_kernel_punned(ord("T"), nk.DTYPE_CODES["i8"], (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))
    assert not fn.value and cap.value == 0
    lib.nk_find_kernel_punned(ord("G"), 1 << 20, (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))  # a complex type: not on this path
    assert not fn.value and cap.value == 0
    lib.nk_find_kernel_punned(ord("G"), nk.DTYPE_CODES["i8"], 0x3, ctypes.byref(fn), ctypes.byref(cap))  # capability masked out
    assert not fn.value and cap.value == 0
    assert lib.nk_configure_thread(1 << 40) == 1
    # moments under 'R' for all nineteen element types, the bulk conversion under '-' with the "unknown" type 0
    # (include/numkong/capabilities.h:225,251; c/numkong.c:897)
    moment_codes = dict(nk.DTYPE_CODES, i16=1 << 3, i32=1 << 4, i64=1 << 5, u16=1 << 7, u32=1 << 8, u64=1 << 9)
    for name in ("f64", "f32", "f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2", "i8", "u8", "i16", "u16", "i32", "u32", "i64", "u64", "i4", "u4", "u1"):
        lib.nk_find_kernel_punned(ord("R"), moment_codes[name], 1 << 40, ctypes.byref(fn), ctypes.byref(cap))
        assert fn.value == ctypes.cast(getattr(lib, f"nk_reduce_moments_{name}"), ctypes.c_void_p).value and cap.value == 1 << 40, name
    lib.nk_find_kernel_punned(ord("-"), 0, (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))
    assert fn.value == ctypes.cast(lib.nk_cast, ctypes.c_void_p).value and cap.value == 1 << 40
    lib.nk_find_kernel_punned(ord("-"), nk.DTYPE_CODES["f32"], (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))
    assert not fn.value and cap.value == 0   # the conversion is looked up without an element type
    lib.nk_find_kernel_punned(ord("R"), 1 << 21, (1 << 64) - 1, ctypes.byref(fn), ctypes.byref(cap))
    assert not fn.value and cap.value == 0   # no moments of complex types


def test_python_mirror_argument_checks():
    with pytest.raises(ValueError):
        nk.dots_pack(np.zeros(8, dtype=np.int8))                      # not 2-D
    with pytest.raises(TypeError):
        nk.dots_pack(np.zeros((2, 2), dtype=np.complex128))           # complex types are not on this path
    with pytest.raises(TypeError):
        nk.dots_pack(np.zeros((2, 2), dtype=np.uint8), dtype="bf16")  # wrong storage width
    with pytest.raises(ValueError):
        nk.dots_pack(np.zeros((4, 4), dtype=np.int8).T[:, ::2])       # rows not contiguous
    fake = nk.PackedMatrix(np.zeros(256, dtype=np.uint8), "i8", 2, 4)
    with pytest.raises(ValueError):
        nk.dots_packed(np.zeros((2, 5), dtype=np.int8), fake)         # depth mismatch
    with pytest.raises(TypeError):
        nk.dots_packed(np.zeros((2, 4), dtype=np.uint8), fake)        # dtype mismatch
    with pytest.raises(TypeError):
        nk.dots_packed(np.zeros((2, 4), dtype=np.int8), np.zeros(4))  # not a PackedMatrix
    ms = nk.MaxSimPackedMatrix(np.zeros(256, dtype=np.uint8), "bf16", 2, 4)
    with pytest.raises(TypeError):
        nk.dots_packed(np.zeros((2, 4), dtype=np.int8), ms)           # packer family mix-up (test_cross.py:454-467)
    with pytest.raises(ValueError):
        nk.maxsim_packed(ms, nk.MaxSimPackedMatrix(np.zeros(256, dtype=np.uint8), "bf16", 2, 8))  # depth mismatch
    with pytest.raises(TypeError):
        nk.maxsim_pack(np.zeros((2, 4), dtype=np.int8))               # MaxSim: bf16 / f16 / f32 only


def test_synthetic_encoders_round_trip():
    import oracle
    rng = np.random.default_rng(1)
    x = rng.standard_normal((16, 64)).astype(np.float32)
    for dt in ("bf16", "f16", "e4m3", "e5m2", "e2m3", "e3m2"):
        once = oracle.decode(syn.encode(x, dt), dt)
        assert np.array_equal(syn.encode(once, dt), syn.encode(x, dt))   # encoding is idempotent on representable values
        assert np.all(np.isfinite(once))
    for dt in ("e4m3", "e5m2", "e2m3", "e3m2"):
        codes = syn.finite_codes_matrix(8, 256, dt, 3)
        assert np.all(np.isfinite(oracle.decode(codes, dt)))
        assert np.array_equal(syn.encode(oracle.decode(codes, dt), dt) & 0x7F if dt[1] in "45" else syn.encode(oracle.decode(codes, dt), dt) & 0x1F,
                              codes & 0x7F if dt[1] in "45" else codes & 0x1F)
