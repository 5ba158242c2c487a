"""Bulk type conversion on the device (nk_cast) against the committed reference vectors and the CPU oracle: every
defined pair of the nineteen real scalar types, host and device buffers, tails, unaligned buffers, infinities and NaN,
and the quantise-then-pack chain the conversion exists for."""
import os

import numpy as np
import pytest
import torch

import numkong_b200 as nk
import oracle
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "cast_path.npz"))
TYPES = ["f64", "f32", "f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2", "i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "i4", "u4", "u1"]
SIGNED = ("i8", "i16", "i32", "i64", "i4")


def defined(a, b):
    return not ((a == "u1" and b in SIGNED) or (a in SIGNED and b in ("u4", "u1")))


def device_bytes(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x).view(np.uint8).copy()).cuda()


def run_on_device(x: np.ndarray, a: str, b: str, n: int) -> np.ndarray:
    out = torch.zeros((n * oracle.CAST_BITS[b] + 7) // 8, dtype=torch.uint8, device="cuda")
    nk.cast(device_bytes(x), b, dtype=a, count=n, out=out)
    assert nk.synchronize() == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("source", TYPES)
def test_cast_matches_reference_vectors(source):
    x = GOLDEN["from_" + source]
    for target in TYPES:
        if target == source or not defined(source, target):
            continue
        want = GOLDEN[f"{source}_to_{target}"].view(np.uint8)
        assert np.array_equal(run_on_device(x, source, target, 136), want), (source, target, "device")
        host = nk.cast(x, target, dtype=source, count=136)
        assert np.array_equal(np.ascontiguousarray(host).view(np.uint8).ravel()[:want.size], want), (source, target, "host")


@pytest.mark.parametrize("source", TYPES)
def test_cast_large_with_tails(source):
    """A hundred thousand values and a ragged count: whole result bytes must match the oracle; the last byte of a
    partial sub-byte batch is compared on the bits that hold converted values."""
    for n in (100_000, 100_003):
        x = syn.cast_samples(source, n, 8000 + TYPES.index(source))
        for target in TYPES:
            if target == source or not defined(source, target):
                continue
            want = oracle.cast(x, source, target, n).view(np.uint8)
            got = run_on_device(x, source, target, n)
            assert got.size == want.size
            bits = oracle.CAST_BITS[target]
            if bits < 8 and (n * bits) % 8:
                keep = 0xFF & ~((1 << (8 - (n * bits) % 8)) - 1)       # converted values sit in the high bits of the last byte
                assert (got[-1] & keep) == (want[-1] & keep), (source, target, n)
                got, want = got[:-1], want[:-1]
            assert np.array_equal(got, want), (source, target, n)


def test_cast_infinities_and_nan():
    x = np.array([np.inf, -np.inf, np.nan, -np.nan, 1.0, -1.0, 0.0, 70000.0, np.nan, np.inf], dtype=np.float32)
    for source in ("f32", "f64"):
        xs = x.astype(np.float64) if source == "f64" else x
        for target in TYPES:
            if target == source or target in ("i4", "u4"):
                continue                                     # NaN to a nibble is left to the C cast in the reference
            want = oracle.cast(xs, source, target, x.size)
            got = run_on_device(xs, source, target, x.size).view(want.dtype)
            if target in ("f64", "f32", "f16", "bf16"):
                decoded = lambda v: v.astype(np.float64) if target in ("f64", "f32") else oracle.decode(v.view(np.uint16).reshape(1, -1), target).ravel()
                g, w = decoded(got), decoded(want)
                assert np.array_equal(np.isnan(g), np.isnan(w)) and np.array_equal(g[~np.isnan(g)], w[~np.isnan(w)]), (source, target)
            else:
                assert np.array_equal(got, want), (source, target)
    assert list(run_on_device(x, "f32", "e4m3", 4)) == [0x7E, 0xFE, 0x7F, 0xFF]      # saturate, keep NaN
    assert list(run_on_device(x, "f32", "e5m2", 4)) == [0x7C, 0xFC, 0x7D, 0xFD]      # infinities exist
    assert list(run_on_device(x, "f32", "e2m3", 4)) == [0x1F, 0x3F, 0x1F, 0x3F]      # no infinity, no NaN: largest value
    assert list(run_on_device(x, "f32", "i8", 4).view(np.int8)) == [127, -128, 0, 0]


def test_cast_unaligned_buffers_and_torch_types():
    x = torch.randn(10_001, device="cuda") * 50
    want = oracle.cast(x[1:].cpu().numpy(), "f32", "bf16")
    got = nk.cast(x[1:].contiguous(), "bf16")
    assert got.dtype == torch.bfloat16 and np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want)
    shifted = torch.empty(10_001 * 4 + 4, dtype=torch.uint8, device="cuda")
    src = shifted[3:3 + 10_000 * 4]                                                 # source starts 3 bytes off
    src.copy_(x[1:].contiguous().view(torch.uint8))
    out = torch.empty(10_000 * 2 + 1, dtype=torch.uint8, device="cuda")
    nk.cast(src, "bf16", dtype="f32", count=10_000, out=out[1:])                    # result starts 1 byte off
    assert nk.synchronize() == 0
    assert np.array_equal(out[1:].cpu().numpy().view(np.uint16), want)
    assert torch.equal(got.float(), x[1:].to(torch.bfloat16).float())
    e = nk.cast(x, "e4m3")
    assert e.dtype == torch.float8_e4m3fn and torch.equal(e.float(), x.clamp(-448, 448).to(torch.float8_e4m3fn).float())
    h = nk.cast(x.double(), "f16")
    assert h.dtype == torch.float16 and torch.equal(h, x.double().float().half())
    same = nk.cast(x, "f32")
    assert torch.equal(same, x) and same.data_ptr() != x.data_ptr()


def test_cast_refuses_undefined_pairs():
    for a, b in (("u1", "i8"), ("i8", "u4"), ("i32", "u1"), ("i4", "u4")):
        with pytest.raises(RuntimeError):
            nk.cast(np.zeros(64, dtype=np.uint8), b, dtype=a, count=8)
    with pytest.raises(TypeError):
        nk.cast(np.zeros(4, dtype=np.complex64), "f32")
    with pytest.raises(ValueError):
        nk.cast(np.zeros(4, dtype=np.float32), "f16", count=5)


def test_quantise_then_pack_chain():
    """f32 source -> e4m3 on the device -> packed product: the same codes and the same product as quantising on the CPU."""
    rng = np.random.default_rng(9)
    a32, b32 = rng.standard_normal((300, 256)).astype(np.float32), rng.standard_normal((500, 256)).astype(np.float32)
    ta, tb = torch.from_numpy(a32).cuda(), torch.from_numpy(b32).cuda()
    qa, qb = nk.cast(ta, "e4m3"), nk.cast(tb, "e4m3")
    assert qa.shape == ta.shape
    ha, hb = oracle.cast(a32, "f32", "e4m3").reshape(300, 256), oracle.cast(b32, "f32", "e4m3").reshape(500, 256)
    assert np.array_equal(qa.view(torch.uint8).cpu().numpy(), ha) and np.array_equal(ha, syn.encode(a32, "e4m3"))
    c = nk.dots_packed(qa, nk.dots_pack(qb))
    assert nk.synchronize() == 0
    exact = oracle.exact_dots_f64(ha, hb, "e4m3")
    scale = np.abs(oracle.decode(ha, "e4m3").astype(np.float64)) @ np.abs(oracle.decode(hb, "e4m3").astype(np.float64)).T
    assert np.max(np.abs(c.cpu().numpy() - exact) / scale) <= 1e-7


def test_cast_sweep_of_the_f32_bit_space():
    """Every 4099th f32 bit pattern (subnormals, infinities and NaN included) to the narrow types: the kernel compiled for
    the pair (aligned buffers; hardware fp8 / fp6 conversions) and the general kernel (a source 4 bytes off a 16-byte
    boundary) must both give the oracle's bytes; for f16 / bf16 a NaN only has to stay a NaN."""
    bits = np.arange(0, 2 ** 32, 4099, dtype=np.uint64).astype(np.uint32)
    n = bits.size
    store = torch.zeros(n * 4 + 16, dtype=torch.uint8, device="cuda")
    aligned, shifted = store[:n * 4], torch.zeros(n * 4 + 16, dtype=torch.uint8, device="cuda")[4:4 + n * 4]
    aligned.copy_(torch.from_numpy(bits.view(np.uint8)).cuda())
    shifted.copy_(aligned)
    nan = np.isnan(bits.view(np.float32))
    for target in ("e4m3", "e5m2", "e2m3", "e3m2", "f16", "bf16", "i8", "u8"):
        want = oracle.cast(bits.view(np.float32), "f32", target)
        for source in (aligned, shifted):
            before = nk.launch_count()
            got = nk.cast(source, target, dtype="f32", count=n)
            assert nk.synchronize() == 0 and nk.launch_count() == before + 1
            got = got.view(torch.uint8).cpu().numpy().view(want.dtype)
            if target in ("f16", "bf16"):
                assert np.array_equal(got[~nan], want[~nan]), target
                assert np.all(np.isnan(oracle.decode(got[nan].view(np.uint16).reshape(1, -1), target))), target
            else:
                assert np.array_equal(got, want), target
