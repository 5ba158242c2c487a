"""Sum and sum of squares on the device (nk_reduce_moments_<t>): integers bit for bit against the committed reference
values and the CPU oracle (saturation rules included), floats against the exactly rounded result within one unit in
the last place of the result type; contiguous, strided, unaligned, host and device data."""
import math
import os

import numpy as np
import pytest
import torch

import numkong_b200 as nk
import oracle
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "moments_path.npz"))
FLOATS = ["f64", "f32", "f16", "bf16", "e4m3", "e5m2", "e2m3", "e3m2"]
INTS = ["i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "i4", "u4", "u1"]


def values_of(x, dtype):
    if dtype in ("f64", "f32"):
        return x.astype(np.float64)
    return oracle.decode(x.reshape(1, -1), dtype).ravel().astype(np.float64)


def check_float(got, x, dtype):
    v = values_of(x, dtype)
    exact_sum, exact_squares = math.fsum(v), math.fsum(v * v)      # squares of <= 24-bit values are exact in f64
    ulp = 2.0 ** -52 if dtype in ("f64", "f32") else 2.0 ** -23
    magnitude = math.fsum(np.abs(v))
    assert abs(got[0] - exact_sum) <= ulp * abs(exact_sum) + 2.0 ** -49 * magnitude, (dtype, got[0], exact_sum)
    assert abs(got[1] - exact_squares) <= (4 if dtype == "f64" else 1) * ulp * exact_squares, (dtype, got[1], exact_squares)


def on_device(x):
    return torch.from_numpy(np.ascontiguousarray(x).view(np.uint8).copy()).cuda()


@pytest.mark.parametrize("dtype", INTS)
def test_integer_moments_match_reference_values(dtype):
    x = GOLDEN["from_" + dtype]
    per_unit = 8 // oracle.CAST_BITS[dtype] if oracle.CAST_BITS[dtype] < 8 else 1
    unit = max(oracle.CAST_BITS[dtype] // 8, 1)
    for source in (x, on_device(x)):
        got = nk.moments(source, dtype=dtype, count=1000)
        assert got == (int(GOLDEN[dtype + "_all_sum"][0]), int(GOLDEN[dtype + "_all_sumsq"][0])), dtype
        got = nk.moments(source, dtype=dtype, count=333 if per_unit == 1 else 40 * per_unit, stride=3 * unit)
        assert got == (int(GOLDEN[dtype + "_strided_sum"][0]), int(GOLDEN[dtype + "_strided_sumsq"][0])), (dtype, "strided")


def test_integer_saturation_cases():
    for key in ("i32", "u32", "i64", "u64", "i64_negative"):
        x = GOLDEN["big_" + key]
        want = (int(GOLDEN[f"big_{key}_sum"][0]), int(GOLDEN[f"big_{key}_sumsq"][0]))
        assert nk.moments(x) == want and nk.moments(on_device(x), dtype=key.split("_")[0]) == want, key
    # enough u32 values to overflow the 64-bit sum of squares inside single threads and across blocks
    x = torch.full((1 << 22,), 2 ** 32 - 1, dtype=torch.int64, device="cuda").to(torch.uint32)
    assert nk.moments(x) == ((2 ** 32 - 1) << 22, 2 ** 64 - 1)
    y = torch.full((1 << 22,), -2 ** 62, dtype=torch.int64, device="cuda")
    assert nk.moments(y) == (-2 ** 63, 2 ** 64 - 1)


@pytest.mark.parametrize("dtype", INTS)
def test_integer_moments_large_and_unaligned(dtype):
    n = 3_000_017
    x = syn.cast_samples(dtype, n, 40 + INTS.index(dtype))
    per_unit = 8 // oracle.CAST_BITS[dtype] if oracle.CAST_BITS[dtype] < 8 else 1
    count = (x.nbytes // max(oracle.CAST_BITS[dtype] // 8, 1)) * per_unit
    want = tuple(int(v) for v in oracle.moments(x, dtype, count))
    dev = on_device(x)
    assert nk.moments(dev, dtype=dtype, count=count) == want
    unit = max(oracle.CAST_BITS[dtype] // 8, 1)
    shifted = torch.empty(dev.numel() + 64, dtype=torch.uint8, device="cuda")[unit * 3:unit * 3 + dev.numel()]   # off a 16-byte boundary
    shifted.copy_(dev)
    assert nk.moments(shifted, dtype=dtype, count=count) == want
    assert nk.moments(x, dtype=dtype, count=count) == want                                                    # host data


@pytest.mark.parametrize("dtype", FLOATS)
def test_float_moments(dtype):
    x = GOLDEN["from_" + dtype]
    reference = (float(GOLDEN[dtype + "_all_sum"][0]), float(GOLDEN[dtype + "_all_sumsq"][0]))
    for source in (x, on_device(x)):
        got = nk.moments(source, dtype=dtype)
        check_float(got, x, dtype)
        check_float(reference, x, dtype)                          # the reference's compensated sums meet the same bound
    big = syn.moments_samples(dtype, 2_000_003, 70 + FLOATS.index(dtype))
    got = nk.moments(on_device(big), dtype=dtype)
    check_float(got, big, dtype)
    assert got == nk.moments(on_device(big), dtype=dtype)         # deterministic: fixed combination order
    unit = big.itemsize
    strided = nk.moments(on_device(big), dtype=dtype, count=big.size // 5, stride=5 * unit)
    check_float(strided, big[::5][:big.size // 5], dtype)


def test_moments_empty_and_results_on_the_device():
    assert nk.moments(np.zeros(0, dtype=np.float32)) == (0.0, 0.0)
    assert nk.moments(np.zeros(0, dtype=np.int8)) == (0, 0)
    import ctypes
    from numkong_b200 import _lib
    x = torch.arange(1, 1001, dtype=torch.float32, device="cuda")
    out = torch.zeros(2, dtype=torch.float64, device="cuda")
    _lib.lib.nk_reduce_moments_f32(x.data_ptr(), 1000, 4, out.data_ptr(), out.data_ptr() + 8)
    assert nk.synchronize() == 0 and out.tolist() == [500500.0, 333833500.0]
    with pytest.raises(ValueError):
        nk.moments(np.zeros(10, dtype=np.float32), count=11)


def test_moments_feed_a_quantisation_scale():
    """The use the reference names: statistics of an f32 source choose the scale, the cast quantises, pack follows."""
    rng = np.random.default_rng(3)
    x = torch.from_numpy((rng.standard_normal((512, 256)) * 3).astype(np.float32)).cuda()
    total, squares = nk.moments(x.view(-1))
    rms = math.sqrt(squares / x.numel())
    assert abs(total - float(x.double().sum())) <= 1e-9 * float(x.double().abs().sum())
    assert abs(rms - float(x.double().pow(2).mean().sqrt())) < 1e-9
    q = nk.cast((x * (32.0 / rms)).contiguous(), "i8")
    assert q.dtype == torch.int8 and q.shape == x.shape
    c = nk.dots_packed(q, nk.dots_pack(q))
    assert nk.synchronize() == 0
    assert torch.equal(c.cpu(), (q.cpu().to(torch.int32) @ q.cpu().to(torch.int32).T))
