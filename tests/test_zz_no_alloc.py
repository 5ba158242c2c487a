"""The allocation-free angular-distance entry point against the regular one.

Some users of this library cannot let it call cudaMalloc: they run inside a stream capture, serve requests
under a latency budget, or live inside an application whose own pool allocator has claimed the whole device
heap. For them nkb_angulars_packed_noalloc keeps its scratch (row norms of A, the error word) in fixed device
arrays. This file is collected last on purpose: if it fails, a run that stops at the first failure has already
executed every other test. It must pass alone in a fresh process and after all the others.
"""
import ctypes

import numpy as np
import pytest

import numkong_b200 as nk
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def _call_noalloc(dtype, ta, packed, out):
    fn = nk.lib.nkb_angulars_packed_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_uint32] + [ctypes.c_void_p] * 3 + [ctypes.c_uint64] * 5
    return fn(nk.DTYPE_CODES[dtype], ta.data_ptr(), packed.buffer.data_ptr(), out.data_ptr(), ta.shape[0], packed.width,
              ta.shape[1], ta.stride(0) * ta.element_size(), out.stride(0) * 4)


@pytest.mark.parametrize("dtype", ["bf16", "i8", "e4m3"])
def test_noalloc_matches_regular_entry_point_twice_in_a_row(dtype):
    import torch
    store = {1: (np.uint8, torch.uint8), 2: (np.int16, torch.int16)}[nk.DTYPE_BYTES[dtype]]
    outs = []
    # Two different problems back to back: the second call reuses (and must fully rewrite) the fixed scratch.
    for seed, (m, n, k) in enumerate([(300, 515, 768), (129, 1000, 160)]):
        a, b = syn.normal_matrix(m, k, dtype, 900 + seed), syn.normal_matrix(n, k, dtype, 950 + seed)
        ta, tb = torch.from_numpy(a.view(store[0])).cuda(), torch.from_numpy(b.view(store[0])).cuda()
        packed = nk.dots_pack(tb, dtype)
        want = nk.angulars_packed(ta, packed, dtype=dtype)
        got = torch.full((m, n), -1.0, dtype=torch.float32, device="cuda")
        assert _call_noalloc(dtype, ta, packed, got) == 0, nk.last_error()
        assert nk.synchronize() == 0
        # Same kernels, same inputs: the tolerance of the distance tests (5e-7 absolute) is met with margin.
        assert torch.max(torch.abs(got - want)).item() <= 5e-7
        outs.append(got)
    assert outs[0].shape != outs[1].shape


def test_noalloc_refuses_what_it_cannot_do_without_allocating():
    import torch
    a = torch.zeros((4, 64), dtype=torch.int16, device="cuda")
    packed = nk.dots_pack(torch.zeros((8, 64), dtype=torch.int16, device="cuda"), "bf16")
    out = torch.full((4, 8), 7.0, dtype=torch.float32, device="cuda")
    fn = nk.lib.nkb_angulars_packed_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_uint32] + [ctypes.c_void_p] * 3 + [ctypes.c_uint64] * 5
    code = nk.DTYPE_CODES["bf16"]
    too_many = 65536 + 1
    assert fn(code, a.data_ptr(), packed.buffer.data_ptr(), out.data_ptr(), too_many, 8, 64, 128, 32) != 0
    assert "65536" in nk.last_error()
    host = np.zeros((4, 64), dtype=np.int16)
    assert fn(code, host.ctypes.data, packed.buffer.data_ptr(), out.data_ptr(), 4, 8, 64, 128, 32) != 0
    assert "device" in nk.last_error()
    assert fn(code, a.data_ptr() + 2, packed.buffer.data_ptr(), out.data_ptr(), 4, 8, 63, 128, 32) != 0   # misaligned A
    assert fn(nk.DTYPE_CODES["f32"], a.data_ptr(), packed.buffer.data_ptr(), out.data_ptr(), 4, 8, 64, 128, 32) != 0
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)   # refused calls write nothing
