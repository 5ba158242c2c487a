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
    return nk.lib.nkb_angulars_packed_noalloc(nk.DTYPE_CODES[dtype], ta.data_ptr(), packed.buffer.data_ptr(), out.data_ptr(),
                                              ta.shape[0], packed.width, ta.shape[1], ta.stride(0) * ta.element_size(), out.stride(0) * 4)


@pytest.mark.parametrize("dtype", ["bf16", "i8", "e4m3"])
def test_noalloc_matches_regular_entry_point_twice_in_a_row(dtype):
    import torch
    import oracle
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
        # Same kernels, same inputs: the tolerance of the distance tests (5e-7 absolute) is met with margin ...
        assert torch.max(torch.abs(got - want)).item() <= 5e-7
        # ... and, independently of the regular entry point, against the CPU oracle of the reference's formula.
        assert np.max(np.abs(got.cpu().numpy() - oracle.angulars(a, b, dtype))) <= 5e-7
        outs.append(got)
    assert outs[0].shape != outs[1].shape


def test_noalloc_error_word_reaches_the_caller():
    """A caller of the allocation-free entry point learns of a pipeline wait that gave up from nkb_synchronize(), which reads
    the entry point's fixed error word too. The failure is made on the host here: a value is stored in that word, as a wait
    that ran out would; the next synchronisation returns it, the one after that is clean. Nothing on the device fails."""
    import torch
    a = torch.from_numpy(syn.normal_matrix(64, 128, "bf16", 1).view(np.int16)).cuda()
    packed = nk.dots_pack(torch.from_numpy(syn.normal_matrix(70, 128, "bf16", 2).view(np.int16)).cuda(), "bf16")
    out = torch.empty((64, 70), dtype=torch.float32, device="cuda")
    assert _call_noalloc("bf16", a, packed, out) == 0, nk.last_error()   # sets the fixed arrays up on this GPU
    assert nk.synchronize() == 0
    assert nk.lib.nkb_test_set_error_word(1, 0x80040002) == 0
    assert nk.synchronize() == 0x80040002
    assert nk.synchronize() == 0
    assert _call_noalloc("bf16", a, packed, out) == 0 and nk.synchronize() == 0


_FRESH_PROCESS = r"""
import ctypes, numpy as np, torch
import numkong_b200 as nk
from numkong_b200 import synthetic as syn
a = torch.from_numpy(syn.normal_matrix(64, 128, "bf16", 1).view(np.int16)).cuda()
blob = torch.zeros(nk.PackedMatrix.packed_size(70, 128, "bf16"), dtype=torch.uint8, device="cuda")
b = torch.from_numpy(syn.normal_matrix(70, 128, "bf16", 2).view(np.int16)).cuda()
out = torch.empty((64, 70), dtype=torch.float32, device="cuda")
nk.lib.nk_dots_pack_bf16(b.data_ptr(), 70, 128, 256, blob.data_ptr())   # device to device: allocates nothing
call = lambda: nk.lib.nkb_angulars_packed_noalloc(nk.DTYPE_CODES["bf16"], a.data_ptr(), blob.data_ptr(), out.data_ptr(), 64, 70, 128, 256, 280)
assert call() == 0, nk.last_error()          # first call on this GPU: looks the fixed arrays up
torch.cuda.synchronize()
free_before = torch.cuda.mem_get_info()[0]
assert nk.synchronize() == 0
assert call() == 0 and nk.synchronize() == 0
free_after = torch.cuda.mem_get_info()[0]
assert free_after == free_before, (free_before, free_after)
print("free memory unchanged:", free_after)
"""


def test_noalloc_and_synchronize_allocate_nothing_in_a_fresh_process():
    """In a process that has used nothing but the allocation-free entry point, neither that entry point nor nkb_synchronize()
    may take device memory: free memory on the GPU is the same before and after (the check runs in a child process so that
    no earlier test has created the regular entry points' error word)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", _FRESH_PROCESS], cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr


def test_noalloc_refuses_what_it_cannot_do_without_allocating():
    import torch
    a = torch.zeros((4, 64), dtype=torch.int16, device="cuda")
    packed = nk.dots_pack(torch.zeros((8, 64), dtype=torch.int16, device="cuda"), "bf16")
    out = torch.full((4, 8), 7.0, dtype=torch.float32, device="cuda")
    fn = nk.lib.nkb_angulars_packed_noalloc
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
