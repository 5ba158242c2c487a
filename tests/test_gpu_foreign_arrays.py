"""Device arrays that are neither NumPy nor torch objects (CuPy, Numba, ... stand-ins) are used in place: through
DLPack when offered for a CUDA device, else through __cuda_array_interface__. The reference's Python binding rejects
CUDA capsules (python/dlpack_interop.c:97-99 of the reference); accepting them is the second "next" row of the plan."""
import numpy as np
import pytest

import numkong_b200 as nk
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


class OnlyCudaArrayInterface:
    def __init__(self, tensor):
        self._keep = tensor
        self.__cuda_array_interface__ = tensor.__cuda_array_interface__


class OnlyDLPack:
    def __init__(self, tensor):
        self._t = tensor

    def __dlpack__(self, stream=None):
        return self._t.__dlpack__()

    def __dlpack_device__(self):
        return self._t.__dlpack_device__()


@pytest.mark.parametrize("wrap", [OnlyCudaArrayInterface, OnlyDLPack])
def test_foreign_cuda_arrays_are_used_in_place(wrap):
    import torch
    a = np.random.default_rng(1).integers(-128, 128, (70, 96), dtype=np.int8)
    b = np.random.default_rng(2).integers(-128, 128, (130, 96), dtype=np.int8)
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    packed = nk.dots_pack(wrap(tb))
    assert packed.is_cuda
    c = nk.dots_packed(wrap(ta), packed)
    assert c.is_cuda and nk.synchronize() == 0
    assert np.array_equal(c.cpu().numpy(), a.astype(np.int32) @ b.astype(np.int32).T)
    # a row slice with a stride: the interface carries byte strides
    wide = torch.zeros((70, 128), dtype=torch.int8, device="cuda")
    wide[:, :96] = ta
    c2 = nk.dots_packed(wrap(wide[:, :96]), packed)
    assert nk.synchronize() == 0 and torch.equal(c2, c)


def test_storage_words_need_a_dtype_name():
    import torch
    v = syn.normal_matrix(40, 64, "bf16", 3)
    t = torch.from_numpy(v.view(np.int16)).cuda()
    want = nk.dots_symmetric(t, dtype="bf16")
    got = nk.dots_symmetric(OnlyCudaArrayInterface(t), dtype="bf16")
    assert nk.synchronize() == 0 and torch.equal(got, want)
    with pytest.raises(TypeError):
        nk.dots_pack(OnlyCudaArrayInterface(t))  # int16 words have no element type of their own
