"""In-place down-casts of a finished dots matrix on the device (nk_dots_compact_bf16 / nk_dots_compact_i8), bit for
bit against the committed reference vectors and the CPU oracle: host and device buffers, padded rows, single rows and
columns, a chain with the i8 product itself, and a full-size matrix."""
import os

import numpy as np
import pytest
import torch

import numkong_b200 as nk
import oracle

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "compact_path.npz"))
SHAPES = [(7, 5, 3), (33, 17, 65), (16, 24, 128), (5, 9, 1031)]


@pytest.mark.parametrize("where", ["host", "device"])
@pytest.mark.parametrize("shape", SHAPES)
def test_compact_matches_reference_vectors(shape, where):
    m, n, k = shape
    for dt in ("i8", "bf16"):
        key = f"{dt}_{m}x{n}x{k}"
        full = GOLDEN[key + "_c"].copy()
        norms = (GOLDEN[key + "_an"], GOLDEN[key + "_bn"]) if dt == "i8" else ()
        if where == "device":
            full_t = torch.from_numpy(full).cuda()
            got = nk.dots_compact(full_t[:, :n], *[torch.from_numpy(x).cuda() for x in norms])
            assert nk.synchronize() == 0
            got = (got.view(torch.int16) if dt == "bf16" else got).cpu().numpy().view(np.uint16 if dt == "bf16" else np.int8)
        else:
            got = nk.dots_compact(full[:, :n], *norms)
        assert got.shape == (m, n)
        assert np.array_equal(got, GOLDEN[key + "_compact_serial"])


@pytest.mark.parametrize("rows,cols,pad", [(1, 1, 0), (1, 5000, 0), (5000, 1, 3), (2, 2049, 1), (257, 300, 0), (1000, 4096, 8)])
def test_compact_bf16_shapes(rows, cols, pad):
    rng = np.random.default_rng(rows + cols)
    wide = np.zeros((rows, cols + pad), dtype=np.float32)
    wide[:, :cols] = (rng.standard_normal((rows, cols)) * np.exp2(rng.integers(-20, 21, (rows, cols)))).astype(np.float32)
    want = oracle.dots_compact(wide[:, :cols])
    dev = torch.from_numpy(wide).cuda()
    got = nk.dots_compact(dev[:, :cols])
    assert nk.synchronize() == 0
    assert got.dtype == torch.bfloat16 and got.data_ptr() == dev.data_ptr()      # a view of the same memory
    assert np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want)
    assert np.array_equal(want, torch.from_numpy(wide[:, :cols].copy()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    host = nk.dots_compact(wide[:, :cols])
    assert np.array_equal(host, want) and host.ctypes.data == wide.ctypes.data


def test_compact_i8_after_the_product_itself():
    """Quantised cosine matrix the way a caller builds it: i8 product on the device, squared norms, compact in place."""
    rng = np.random.default_rng(5)
    a, b = rng.integers(-128, 128, (700, 384), dtype=np.int8), rng.integers(-128, 128, (1300, 384), dtype=np.int8)
    a[17], b[5] = 0, 0
    b[9] = a[3]
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c = nk.dots_packed(ta, nk.dots_pack(tb))
    an = (ta.to(torch.int32) ** 2).sum(1).to(torch.int32)
    bn = (tb.to(torch.int32) ** 2).sum(1).to(torch.int32)
    want = oracle.dots_compact(oracle.dots(a, b, "i8"), an.cpu().numpy(), bn.cpu().numpy())
    got = nk.dots_compact(c, an, bn)
    assert nk.synchronize() == 0
    assert got.dtype == torch.int8 and np.array_equal(got.cpu().numpy(), want)
    assert np.all(want[17] == 0) and np.all(want[:, 5] == 0) and want[3, 9] in (126, 127)
    # host norms with a device matrix
    c2 = nk.dots_packed(ta, nk.dots_pack(tb))
    got2 = nk.dots_compact(c2, an.cpu().numpy(), bn.cpu().numpy())
    assert nk.synchronize() == 0 and np.array_equal(got2.cpu().numpy(), want)


def test_compact_full_size_matrix():
    """8192 x 8192 cells (256 MiB): bf16 against torch's own rounding, i8 on sampled rows against the oracle."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(1)
    f = torch.randn((n, n), device="cuda", generator=g) * 100
    want = f.to(torch.bfloat16)
    got = nk.dots_compact(f)
    assert nk.synchronize() == 0
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    a = torch.randint(-128, 128, (n, 512), device="cuda", generator=g, dtype=torch.int32).to(torch.int8)
    c = nk.dots_packed(a, nk.dots_pack(a))
    keep = c[::511].cpu().numpy().copy()
    norms = (a.to(torch.int32) ** 2).sum(1).to(torch.int32)
    got = nk.dots_compact(c, norms, norms)
    assert nk.synchronize() == 0
    hn = norms.cpu().numpy()
    assert np.array_equal(got[::511].cpu().numpy(), oracle.dots_compact(keep, hn[::511], hn))


def test_compact_argument_errors():
    with pytest.raises(TypeError):
        nk.dots_compact(np.zeros((2, 2), dtype=np.float64))
    with pytest.raises(ValueError):
        nk.dots_compact(np.zeros((2, 2), dtype=np.int32))                      # norms missing
    with pytest.raises(ValueError):
        nk.dots_compact(np.zeros((2, 2), dtype=np.int32), np.zeros(3, np.int32), np.zeros(2, np.int32))
