"""The give-up path of the kernels' bounded waits, made to run on purpose - without faulting anything.

Every mbarrier wait inside the tensor-core kernels has a time limit (2 s by default); when it runs out the waiting role
records its wait site in an error word, stops touching the pipeline and walks to the end of the kernel, where the CTA
drains its own copies and MMAs and frees its TMEM. nkb_set_wait_limit_ns shortens the limits per site, so a test can make
one wait run out while everything it waits for is in fact on its way: the epilogue's wait for a finished accumulator
(site 4) gets a few microseconds on a problem whose first accumulator takes tens of microseconds, the other sites get
20 ms. The epilogue gives up, the MMA issuer and the loader come to rest on their own waits and give up later, with the
pipeline quiet. Nothing traps, faults or spins without a bound.
"""
import numpy as np
import pytest

import numkong_b200 as nk
from numkong_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def _site(word):
    return (word >> 16) & 0x7fff if word >> 31 else 0


@pytest.fixture
def short_epilogue_wait():
    nk.set_wait_limit_ns(0, 20_000_000)   # every site: 20 ms
    nk.set_wait_limit_ns(4, 3_000)        # the epilogue's wait for an accumulator: 3 microseconds
    yield
    nk.set_wait_limit_ns(0, 0)
    nk.set_accumulation_span(0)
    nk.lib.nkb_set_gemm_variant(0)


# (rows, columns, forced tile variant, accumulation span): one tile on one CTA; two tiles per CTA of two spans each, so that
# the MMA issuer blocks on the third span's accumulator, the loader behind it, and both give up too (single-CTA kernel);
# then the same two shapes on the CTA-pair kernel.
@pytest.mark.parametrize("rows,cols,variant,span", [(128, 128, 2, 128), (2048, 2432, 2, 64), (256, 256, 3, 128), (3072, 3328, 3, 64)])
def test_epilogue_wait_runs_out_then_the_next_call_is_exact(rows, cols, variant, span, short_epilogue_wait):
    import torch
    depth = 8192   # 128 pipeline stages: a full-depth accumulator takes ~35 microseconds, a 64-stage span ~17
    a, b = syn.normal_matrix(rows, depth, "bf16", 41), syn.normal_matrix(cols, depth, "bf16", 42)
    ta, tb = torch.from_numpy(a.view(np.int16)).cuda(), torch.from_numpy(b.view(np.int16)).cuda()
    packed = nk.dots_pack(tb, "bf16")
    nk.set_wait_limit_ns(0, 0)
    nk.lib.nkb_set_gemm_variant(variant)
    nk.set_accumulation_span(span)
    good = nk.dots_packed(ta, packed, dtype="bf16")
    assert nk.synchronize() == 0
    # now with the short limits
    nk.set_wait_limit_ns(0, 20_000_000)
    nk.set_wait_limit_ns(4, 3_000)
    out = torch.full((rows, cols), -7.0, dtype=torch.float32, device="cuda")
    nk.dots_packed(ta, packed, out=out, dtype="bf16")
    word = nk.synchronize()
    assert _site(word) == 4, hex(word)          # the call returned, and the first wait to give up was the epilogue's
    assert nk.synchronize() == 0                # a failure is reported once
    nk.set_wait_limit_ns(0, 0)
    again = nk.dots_packed(ta, packed, dtype="bf16")
    assert nk.synchronize() == 0
    assert torch.equal(again, good)             # TMEM was freed, barriers start clean: bit-identical to the healthy call


def test_host_operand_call_reports_the_failure_itself(short_epilogue_wait):
    """A call with host-resident operands synchronises on its own: it fills the result with 0xFF bytes (the reference's
    failure convention, c/numkong.c:78-81), says why, and leaves the error word clean for the next call."""
    depth = 8192
    a, b = syn.normal_matrix(128, depth, "bf16", 43), syn.normal_matrix(128, depth, "bf16", 44)
    nk.set_wait_limit_ns(0, 0)
    packed = nk.dots_pack(b, "bf16")
    good = nk.dots_packed(a, packed)
    nk.set_accumulation_span(128)
    nk.set_wait_limit_ns(0, 20_000_000)
    nk.set_wait_limit_ns(4, 3_000)
    out = np.zeros((128, 128), dtype=np.float32)
    with pytest.raises(RuntimeError, match="gave up"):
        nk.dots_packed(a, packed, out=out)
    assert np.all(out.view(np.uint8) == 0xFF)
    nk.set_wait_limit_ns(0, 0)
    nk.set_accumulation_span(0)
    assert np.array_equal(nk.dots_packed(a, packed), good)


def test_error_word_is_reported_once_and_cleared():
    """The host side of the same story, with the failure made on the host: a value stored in the error word (as a wait that
    gave up would) fails the next host-operand call, is cleared by the report, and the call after that succeeds."""
    a, b = syn.normal_matrix(40, 96, "i8", 45), syn.normal_matrix(50, 96, "i8", 46)
    packed = nk.dots_pack(b, "i8")
    good = nk.dots_packed(a, packed)
    assert nk.lib.nkb_test_set_error_word(0, 0x80030007) == 0
    out = np.zeros_like(good)
    with pytest.raises(RuntimeError, match="0x80030007"):
        nk.dots_packed(a, packed, out=out)
    assert np.all(out.view(np.uint8) == 0xFF)
    assert np.array_equal(nk.dots_packed(a, packed), good)
    assert nk.synchronize() == 0
