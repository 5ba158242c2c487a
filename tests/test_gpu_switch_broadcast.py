"""Delivery of a packed matrix through the NVSwitch multicast (nkb_multicast_store + nkb_peer_barrier, wrapped by
numkong_b200.sharding.SwitchBroadcast). The barrier kernel is also exercised on one GPU: alone, and with a peer that never
arrives, where its bounded wait must give up and leave the error word (site 8) instead of spinning."""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _flag_array(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_barrier_of_one_gpu_returns_at_once():
    import numkong_b200 as nk
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):
        assert nk.lib.nkb_peer_barrier(_flag_array(flags), 1, 0, epoch) == 0, nk.last_error()
    assert nk.synchronize() == 0
    assert int(flags[0].item()) == 3


def test_barrier_gives_up_on_a_peer_that_never_arrives():
    """Two flag buffers on this GPU stand for two GPUs; only "rank 0" ever runs, so slot 1 of its buffer stays 0."""
    import numkong_b200 as nk
    mine, theirs = torch.zeros(64, dtype=torch.int32, device="cuda"), torch.zeros(64, dtype=torch.int32, device="cuda")
    assert nk.synchronize() == 0
    nk.set_wait_limit_ns(8, 20_000)
    try:
        assert nk.lib.nkb_peer_barrier(_flag_array(mine, theirs), 2, 0, 1) == 0, nk.last_error()
        word = nk.synchronize()
    finally:
        nk.set_wait_limit_ns(8, 0)
    assert word == (0x80000000 | (8 << 16) | 1), hex(word)
    assert int(theirs[0].item()) == 1 and int(mine[0].item()) == 1   # it did announce itself to both
    assert nk.synchronize() == 0                                      # reported once, then clean
    # the "peer" arrives late: the next barrier passes
    theirs_arrives = torch.full((1,), 2, dtype=torch.int32, device="cuda")
    mine[1:2] = theirs_arrives
    assert nk.lib.nkb_peer_barrier(_flag_array(mine, theirs), 2, 0, 2) == 0
    assert nk.synchronize() == 0


def test_arguments_are_checked():
    import numkong_b200 as nk
    buf = torch.zeros(256, dtype=torch.uint8, device="cuda")
    assert nk.lib.nkb_multicast_store(buf.data_ptr() + 4, buf.data_ptr(), 64, 0) == 1
    assert nk.lib.nkb_multicast_store(buf.data_ptr(), buf.data_ptr(), 24, 0) == 1
    assert "16" in nk.last_error()
    host = np.zeros(64, dtype=np.uint8)
    assert nk.lib.nkb_multicast_store(buf.data_ptr(), host.ctypes.data & ~15, 16, 0) in (1, 2)
    assert nk.lib.nkb_multicast_store(buf.data_ptr(), buf.data_ptr(), 0, 0) == 0   # nothing to do
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert nk.lib.nkb_peer_barrier(_flag_array(flags), 17, 0, 1) == 1
    assert nk.lib.nkb_peer_barrier(_flag_array(flags), 1, 1, 1) == 1
    assert nk.synchronize() == 0


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import numkong_b200 as nk
        from numkong_b200 import sharding, synthetic as syn
        nk.set_stream(torch.cuda.current_stream().cuda_stream)
        n, k, dtype = 1000, 520, "bf16"
        b = syn.normal_matrix(n, k, dtype, 21)
        a = syn.normal_matrix(300, k, dtype, 22)
        size = nk.PackedMatrix.packed_size(n, k, dtype)
        channel = sharding.SwitchBroadcast(size)
        source = None
        if rank == 0:
            source = nk.dots_pack(torch.from_numpy(b.view(np.int16)).cuda(), dtype).buffer
        # three rounds: the buffer is reused, every delivery must be whole when `send` returns on the stream
        for round_ in range(3):
            channel.buffer.zero_()
            blob = channel.send(source, src=0)
            packed = nk.PackedMatrix(blob[:size], dtype, n, k)
            lo, hi = sharding.row_shard(a.shape[0], world, rank)
            got = nk.dots_packed(torch.from_numpy(a[lo:hi].view(np.int16)).cuda(), packed, dtype=dtype).cpu().numpy()
            want = nk.dots_packed(a[lo:hi], nk.dots_pack(b, dtype))
            assert np.array_equal(got, want), (rank, round_)
        assert nk.synchronize() == 0
        flag = torch.tensor([1.0 if channel.available else 0.0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print("multicast mapping available on every rank:", bool(flag.item()))
        channel.close()
    finally:
        dist.destroy_process_group()


def test_packed_matrix_travels_through_the_switch():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
