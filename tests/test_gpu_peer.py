"""The kernels of the peer-memory transport on one GPU: record packing with
per-owner destination pointers against the send-buffer form, and the flag
barrier with its peers' flags written by the test (no second kernel that it
could wait on).  The transport across real ranks is in test_gpu_dist.py."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("cols", [[0, 5, 5, 12, 20], [0, 20], [0, 7, 20]])
def test_records_stored_through_owner_pointers_equal_the_send_buffer(cols):
    from maxsim_b200 import _ops
    dev = _dev()
    gen = torch.Generator().manual_seed(11)
    Nq, Nb, Lq = 9, cols[-1], 13
    argmax = torch.randint(0, 300, (Nq, Nb, Lq), generator=gen, dtype=torch.int32).to(dev)
    dscore = torch.randn(Nq, Nb, generator=gen).to(dev)
    col_start = torch.tensor(cols, dtype=torch.int32, device=dev)
    send = _ops.pack_owner_records(argmax, dscore, col_start)
    # every owner gets a buffer of its own, with room in front as if other ranks' queries came first
    width = Lq + 1
    bufs, ptrs, lead = [], [], 3
    for o in range(len(cols) - 1):
        n_o = cols[o + 1] - cols[o]
        buf = torch.full(((lead + Nq) * n_o * width + 8,), -7, dtype=torch.int32, device=dev)
        bufs.append(buf)
        ptrs.append(buf.data_ptr() + 4 * lead * n_o * width)
    table = torch.tensor(ptrs, dtype=torch.int64, device=dev)
    _ops.pack_owner_records_to(argmax, dscore, col_start, table)
    for o, buf in enumerate(bufs):
        n_o = cols[o + 1] - cols[o]
        words = Nq * n_o * width
        begin = lead * n_o * width
        assert torch.equal(buf[begin:begin + words], send[cols[o] * Nq * width:cols[o] * Nq * width + words])
        assert bool((buf[:begin] == -7).all()) and bool((buf[begin + words:] == -7).all())


def test_barrier_passes_when_the_peers_have_signalled_and_reports_when_they_have_not():
    from maxsim_b200 import _ops
    dev = _dev()
    _ops.device_status()  # clear
    world, rank = 4, 1
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    table = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    # the peers are already at barrier 1 (one of them a barrier ahead)
    flags[rank].copy_(torch.tensor([1, 0, 2, 1], dtype=torch.int32))
    _ops.peer_barrier(table, rank, world, counter, polls=2000)
    assert _ops.device_status() == 0 and int(counter.item()) == 1
    for r in range(world):
        if r != rank:
            assert flags[r].tolist()[rank] == 1  # this rank's arrival, stored in every peer's flags
    # barrier 2: rank 2 is there, ranks 0 and 3 never arrive -- the wait gives up and says so
    _ops.peer_barrier(table, rank, world, counter, polls=2000)
    assert _ops.device_status() & 4
    assert _ops.device_status() == 0 and int(counter.item()) == 2
    # a single rank has nobody to wait for
    alone = torch.zeros(1, dtype=torch.int32, device=dev)
    _ops.peer_barrier(table, 0, 1, alone)
    assert _ops.device_status() == 0 and int(alone.item()) == 1


def test_gather_of_segments_by_address():
    from maxsim_b200 import _ops
    dev = _dev()
    gen = torch.Generator().manual_seed(5)
    srcs = [torch.randint(-1000, 1000, (n,), generator=gen, dtype=torch.int32).to(dev)
            for n in (7, 1024, 36, 4096 + 4)]
    dst0 = torch.full((8000,), -1, dtype=torch.int32, device=dev)
    dst1 = torch.full((6000,), -1, dtype=torch.int32, device=dev)
    # (source, destination, offset in words): aligned and unaligned pieces, both destinations
    plan = [(0, 0, 3), (1, 1, 16), (2, 0, 100), (3, 1, 1200)]
    rows = [[srcs[i].data_ptr(), which, 4 * at, 4 * srcs[i].numel()] for i, which, at in plan]
    table = torch.tensor(rows, dtype=torch.int64, device=dev)
    _ops.peer_gather(table, max(r[3] for r in rows), dst0, dst1)
    want0 = torch.full((8000,), -1, dtype=torch.int32, device=dev)
    want1 = torch.full((6000,), -1, dtype=torch.int32, device=dev)
    for i, which, at in plan:
        (want1 if which else want0)[at:at + srcs[i].numel()] = srcs[i]
    assert torch.equal(dst0, want0) and torch.equal(dst1, want1)
    # nothing to do
    _ops.peer_gather(table[:0].contiguous(), 0, dst0)


def test_many_copies_with_one_call():
    from maxsim_b200 import _ops
    dev = _dev()
    gen = torch.Generator().manual_seed(9)
    srcs = [torch.randint(0, 255, (n,), generator=gen, dtype=torch.uint8).to(dev) for n in (5, 4096, 0, 333)]
    dst = torch.zeros(6000, dtype=torch.uint8, device=dev)
    at = [10, 100, 4500, 5000]
    _ops.copy_many([dst.data_ptr() + a for a in at], [s.data_ptr() for s in srcs],
                   [s.numel() for s in srcs], dev)
    want = torch.zeros(6000, dtype=torch.uint8, device=dev)
    for a, s in zip(at, srcs):
        want[a:a + s.numel()] = s
    assert torch.equal(dst, want)
    _ops.copy_many([], [], [], dev)
    with pytest.raises(ValueError):
        _ops.copy_many([1], [], [4], dev)
