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
    # the peers are already at epoch 1 (one of them a barrier ahead)
    flags[rank].copy_(torch.tensor([1, 0, 2, 1], dtype=torch.int32))
    _ops.peer_barrier(table, rank, world, 1, polls=2000)
    assert _ops.device_status() == 0
    for r in range(world):
        if r != rank:
            assert flags[r].tolist()[rank] == 1  # this rank's arrival, stored in every peer's flags
    # epoch 2: rank 2 is there, ranks 0 and 3 never arrive -- the wait gives up and says so
    _ops.peer_barrier(table, rank, world, 2, polls=2000)
    assert _ops.device_status() & 4
    assert _ops.device_status() == 0
    # a single rank has nobody to wait for
    _ops.peer_barrier(table, 0, 1, 5)
    assert _ops.device_status() == 0
