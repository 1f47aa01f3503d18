"""The allocation-free grouping entry point, ``maxsim_b200_group_pairs_static``.

Some hosts of this library cannot allocate device memory while they run: a
service that binds the C ABI with fixed buffers and no device allocator, a
process whose memory pool took the whole GPU at start-up, a loop that cannot
afford the device-wide synchronisation of ``cudaMalloc``.  For them the
counters of the pair grouping live in a fixed array inside the library.  This
file calls that entry point through the C ABI and checks it against
``maxsim_b200_group_pairs`` (caller-provided counters) on two calls in a row --
the second with other ids and fewer bins, so stale counters of the first call
would show -- and checks that the order it produces drives the ordered forward
operator to the scores of the plain one.  It is named to be collected last.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from maxsim_b200 import _ops
from maxsim_b200 import workloads as W

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
STATIC_LIMIT = 1 << 20


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _group_static(ids: torch.Tensor, n_bins: int) -> torch.Tensor:
    lib = _ops.load_library()
    order = torch.full((ids.shape[0],), -1, dtype=torch.int32, device=ids.device)
    rc = lib.maxsim_b200_group_pairs_static(ids.data_ptr(), ids.shape[0], n_bins,
                                            order.data_ptr(), _stream())
    assert rc == 0, lib.maxsim_b200_last_error().decode()
    return order


def _group_with_caller_memory(ids: torch.Tensor, n_bins: int) -> torch.Tensor:
    lib = _ops.load_library()
    order = torch.full((ids.shape[0],), -1, dtype=torch.int32, device=ids.device)
    ends = torch.empty((n_bins,), dtype=torch.int32, device=ids.device)
    rc = lib.maxsim_b200_group_pairs(ids.data_ptr(), ids.shape[0], n_bins, ends.data_ptr(),
                                     order.data_ptr(), _stream())
    assert rc == 0, lib.maxsim_b200_last_error().decode()
    return order


def _same_grouping(ids, got, want):
    n = ids.shape[0]
    # both are permutations ...
    assert torch.equal(got.long().sort().values, torch.arange(n, device=ids.device))
    assert torch.equal(want.long().sort().values, torch.arange(n, device=ids.device))
    # ... that put the same ids in the same positions (members of one group may
    # come in any order: the kernels place them with atomics)
    assert torch.equal(ids[got.long()], ids[want.long()])
    grouped = ids[got.long()]
    assert bool((grouped[1:] >= grouped[:-1]).all())


def test_static_grouping_matches_the_caller_memory_entry_point_twice_in_a_row():
    torch.cuda.set_device(0)
    rng = np.random.default_rng(11)
    first = torch.from_numpy(rng.integers(0, 20000, size=65536).astype(np.int32)).to(DEV)
    second = torch.from_numpy(rng.integers(0, 37, size=5000).astype(np.int32)).to(DEV)
    _same_grouping(first, _group_static(first, 20000), _group_with_caller_memory(first, 20000))
    _same_grouping(second, _group_static(second, 37), _group_with_caller_memory(second, 37))
    # and the first again, over the second call's leftovers
    _same_grouping(first, _group_static(first, 20000), _group_with_caller_memory(first, 20000))


def test_static_grouping_allocates_nothing_and_reports_its_limit():
    torch.cuda.set_device(0)
    lib = _ops.load_library()
    ids = torch.randint(0, 1000, (30000,), dtype=torch.int32, device=DEV)
    order = torch.empty_like(ids)
    _group_static(ids, 1000)                      # set-up call: symbol address lookup
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        rc = lib.maxsim_b200_group_pairs_static(ids.data_ptr(), ids.shape[0], 1000,
                                                order.data_ptr(), _stream())
        assert rc == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before              # the driver handed out no memory

    rc = lib.maxsim_b200_group_pairs_static(ids.data_ptr(), ids.shape[0], STATIC_LIMIT + 1,
                                            order.data_ptr(), _stream())
    assert rc != 0
    assert "exceeds" in lib.maxsim_b200_last_error().decode()
    rc = lib.maxsim_b200_group_pairs_static(ids.data_ptr(), ids.shape[0], STATIC_LIMIT,
                                            order.data_ptr(), _stream())
    assert rc == 0                                # the limit itself is accepted
    torch.cuda.synchronize()
    assert _ops.device_status() == 0


def test_static_order_drives_the_ordered_forward_to_the_plain_scores():
    torch.cuda.set_device(0)
    lib = _ops.load_library()
    wl = W.c4_packed_grid_fp16(seed=9, n_queries=200, n_docs=900, n_pairs=7000, dim=96)
    q = W.to_torch(wl.queries, "fp16", DEV)
    d = W.to_torch(wl.documents, "fp16", DEV)
    qo = torch.from_numpy(wl.query_offsets).to(DEV)
    do = torch.from_numpy(wl.document_offsets).to(DEV)
    pq = torch.from_numpy(wl.pair_query_ids).to(DEV)
    pd = torch.from_numpy(wl.pair_document_ids).to(DEV)
    n = pq.shape[0]
    sizes = (n, qo.shape[0] - 1, do.shape[0] - 1, q.shape[0], d.shape[0], 96, 32, 1)  # 1 = fp16
    for _ in range(2):                            # two calls in a row
        order = _group_static(pd, do.shape[0] - 1)
        got = torch.empty(n, dtype=torch.float32, device=DEV)
        rc = lib.maxsim_forward_ordered(q.data_ptr(), qo.data_ptr(), d.data_ptr(), do.data_ptr(),
                                        pq.data_ptr(), pd.data_ptr(), order.data_ptr(),
                                        got.data_ptr(), *sizes, _stream())
        assert rc == 0, lib.maxsim_b200_last_error().decode()
        want = torch.empty(n, dtype=torch.float32, device=DEV)
        rc = lib.maxsim_forward(q.data_ptr(), qo.data_ptr(), d.data_ptr(), do.data_ptr(),
                                pq.data_ptr(), pd.data_ptr(), want.data_ptr(), *sizes, _stream())
        assert rc == 0, lib.maxsim_b200_last_error().decode()
        assert torch.equal(got, want)             # every pair computed once, by the same code
