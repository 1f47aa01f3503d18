"""Document-order pass of the packed operators: the permutation is a
permutation with equal documents adjacent, and the operators give the same
results with it as in list order and as the oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from maxsim_b200 import workloads as W
from oracle import maxsim_oracle as oracle

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _grouping_on():
    _ops.set_pair_grouping(True)
    yield
    _ops.set_pair_grouping(True)


def _wl(n_pairs, n_docs=300, n_queries=80, dim=96, seed=5):
    return W.c4_packed_grid_fp16(seed=seed, n_queries=n_queries, n_docs=n_docs,
                                 n_pairs=n_pairs, dim=dim)


def _dev(wl, dtype="fp16"):
    return (W.to_torch(wl.queries, dtype, DEV), torch.from_numpy(wl.query_offsets).to(DEV),
            W.to_torch(wl.documents, dtype, DEV), torch.from_numpy(wl.document_offsets).to(DEV),
            torch.from_numpy(wl.pair_query_ids).to(DEV), torch.from_numpy(wl.pair_document_ids).to(DEV))


@pytest.mark.parametrize("n_pairs,n_docs", [(1, 1), (5, 3), (4096, 300), (65536, 20000), (10000, 1),
                                            (0, 7)])
def test_group_pairs_is_a_permutation_with_equal_ids_adjacent(n_pairs, n_docs):
    rng = np.random.default_rng(n_pairs + n_docs)
    ids_np = rng.integers(0, n_docs, size=n_pairs).astype(np.int32)
    ids = torch.from_numpy(ids_np).to(DEV)
    order, ends = _ops.group_pairs(ids, n_docs)
    assert order.dtype == torch.int32 and order.shape == (n_pairs,)
    assert ends.dtype == torch.int32 and ends.shape == (n_docs,)
    assert torch.equal(order.long().sort().values, torch.arange(n_pairs, device=DEV))
    grouped = ids[order.long()]
    assert bool((grouped[1:] >= grouped[:-1]).all())
    want_ends = np.cumsum(np.bincount(ids_np, minlength=n_docs))
    np.testing.assert_array_equal(ends.cpu().numpy(), want_ends)
    # twice in a row: same groups
    order2, ends2 = _ops.group_pairs(ids, n_docs)
    assert torch.equal(ids[order2.long()], grouped) and torch.equal(ends2, ends)


@pytest.mark.parametrize("dtype", ["fp16", "bf16", "fp32"])
def test_grouped_forward_equals_list_order_and_oracle(dtype):
    wl = _wl(6000)
    q, qo, d, do, pq, pd = _dev(wl, dtype)
    _ops.set_pair_grouping(False)
    s0, a0 = maxsim.score_pairs_packed_with_argmax(q, qo, d, do, pq, pd)
    p0 = maxsim.score_pairs_packed(q, qo, d, do, pq, pd)
    _ops.set_pair_grouping(True)
    launches = _ops.launch_count()
    s1, a1 = maxsim.score_pairs_packed_with_argmax(q, qo, d, do, pq, pd)
    assert _ops.launch_count() - launches == 4          # three grouping kernels + the operator
    launches = _ops.launch_count()
    p1 = maxsim.score_pairs_packed(q, qo, d, do, pq, pd)
    assert _ops.launch_count() - launches == 1          # the order is remembered for this tensor
    assert torch.equal(s0, s1) and torch.equal(a0, a1) and torch.equal(p0, p1)

    ws, wa, gaps = oracle.score_pairs_packed(
        q.float().cpu().numpy(), wl.query_offsets, d.float().cpu().numpy(), wl.document_offsets,
        wl.pair_query_ids[:800], wl.pair_document_ids[:800], int(a1.shape[1]), want_gap=True)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "fp32" else dict(rtol=2e-2, atol=1e-2)
    np.testing.assert_allclose(s1[:800].cpu().numpy(), ws, **tol)
    assert oracle.argmax_mismatch_allowed(a1[:800].cpu().numpy(), wa, gaps,
                                          1e-6 if dtype == "fp32" else 1e-3).all()


@pytest.mark.parametrize("dtype,dim", [("fp16", 96), ("bf16", 128), ("fp32", 64), ("fp16", 36),
                                       ("fp16", 160)])
def test_grouped_backward_equals_list_order_and_oracle(dtype, dim):
    wl = _wl(5000, dim=dim)
    q, qo, d, do, pq, pd = _dev(wl, dtype)
    g = torch.from_numpy(wl.dscore).to(DEV)
    grads = []
    for on in (False, True, True):
        _ops.set_pair_grouping(on)
        ql = q.clone().requires_grad_(True)
        dl = d.clone().requires_grad_(True)
        launches = _ops.launch_count()
        s = maxsim.score_pairs_packed_train(ql, qo, dl, do, pq, pd, max_q_len=32)
        s.backward(g)
        grads.append((s.detach(), ql.grad.float(), dl.grad.float(), _ops.launch_count() - launches))
    assert torch.equal(grads[0][0], grads[1][0])
    # sums of the same terms in a different order
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == "fp32" else dict(rtol=2e-2, atol=2e-3)
    torch.testing.assert_close(grads[0][1], grads[1][1], **tol)
    torch.testing.assert_close(grads[0][2], grads[1][2], **tol)
    if dim % 8 == 0:
        # owner warps: a remembered grouping gives the same bits on every run,
        # with one forward and two backward launches
        assert torch.equal(grads[1][1], grads[2][1]) and torch.equal(grads[1][2], grads[2][2])
        assert grads[2][3] == 3

    _, a = maxsim.score_pairs_packed_with_argmax(q, qo, d, do, pq, pd, max_q_len=32)
    wq, wd = oracle.pairs_packed_backward(
        wl.dscore, q.float().cpu().numpy(), wl.query_offsets, d.float().cpu().numpy(),
        wl.document_offsets, wl.pair_query_ids, wl.pair_document_ids, a.cpu().numpy())
    # autograd casts the fp32 gradient to the leaf dtype
    otol = dict(rtol=1e-4, atol=1e-5) if dtype == "fp32" else dict(rtol=2e-2, atol=1e-2)
    np.testing.assert_allclose(grads[1][1].cpu().numpy(), wq, **otol)
    np.testing.assert_allclose(grads[1][2].cpu().numpy(), wd, **otol)


def test_grouped_backward_leaves_no_row_unwritten():
    # documents and queries that no pair names must come back as exact zeros
    wl = _wl(2100, n_docs=900, n_queries=400)
    q, qo, d, do, pq, pd = _dev(wl)
    lib_dq, lib_dd = _ops.ops.maxsim_packed_backward(
        torch.from_numpy(wl.dscore).to(DEV), q, qo, d, do, pq, pd,
        maxsim.score_pairs_packed_with_argmax(q, qo, d, do, pq, pd, max_q_len=32)[1], 32)
    used_d = np.zeros(900, bool); used_d[wl.pair_document_ids] = True
    used_q = np.zeros(400, bool); used_q[wl.pair_query_ids] = True
    assert (~used_d).any() and (~used_q).any()
    for b in np.nonzero(~used_d)[0][:50]:
        assert bool((lib_dd[wl.document_offsets[b]:wl.document_offsets[b + 1]] == 0).all())
    for b in np.nonzero(~used_q)[0][:50]:
        assert bool((lib_dq[wl.query_offsets[b]:wl.query_offsets[b + 1]] == 0).all())
    assert bool(torch.isfinite(lib_dd).all()) and bool(torch.isfinite(lib_dq).all())


def test_order_follows_an_in_place_change_of_the_pair_list():
    wl = _wl(3000)
    q, qo, d, do, pq, pd = _dev(wl)
    s0 = maxsim.score_pairs_packed(q, qo, d, do, pq, pd)
    w = torch.randn(3000, device=DEV)

    def grads():
        qr, dr = q.clone().requires_grad_(True), d.clone().requires_grad_(True)
        maxsim.score_pairs_packed_train(qr, qo, dr, do, pq, pd, max_q_len=32).backward(w)
        return qr.grad.float(), dr.grad.float()

    grads()  # builds and remembers the groupings of the current lists
    pd.copy_(pd.flip(0))
    pq.copy_(pq.roll(7))
    s1 = maxsim.score_pairs_packed(q, qo, d, do, pq, pd)
    gq1, gd1 = grads()  # the grouped backward has to follow the new lists
    _ops.set_pair_grouping(False)
    want = maxsim.score_pairs_packed(q, qo, d, do, pq, pd)
    wq, wd = grads()
    assert torch.equal(s1, want)
    assert not torch.equal(s0, s1)
    torch.testing.assert_close(gq1, wq, rtol=2e-2, atol=1e-3)
    torch.testing.assert_close(gd1, wd, rtol=2e-2, atol=1e-3)


def test_int64_pair_ids_and_short_lists():
    wl = _wl(2500)
    q, qo, d, do, pq, pd = _dev(wl)
    s32 = maxsim.score_pairs_packed(q, qo, d, do, pq, pd)
    s64 = maxsim.score_pairs_packed(q, qo.long(), d, do.long(), pq.long(), pd.long())
    assert torch.equal(s32, s64)
    few = maxsim.score_pairs_packed(q, qo, d, do, pq[:100].contiguous(), pd[:100].contiguous())
    assert torch.equal(few, s32[:100])
