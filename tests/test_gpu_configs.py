"""The five benchmark configurations as seeded parity tests: against the
golden outputs of the reference where a fixture exists, against the CPU oracle
at sizes it finishes in seconds, and through size-independent properties
(pair independence, agreement between kernel families, routing identities) at
the full sizes."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from maxsim_b200 import workloads as W
from _util import (GOLDEN, assert_all_pairs, assert_argmax, assert_grads, assert_scores, f32,
                   gpu_einsum_contrastive, gpu_einsum_padded, i64, oracle)

pytestmark = pytest.mark.gpu
DEV = "cuda"
G = np.load(GOLDEN)


@pytest.fixture(autouse=True)
def _clean():
    _ops.set_forward_path(0)
    yield
    _ops.set_forward_path(0)
    assert _ops.device_status() == 0


def test_config1_padded_rerank_fp32_against_reference_golden():
    wl = W.c1_padded_rerank_fp32()
    q, d = W.to_torch(wl.queries, "fp32", DEV), W.to_torch(wl.documents, "fp32", DEV)
    ql = torch.from_numpy(wl.query_lengths).to(DEV)
    dl = torch.from_numpy(wl.doc_lengths).to(DEV)
    s, a = maxsim.score_candidates_padded_with_argmax(q, d, ql, dl)
    assert s.shape == (16, 32) and a.shape == (16, 32, 32) and a.dtype == torch.int32
    _, _, gaps = oracle.score_candidates_padded(wl.queries, wl.documents, wl.query_lengths,
                                                wl.doc_lengths, want_gap=True)
    assert_scores(f32(s), G["c1/scores"], "fp32")
    assert_argmax(a.cpu().numpy(), G["c1/argmax"].astype(np.int32), gaps, "fp32")
    assert torch.equal(s, maxsim.score_candidates_padded(q, d, ql, dl))


def test_config2_contrastive_train_bf16():
    wl = W.c2_contrastive_train_bf16()
    q = W.to_torch(wl.queries, "bf16", DEV).requires_grad_(True)
    d = W.to_torch(wl.documents, "bf16", DEV).requires_grad_(True)
    off = torch.from_numpy(wl.document_offsets).to(DEV)
    s = maxsim.score_contrastive_train(q, d, off)
    loss = torch.nn.functional.cross_entropy(s, torch.arange(64, device=DEV))
    loss.backward()
    s2, a = maxsim.score_contrastive_with_argmax(q.detach(), d.detach(), off)
    qf, df = f32(q), f32(d)
    ws, wa, gaps = oracle.score_contrastive(qf, df, wl.document_offsets, want_gap=True)
    assert_scores(f32(s), G["c2/scores"], "bf16")
    assert_argmax(a.cpu().numpy(), G["c2/argmax"].astype(np.int32), gaps, "bf16")
    g = torch.softmax(s.detach(), dim=1)
    g[torch.arange(64), torch.arange(64)] -= 1.0
    g /= 64
    wq, wd = oracle.contrastive_backward(f32(g), qf, df, wl.document_offsets, a.cpu().numpy())
    assert_grads(f32(q.grad), wq, "bf16", "queries.grad")
    assert_grads(f32(d.grad), wd, "bf16", "documents.grad")
    want_loss = torch.nn.functional.cross_entropy(torch.from_numpy(ws), torch.arange(64))
    assert abs(float(loss.detach()) - float(want_loss)) < 2e-2


def test_config3_large_rerank_fp16_scaled_against_oracle():
    wl = W.c3_large_rerank_fp16(Nq=6, C=120)
    q, d = W.to_torch(wl.queries, "fp16", DEV), W.to_torch(wl.documents, "fp16", DEV)
    ql = torch.from_numpy(wl.query_lengths).to(DEV)
    dl = torch.from_numpy(wl.doc_lengths).to(DEV)
    s, a = maxsim.score_candidates_padded_with_argmax(q, d, ql, dl)
    ws, wa, gaps = oracle.score_candidates_padded(f32(q), f32(d), wl.query_lengths, wl.doc_lengths,
                                                  want_gap=True)
    assert_scores(f32(s), ws, "fp16")
    assert_argmax(a.cpu().numpy(), wa, gaps, "fp16")
    assert (wl.query_lengths < 32).any(), "the workload masks trailing query tokens"
    # a prefix mask converts to the same lengths
    mask = torch.arange(32)[None, :] < torch.from_numpy(wl.query_lengths)[:, None]
    assert maxsim.lengths_from_prefix_mask(mask).tolist() == wl.query_lengths.tolist()


def test_config3_full_size_properties():
    """256 x 1000 pairs, 19.7 GB of padded documents: a strided subset against
    the oracle, and pair independence (scoring a query alone gives bit-identical
    scores to scoring it inside the batch)."""
    free, _ = torch.cuda.mem_get_info()
    if free < 45 * 2 ** 30:
        pytest.skip("needs about 40 GB of free device memory")
    data = W.c3_device_shard(0, 256, DEV)
    q, d, ql, dl = data["queries"], data["documents"], data["query_lengths"], data["doc_lengths"]
    s = maxsim.score_candidates_padded(q, d, ql, dl)
    assert s.shape == (256, 1000) and torch.isfinite(s).all()
    for b in (0, 101, 255):
        alone = maxsim.score_candidates_padded(q[b:b + 1], d[b:b + 1], ql[b:b + 1], dl[b:b + 1])
        assert torch.equal(alone[0], s[b])
        ws, _ = oracle.score_candidates_padded(f32(q[b:b + 1]), f32(d[b:b + 1, :200]),
                                               i64(ql[b:b + 1]), i64(dl[b:b + 1, :200]))
        assert_scores(f32(s[b:b + 1, :200]), ws, "fp16")
    # sharding by query reproduces the unsharded tensor (what the multi-GPU path relies on)
    shard = W.c3_device_shard(128, 130, DEV)
    assert torch.equal(shard["documents"], d[128:130]) and torch.equal(shard["doc_lengths"], dl[128:130])


def test_config3_full_size_every_pair_against_fp32_einsum():
    """All 256 000 pairs of the full-size rerank configuration, scores and
    argmax, against the chunked fp32 einsum on the same device; the checker
    itself is pinned to the CPU oracle on a few candidates first."""
    free, _ = torch.cuda.mem_get_info()
    if free < 45 * 2 ** 30:
        pytest.skip("needs about 40 GB of free device memory")
    data = W.c3_device_shard(0, 256, DEV)
    q, d, ql, dl = data["queries"], data["documents"], data["query_lengths"], data["doc_lengths"]
    cs, ca, cg = gpu_einsum_padded(q[:2], d[:2, :40], ql[:2], dl[:2, :40])
    ws, wa, wg = oracle.score_candidates_padded(f32(q[:2]), f32(d[:2, :40]), i64(ql[:2]),
                                                i64(dl[:2, :40]), want_gap=True)
    assert_scores(f32(cs), ws, "fp32")
    assert_argmax(ca.cpu().numpy(), wa, wg, "fp16")
    s, a = maxsim.score_candidates_padded_with_argmax(q, d, ql, dl)
    s_only = maxsim.score_candidates_padded(q, d, ql, dl)
    assert torch.equal(s, s_only)
    want_s, want_a, gaps = gpu_einsum_padded(q, d, ql, dl)
    n_diff, max_err = assert_all_pairs(s, a, want_s, want_a, gaps, "fp16")
    assert max_err < 1e-3
    assert n_diff < 1e-3 * a.numel()


def test_config4_packed_grid_fp16_forward_backward():
    wl = W.c4_packed_grid_fp16()
    q = W.to_torch(wl.queries, "fp16", DEV).requires_grad_(True)
    d = W.to_torch(wl.documents, "fp16", DEV).requires_grad_(True)
    qo = torch.from_numpy(wl.query_offsets).to(DEV)
    do = torch.from_numpy(wl.document_offsets).to(DEV)
    pq = torch.from_numpy(wl.pair_query_ids).to(DEV)
    pd = torch.from_numpy(wl.pair_document_ids).to(DEV)
    g = torch.from_numpy(wl.dscore).to(DEV)
    pairs = np.stack([wl.pair_query_ids, wl.pair_document_ids], 1)
    assert len(np.unique(pairs, axis=0)) < len(pairs), "the grid is meant to contain duplicate pairs"
    s = maxsim.score_pairs_packed_train(q, qo, d, do, pq, pd)
    (s * g).sum().backward()
    s2, a = maxsim.score_pairs_packed_with_argmax(q.detach(), qo, d.detach(), do, pq, pd)
    assert a.shape == (65536, 32)
    qf, df = f32(q), f32(d)
    # forward against the oracle on all 65 536 pairs
    ws, wa, gaps = oracle.score_pairs_packed(qf, wl.query_offsets, df, wl.document_offsets,
                                             wl.pair_query_ids, wl.pair_document_ids,
                                             max_q_len=32, want_gap=True)
    assert_scores(f32(s2), ws, "fp16")
    assert_scores(f32(s), ws, "fp16", "scores(train)")
    assert_argmax(a.cpu().numpy(), wa, gaps, "fp16")
    # backward against the oracle on all pairs (routing through the kernel's argmax)
    wq, wd = oracle.pairs_packed_backward(wl.dscore, qf, wl.query_offsets, df, wl.document_offsets,
                                          wl.pair_query_ids, wl.pair_document_ids, a.cpu().numpy())
    assert_grads(f32(q.grad), wq, "fp16", "queries.grad")
    assert_grads(f32(d.grad), wd, "fp16", "documents.grad")


def test_config5_contrastive_ties_scaled_against_oracle():
    wl = W.c5_contrastive_ties_bf16(Nq=64, Nb=96)
    q = W.to_torch(wl.queries, "bf16", DEV).requires_grad_(True)
    d = W.to_torch(wl.documents, "bf16", DEV).requires_grad_(True)
    off = torch.from_numpy(wl.document_offsets).to(DEV)
    s = maxsim.score_contrastive_train(q, d, off)
    loss = torch.nn.functional.cross_entropy(s, torch.arange(64, device=DEV))
    loss.backward()
    _, a = maxsim.score_contrastive_with_argmax(q.detach(), d.detach(), off)
    qf, df = f32(q), f32(d)
    ws, wa, gaps = oracle.score_contrastive(qf, df, wl.document_offsets, want_gap=True)
    assert_scores(f32(s), ws, "bf16")
    exact = gaps == 0
    assert exact.mean() > 0.01
    assert np.array_equal(a.cpu().numpy()[exact], wa[exact]), "an exact tie did not pick the first index"
    assert_argmax(a.cpu().numpy(), wa, gaps, "bf16")
    g = torch.softmax(s.detach(), dim=1)
    g[torch.arange(64), torch.arange(64)] -= 1.0
    g /= 64
    wq, wd = oracle.contrastive_backward(f32(g), qf, df, wl.document_offsets, a.cpu().numpy())
    assert_grads(f32(q.grad), wq, "bf16", "queries.grad")
    assert_grads(f32(d.grad), wd, "bf16", "documents.grad")


def test_config5_full_size_properties():
    """1024 x 1024 pairs: a strided subset of queries against the oracle, the
    two tensor-core kernel families against each other, and the backward
    identity sum(grad_q * q) == sum(dscore * scores) (every routed term appears
    once on each side)."""
    data = W.c5_device(DEV)
    q, d, off = data["queries"], data["documents"], data["document_offsets"]
    s, a = maxsim.score_contrastive_with_argmax(q, d, off)
    assert s.shape == (1024, 1024) and a.shape == (1024, 1024, 32)
    sel = torch.arange(0, 1024, 128, device=DEV)
    ws, wa, gaps = oracle.score_contrastive(f32(q[sel]), f32(d), i64(off), want_gap=True)
    assert_scores(f32(s[sel]), ws, "bf16")
    assert_argmax(a[sel].cpu().numpy(), wa, gaps, "bf16")
    exact = gaps == 0
    assert np.array_equal(a[sel].cpu().numpy()[exact], wa[exact])
    _ops.set_forward_path(2)
    s_mma, a_mma = maxsim.score_contrastive_with_argmax(q[:64].contiguous(), d, off)
    _ops.set_forward_path(0)
    torch.testing.assert_close(s[:64], s_mma, rtol=1e-4, atol=1e-4)
    assert (a[:64] != a_mma).float().mean() < 1e-3
    g = torch.randn(1024, 1024, device=DEV)
    dq, dd = _ops.ops.maxsim_contrastive_backward(g, q, d, off, a)
    lhs = float((dq * q.float()).sum())
    mid = float((dd * d.float()).sum())
    rhs = float((g * s).sum())
    assert abs(lhs - rhs) <= 2e-3 * abs(rhs) + 1.0
    assert abs(mid - rhs) <= 2e-3 * abs(rhs) + 1.0


def test_config5_full_size_every_pair_against_fp32_einsum():
    """All 1 048 576 pairs of the full-size ties configuration, scores and
    argmax, against the chunked fp32 einsum on the same device (pinned to the
    CPU oracle on a block of queries first), for both tilings of the tcgen05
    kernel; duplicated tokens (exact ties in the checker) must give the first
    index everywhere."""
    data = W.c5_device(DEV)
    q, d, off = data["queries"], data["documents"], data["document_offsets"]
    want_s, want_a, gaps = gpu_einsum_contrastive(q, d, off)
    ws, wa, wg = oracle.score_contrastive(f32(q[:4]), f32(d), i64(off), want_gap=True)
    assert_scores(f32(want_s[:4]), ws, "fp32")
    assert_argmax(want_a[:4].cpu().numpy(), wa, wg, "bf16")
    exact = gaps == 0
    assert float(exact.float().mean()) > 0.01
    for path in (8, 9):
        _ops.set_forward_path(path)
        s, a = maxsim.score_contrastive_with_argmax(q, d, off)
        n_diff, max_err = assert_all_pairs(s, a, want_s, want_a, gaps, "bf16")
        assert max_err < 2e-3 and n_diff < 1e-3 * a.numel()
        # A tie of the checker is either a duplicated token (identical rows: the first copy
        # has to win in any arithmetic) or, a few times in 33 million, two different tokens
        # whose fp32 sums happen to coincide in the checker's summation order.
        mism = exact & (a != want_a)
        if bool(mism.any()):
            _, d_idx, _ = mism.nonzero(as_tuple=True)
            base = off.to(torch.int64)[d_idx]
            got_rows = d[base + a[mism].to(torch.int64)]
            want_rows = d[base + want_a[mism].to(torch.int64)]
            duplicated = (got_rows == want_rows).all(dim=1)
            assert not bool(duplicated.any()), "a duplicated token did not give its first copy"
            assert int(mism.sum()) < 1e-5 * a.numel()
    _ops.set_forward_path(0)
    s_only = maxsim.score_contrastive(q, d, off)
    torch.testing.assert_close(s_only, want_s, rtol=1e-4, atol=1e-3)
