"""The CPU oracle against golden outputs of the reference's own PyTorch
implementation (made by tests/golden/make_golden.py).  This is what pins the
oracle; everything on the GPU is then compared with the oracle."""

from __future__ import annotations

import hashlib

import numpy as np
import pytest

from _util import GOLDEN, oracle
from maxsim_b200 import workloads as W

G = np.load(GOLDEN)


def _digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def _close(a, b, tol=2e-6):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return np.allclose(a, b, rtol=tol, atol=tol)


def _padded_small(dtype):
    wl = W.c1_padded_rerank_fp32(seed=10, Nq=3, Lq=12, C=4, Ld=40, dim=32, lo=1)
    wl.dtype = dtype
    wl.query_lengths = np.array([12, 7, 1], dtype=np.int32)
    return wl


@pytest.mark.parametrize("dtype", ["fp32", "fp16", "bf16"])
def test_padded_small(dtype):
    wl = _padded_small(dtype)
    q, d = W.on_grid(wl.queries, dtype), W.on_grid(wl.documents, dtype)
    s, a, gaps = oracle.score_candidates_padded(q, d, wl.query_lengths, wl.doc_lengths, want_gap=True)
    key = f"padded_small_{dtype}"
    assert _close(s, G[f"{key}/scores"])
    assert (oracle.argmax_mismatch_allowed(a, G[f"{key}/argmax"], gaps, 1e-6)).all()
    assert np.array_equal(a, G[f"{key}/argmax"])
    dq, dd = oracle.candidates_padded_backward(G[f"{key}/dscore"], q, d, wl.query_lengths,
                                               wl.doc_lengths, G[f"{key}/argmax"])
    assert _close(dq, G[f"{key}/dq"], 1e-5)
    assert _close(dd, G[f"{key}/dd"], 1e-5)


@pytest.mark.parametrize("dtype", ["fp32", "fp16", "bf16"])
def test_contrastive_small(dtype):
    wl = W.c2_contrastive_train_bf16(seed=11, Nq=5, Nb=6, Lq=16, dim=64, lo=1, hi=70, dtype=dtype)
    q, d = W.on_grid(wl.queries, dtype), W.on_grid(wl.documents, dtype)
    s, a = oracle.score_contrastive(q, d, wl.document_offsets)
    key = f"contrastive_small_{dtype}"
    assert _close(s, G[f"{key}/scores"])
    assert np.array_equal(a, G[f"{key}/argmax"])
    dq, dd = oracle.contrastive_backward(G[f"{key}/dscore"], q, d, wl.document_offsets,
                                         G[f"{key}/argmax"])
    assert _close(dq, G[f"{key}/dq"], 1e-5)
    assert _close(dd, G[f"{key}/dd"], 1e-5)


@pytest.mark.parametrize("dtype", ["fp32", "fp16", "bf16"])
def test_packed_small(dtype):
    wl = W.c4_packed_grid_fp16(seed=12, n_queries=7, n_docs=9, n_pairs=40, dim=96)
    q, d = W.on_grid(wl.queries, dtype), W.on_grid(wl.documents, dtype)
    s, a = oracle.score_pairs_packed(q, wl.query_offsets, d, wl.document_offsets,
                                     wl.pair_query_ids, wl.pair_document_ids)
    key = f"packed_small_{dtype}"
    assert _close(s, G[f"{key}/scores"])
    assert np.array_equal(a, G[f"{key}/argmax"])
    dq, dd = oracle.pairs_packed_backward(wl.dscore, q, wl.query_offsets, d, wl.document_offsets,
                                          wl.pair_query_ids, wl.pair_document_ids,
                                          G[f"{key}/argmax"])
    assert _close(dq, G[f"{key}/dq"], 1e-5)
    assert _close(dd, G[f"{key}/dd"], 1e-5)


def test_contrastive_exact_ties_pick_first_index():
    wl = W.c5_contrastive_ties_bf16(seed=13, Nq=6, Nb=8, Lq=32, dim=128, lo=20, hi=90, dup_frac=0.2)
    q, d = W.on_grid(wl.queries, "bf16"), W.on_grid(wl.documents, "bf16")
    s, a, gaps = oracle.score_contrastive(q, d, wl.document_offsets, want_gap=True)
    key = "contrastive_ties_bf16"
    assert _close(s, G[f"{key}/scores"])
    assert np.array_equal(a, G[f"{key}/argmax"])
    assert (gaps == 0).sum() > 0, "the workload is meant to contain exact ties"
    dq, dd = oracle.contrastive_backward(G[f"{key}/dscore"], q, d, wl.document_offsets, a)
    assert _close(dq, G[f"{key}/dq"], 1e-5)
    assert _close(dd, G[f"{key}/dd"], 1e-5)


def test_config1_full_size():
    wl = W.c1_padded_rerank_fp32()
    assert _digest(wl.queries, wl.documents, wl.doc_lengths).encode() == G["c1/input_digest"].tobytes(), \
        "the seeded generator no longer reproduces the inputs the fixture was made from"
    s, a, gaps = oracle.score_candidates_padded(wl.queries, wl.documents, wl.query_lengths,
                                                wl.doc_lengths, want_gap=True)
    assert _close(s, G["c1/scores"], 1e-5)
    assert oracle.argmax_mismatch_allowed(a, G["c1/argmax"].astype(np.int32), gaps, 1e-6).all()


def test_config2_full_size_forward():
    wl = W.c2_contrastive_train_bf16()
    assert _digest(wl.queries, wl.documents, wl.document_offsets).encode() == \
        G["c2/input_digest"].tobytes()
    q, d = W.on_grid(wl.queries, "bf16"), W.on_grid(wl.documents, "bf16")
    s, a, gaps = oracle.score_contrastive(q, d, wl.document_offsets, want_gap=True)
    assert _close(s, G["c2/scores"], 1e-5)
    assert oracle.argmax_mismatch_allowed(a, G["c2/argmax"].astype(np.int32), gaps, 1e-6).all()


def test_nan_never_wins():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((4, 8)).astype(np.float32)
    d = rng.standard_normal((6, 8)).astype(np.float32)
    q[1, 0] = np.nan
    s, a = oracle.pair_score_argmax(q, d)
    assert np.isneginf(s) and a[1] == 0
    q = rng.standard_normal((4, 8)).astype(np.float32)
    d[2, 3] = np.nan
    s, a = oracle.pair_score_argmax(q, d)
    assert np.isfinite(s) and (a != 2).all()


def test_gap_helper():
    q = np.eye(3, dtype=np.float32)
    d = np.array([[1, 0, 0], [1, 0, 0], [0, 0.5, 0]], dtype=np.float32)
    gap = oracle.top2_gap_pair(q, d)
    assert gap[0] == 0.0 and gap[1] == 0.5
