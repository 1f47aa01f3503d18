"""Shapes beyond the common case, which take the multi-pass branches of the
kernels: documents longer than one shared-memory chunk of the contrastive
grad_documents kernel (2048 tokens), more (query, token) entries per document
than one pass holds (32768), documents longer than one bitmap pass of the
packed grad_documents kernel (1024 rows), queries of several 32-row passes,
and embedding dims beyond the tensor-core kernels' range."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from _util import assert_argmax, assert_grads, assert_scores, f32, i64, oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status_clean():
    _ops.set_pair_grouping(True)
    yield
    assert _ops.device_status() == 0


def _unit(shape, gen, dtype):
    x = torch.randn(shape, generator=gen)
    return torch.nn.functional.normalize(x, dim=-1).to(DEV, dtype)


def _contrastive_case(Nq, Lq, d_lens, dim, dtype, name, seed):
    g = torch.Generator().manual_seed(seed)
    q = _unit((Nq, Lq, dim), g, dtype)
    d = _unit((sum(d_lens), dim), g, dtype)
    off = torch.zeros(len(d_lens) + 1, dtype=torch.int32)
    off[1:] = torch.tensor(d_lens, dtype=torch.int32).cumsum(0)
    off = off.to(DEV)
    w = torch.randn(Nq, len(d_lens), generator=g).to(DEV)
    s, a = maxsim.score_contrastive_with_argmax(q, d, off)
    ws, wa, gaps = oracle.score_contrastive(f32(q), f32(d), i64(off), want_gap=True)
    assert_scores(f32(s), ws, name)
    assert_argmax(a.cpu().numpy(), wa, gaps, name)
    dq, dd = _ops.ops.maxsim_contrastive_backward(w, q, d, off, a)
    wq, wd = oracle.contrastive_backward(f32(w), f32(q), f32(d), i64(off), a.cpu().numpy())
    assert_grads(f32(dq), wq, name, "grad_queries")
    assert_grads(f32(dd), wd, name, "grad_documents")


def test_contrastive_documents_longer_than_one_chunk():
    _contrastive_case(12, 32, [2500, 10, 5000, 2048, 2049], 128, torch.bfloat16, "bf16", 1)


def test_contrastive_more_entries_than_one_pass():
    # 1100 queries x 32 tokens = 35200 entries per document
    _contrastive_case(1100, 32, [70, 33, 200], 128, torch.float16, "fp16", 2)


def test_contrastive_long_queries_fp32():
    _contrastive_case(3, 150, [40, 700], 64, torch.float32, "fp32", 3)


def test_packed_documents_longer_than_one_bitmap_pass():
    rng = np.random.default_rng(4)
    g = torch.Generator().manual_seed(4)
    q_lens = rng.integers(4, 33, size=30)
    d_lens = np.array([3000, 1500, 40, 2, 1100, 1024, 1025])
    dim, n_pairs = 64, 2100
    q = _unit((int(q_lens.sum()), dim), g, torch.float16)
    d = _unit((int(d_lens.sum()), dim), g, torch.float16)
    qo = torch.from_numpy(np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)).to(DEV)
    do = torch.from_numpy(np.concatenate([[0], np.cumsum(d_lens)]).astype(np.int32)).to(DEV)
    pq = torch.from_numpy(rng.integers(0, 30, size=n_pairs).astype(np.int32)).to(DEV)
    pd = torch.from_numpy(rng.integers(0, 7, size=n_pairs).astype(np.int32)).to(DEV)
    w = torch.randn(n_pairs, generator=g).to(DEV)
    s, a = maxsim.score_pairs_packed_with_argmax(q, qo, d, do, pq, pd, max_q_len=32)
    ws, wa, gaps = oracle.score_pairs_packed(f32(q), i64(qo), f32(d), i64(do), i64(pq), i64(pd), 32,
                                             want_gap=True)
    assert_scores(f32(s), ws, "fp16")
    assert_argmax(a.cpu().numpy(), wa, gaps, "fp16")
    launches = _ops.launch_count()
    dq, dd = _ops.ops.maxsim_packed_backward(w, q, qo, d, do, pq, pd, a, 32)
    assert _ops.launch_count() - launches <= 2 + 6      # owner-warp kernels (+ grouping by query)
    wq, wd = oracle.pairs_packed_backward(f32(w), f32(q), i64(qo), f32(d), i64(do), i64(pq), i64(pd),
                                          a.cpu().numpy())
    assert_grads(f32(dq), wq, "fp16", "grad_queries")
    assert_grads(f32(dd), wd, "fp16", "grad_documents")


def test_padded_long_queries_and_wide_embeddings():
    g = torch.Generator().manual_seed(5)
    for (B, C, Lq, Ld, dim, dtype, name) in [(2, 3, 300, 90, 128, torch.float16, "fp16"),
                                             (1, 2, 40, 60, 512, torch.float16, "fp16"),
                                             (1, 2, 33, 50, 256, torch.float32, "fp32")]:
        q = _unit((B, Lq, dim), g, dtype)
        d = _unit((B, C, Ld, dim), g, dtype)
        ql = torch.randint(Lq // 2, Lq + 1, (B,), generator=g, dtype=torch.int32).to(DEV)
        dl = torch.randint(1, Ld + 1, (B, C), generator=g, dtype=torch.int32).to(DEV)
        s, a = maxsim.score_candidates_padded_with_argmax(q, d, ql, dl)
        ws, wa, gaps = oracle.score_candidates_padded(f32(q), f32(d), i64(ql), i64(dl), want_gap=True)
        assert_scores(f32(s), ws, name)
        valid = np.arange(Lq)[None, None, :] < i64(ql)[:, None, None]
        assert_argmax(a.cpu().numpy(), wa, gaps, name, valid=np.broadcast_to(valid, wa.shape))
        w = torch.randn(B, C, generator=g).to(DEV)
        dq, dd = _ops.ops.maxsim_padded_backward(w.reshape(-1), q.reshape(B * Lq, dim),
                                                 d.reshape(B * C * Ld, dim), ql, dl.reshape(-1),
                                                 a.reshape(B * C, Lq), Lq, Ld, C)
        wq, wd = oracle.candidates_padded_backward(f32(w), f32(q), f32(d), i64(ql), i64(dl),
                                                   a.cpu().numpy())
        assert_grads(f32(dq).reshape(wq.shape), wq, name, "grad_queries")
        assert_grads(f32(dd).reshape(wd.shape), wd, name, "grad_documents")
