"""Forward parity on the GPU through the C ABI, against the CPU oracle.

Covers what the reference's own suite covers for the forward path
(tests/test_padded.py, test_argmax.py, test_contrastive.py, test_correctness.py,
test_dtypes.py, test_ragged.py, test_edge_shapes.py, test_fuzz.py): all three
layouts, three dtypes, tile-boundary shapes, garbage in padding, ties, empty
pair lists, shared ids, and every forward kernel family (forced by
``set_forward_path``)."""

from __future__ import annotations

import random

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from _util import NAME_OF, TORCH_DTYPE, assert_argmax, assert_scores, f32, i64, oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status_clean():
    _ops.set_forward_path(0)
    yield
    _ops.set_forward_path(0)
    assert _ops.device_status() == 0, "a kernel reported a bounded wait that ran out"


def _check_padded(q, d, qlen, dlen, dtype, path=0):
    _ops.set_forward_path(path)
    name = NAME_OF[dtype]
    s = maxsim.score_candidates_padded(q, d, qlen, dlen)
    s2, a = maxsim.score_candidates_padded_with_argmax(q, d, qlen, dlen)
    ws, wa, gaps = oracle.score_candidates_padded(f32(q), f32(d), i64(qlen), i64(dlen), want_gap=True)
    assert s.dtype == torch.float32 and a.dtype == torch.int32
    assert_scores(f32(s), ws, name)
    assert_scores(f32(s2), ws, name, "scores(with_argmax)")
    assert_argmax(a.cpu().numpy(), wa, gaps, name)
    return s, a


def _rand_padded(B, C, Lq, Ld, dim, dtype, seed, full=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Lq, dim, generator=g).to(DEV, dtype)
    d = torch.randn(B, C, Ld, dim, generator=g).to(DEV, dtype)
    if full:
        qlen = torch.full((B,), Lq, dtype=torch.int32)
        dlen = torch.full((B, C), Ld, dtype=torch.int32)
    else:
        qlen = torch.randint(1, Lq + 1, (B,), generator=g, dtype=torch.int32)
        dlen = torch.randint(1, Ld + 1, (B, C), generator=g, dtype=torch.int32)
    return q, d, qlen.to(DEV), dlen.to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("path", [0, 1])
def test_padded_matches_oracle(dtype, path):
    q, d, qlen, dlen = _rand_padded(3, 5, 32, 100, 128, dtype, 0)
    _check_padded(q, d, qlen, dlen, dtype, path)


PADDED_EDGE = [
    (1, 1, 1, 1, 16), (1, 1, 1, 16, 16), (1, 1, 16, 1, 16), (1, 1, 16, 16, 16),
    (1, 1, 16, 17, 16), (1, 1, 16, 32, 16), (1, 1, 16, 33, 16), (1, 1, 16, 48, 16),
    (1, 1, 16, 64, 16), (1, 1, 16, 65, 16), (2, 2, 8, 24, 24), (1, 1, 32, 100, 96),
    (4, 1, 16, 32, 64), (1, 8, 16, 32, 64), (2, 3, 33, 50, 128), (1, 2, 64, 31, 32),
    (2, 2, 70, 129, 64), (1, 3, 17, 15, 32), (1, 1, 5, 300, 128),
]


@pytest.mark.parametrize("B,C,Lq,Ld,dim", PADDED_EDGE)
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_padded_edge_shapes(B, C, Lq, Ld, dim, dtype):
    q, d, qlen, dlen = _rand_padded(B, C, Lq, Ld, dim, dtype, 1, full=True)
    _check_padded(q, d, qlen, dlen, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_padded_garbage_in_padding_is_ignored(dtype):
    q, d, qlen, dlen = _rand_padded(2, 4, 32, 64, 64, dtype, 2)
    base = maxsim.score_candidates_padded(q, d, qlen, dlen)
    q2, d2 = q.clone(), d.clone()
    for b in range(q.shape[0]):
        q2[b, int(qlen[b]):] = 1e4
        for c in range(d.shape[1]):
            d2[b, c, int(dlen[b, c]):] = 1e4
    again, a = maxsim.score_candidates_padded_with_argmax(q2, d2, qlen, dlen)
    assert torch.equal(base, again)
    for b in range(q.shape[0]):
        assert (a[b, :, int(qlen[b]):] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_identical_doc_tokens_tie_to_index_zero(dtype):
    B, C, Lq, Ld, dim = 2, 3, 16, 50, 64
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, Lq, dim, generator=g).to(DEV, dtype)
    tok = torch.randn(B, C, 1, dim, generator=g).to(DEV, dtype)
    d = tok.expand(B, C, Ld, dim).contiguous()
    qlen = torch.full((B,), Lq, dtype=torch.int32, device=DEV)
    dlen = torch.full((B, C), Ld, dtype=torch.int32, device=DEV)
    _, a = maxsim.score_candidates_padded_with_argmax(q, d, qlen, dlen)
    assert (a == 0).all()
    # contrastive and packed views of the same data
    docs = d.reshape(B * C * Ld, dim)
    off = torch.arange(0, (B * C + 1) * Ld, Ld, dtype=torch.int32, device=DEV)
    _, a2 = maxsim.score_contrastive_with_argmax(q, docs, off)
    assert (a2 == 0).all()
    qoff = torch.arange(0, (B + 1) * Lq, Lq, dtype=torch.int32, device=DEV)
    pq = torch.tensor([0, 1, 1], dtype=torch.int32, device=DEV)
    pd = torch.tensor([2, 0, 5], dtype=torch.int32, device=DEV)
    _, a3 = maxsim.score_pairs_packed_with_argmax(q.reshape(B * Lq, dim), qoff, docs, off, pq, pd)
    assert (a3 == 0).all()


def _check_contrastive(q, d, off, dtype, path=0):
    _ops.set_forward_path(path)
    name = NAME_OF[dtype]
    s = maxsim.score_contrastive(q, d, off)
    s2, a = maxsim.score_contrastive_with_argmax(q, d, off)
    ws, wa, gaps = oracle.score_contrastive(f32(q), f32(d), i64(off), want_gap=True)
    assert_scores(f32(s), ws, name)
    assert_scores(f32(s2), ws, name, "scores(with_argmax)")
    assert_argmax(a.cpu().numpy(), wa, gaps, name)


def _rand_contrastive(Nq, Lq, d_lens, dim, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(Nq, Lq, dim, generator=g).to(DEV, dtype)
    d = torch.randn(sum(d_lens), dim, generator=g).to(DEV, dtype)
    off = torch.zeros(len(d_lens) + 1, dtype=torch.int32)
    off[1:] = torch.tensor(d_lens, dtype=torch.int32).cumsum(0)
    return q, d, off.to(DEV)


CONTRASTIVE_EDGE = [
    (1, 16, [16], 16), (1, 16, [1], 16), (1, 16, [17], 16), (1, 16, [16, 32, 48, 64], 32),
    (2, 16, [7, 8, 100], 32), (4, 32, [50, 50, 50, 50], 128), (1, 16, [1], 96),
    (3, 32, [1, 2, 3, 127, 128, 129, 255, 256, 257], 128), (5, 32, [300, 5, 64, 64], 128),
    (9, 32, [40] * 7, 128), (2, 48, [33, 90], 64), (3, 20, [10, 200], 128),
]


@pytest.mark.parametrize("Nq,Lq,d_lens,dim", CONTRASTIVE_EDGE)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("path", [0, 2])
def test_contrastive_edge_shapes(Nq, Lq, d_lens, dim, dtype, path):
    q, d, off = _rand_contrastive(Nq, Lq, d_lens, dim, dtype, 4)
    _check_contrastive(q, d, off, dtype, path)


def test_contrastive_fp32_is_accepted():
    q, d, off = _rand_contrastive(3, 12, [5, 40, 17], 48, torch.float32, 5)
    _check_contrastive(q, d, off, torch.float32)


def _check_packed(q, qoff, d, doff, pq, pd, dtype, path=0, max_q_len=None):
    _ops.set_forward_path(path)
    name = NAME_OF[dtype]
    s = maxsim.score_pairs_packed(q, qoff, d, doff, pq, pd, max_q_len=max_q_len)
    s2, a = maxsim.score_pairs_packed_with_argmax(q, qoff, d, doff, pq, pd, max_q_len=max_q_len)
    ws, wa, gaps = oracle.score_pairs_packed(f32(q), i64(qoff), f32(d), i64(doff), i64(pq), i64(pd),
                                             max_q_len=a.shape[1], want_gap=True)
    assert_scores(f32(s), ws, name)
    assert_scores(f32(s2), ws, name, "scores(with_argmax)")
    assert_argmax(a.cpu().numpy(), wa, gaps, name)


def _rand_packed(q_lens, d_lens, n_pairs, dim, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(sum(q_lens), dim, generator=g).to(DEV, dtype)
    d = torch.randn(sum(d_lens), dim, generator=g).to(DEV, dtype)
    qoff = torch.zeros(len(q_lens) + 1, dtype=torch.int32)
    qoff[1:] = torch.tensor(q_lens, dtype=torch.int32).cumsum(0)
    doff = torch.zeros(len(d_lens) + 1, dtype=torch.int32)
    doff[1:] = torch.tensor(d_lens, dtype=torch.int32).cumsum(0)
    pq = torch.randint(0, len(q_lens), (n_pairs,), generator=g, dtype=torch.int32)
    pd = torch.randint(0, len(d_lens), (n_pairs,), generator=g, dtype=torch.int32)
    return q, qoff.to(DEV), d, doff.to(DEV), pq.to(DEV), pd.to(DEV)


PACKED_EDGE = [
    ([1], [1], 1, 16), ([1], [100], 1, 16), ([100], [1], 1, 16), ([16], [16], 1, 24),
    ([8], [7], 1, 8), ([16, 16], [16, 16], 4, 32), ([10, 10, 10], [50] * 5, 1, 64),
    ([32] * 5, [100] * 5, 25, 128), ([8, 32, 17, 9], [8, 512, 33, 120, 64], 40, 96),
    ([40, 3], [19, 300], 6, 128),
]


@pytest.mark.parametrize("q_lens,d_lens,n_pairs,dim", PACKED_EDGE)
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
def test_packed_edge_shapes(q_lens, d_lens, n_pairs, dim, dtype):
    args = _rand_packed(q_lens, d_lens, n_pairs, dim, dtype, 6)
    _check_packed(*args, dtype)
    _check_packed(*args, dtype, max_q_len=max(q_lens) + 3)


def test_packed_int64_indices_and_empty_pairs():
    q, qoff, d, doff, pq, pd = _rand_packed([4, 9], [12, 30, 7], 5, 32, torch.float32, 7)
    a = maxsim.score_pairs_packed(q, qoff, d, doff, pq, pd)
    b = maxsim.score_pairs_packed(q, qoff.long(), d, doff.long(), pq.long(), pd.long())
    assert torch.equal(a, b)
    out = maxsim.score_pairs_packed(q, qoff, d, doff, pq[:0], pd[:0])
    assert out.shape == (0,) and out.dtype == torch.float32
    s, am = maxsim.score_pairs_packed_with_argmax(q, qoff, d, doff, pq[:0], pd[:0])
    assert s.shape == (0,) and am.shape == (0, 9)


# Random shapes, 50 per layout and dtype, with the shape distributions of the
# reference's fuzz suite (tests/test_fuzz.py:51-170 there); the contrastive one also
# draws query counts large enough for the tensor-core kernels.
FUZZ_ITERS = 50


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fuzz_padded(dtype):
    rng = random.Random(123)
    for it in range(FUZZ_ITERS):
        dim = rng.choice([16, 24, 32, 64, 96, 128])
        B, C = rng.randint(1, 4), rng.randint(1, 8)
        Lq, Ld = rng.randint(1, 64), rng.randint(1, 200)
        q, d, qlen, dlen = _rand_padded(B, C, Lq, Ld, dim, dtype, 1000 + it)
        _check_padded(q, d, qlen, dlen, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fuzz_packed(dtype):
    rng = random.Random(7777)
    for it in range(FUZZ_ITERS):
        dim = rng.choice([16, 24, 32, 64, 96, 128])
        q_lens = [rng.randint(1, 32) for _ in range(rng.randint(1, 6))]
        d_lens = [rng.randint(1, 128) for _ in range(rng.randint(1, 8))]
        args = _rand_packed(q_lens, d_lens, rng.randint(1, 16), dim, dtype, 2000 + it)
        _check_packed(*args, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fuzz_contrastive(dtype):
    rng = random.Random(31337)
    for it in range(FUZZ_ITERS):
        Lq = rng.choice([16, 32, 48, 64])
        dl = [rng.randint(1, 200) for _ in range(rng.randint(1, 8))]
        nq = rng.randint(1, 6) if it % 2 else rng.randint(8, 40)
        qc, dc, off = _rand_contrastive(nq, Lq, dl, rng.choice([16, 32, 64, 96, 128]), dtype, 3000 + it)
        _check_contrastive(qc, dc, off, dtype)


def test_non_contiguous_inputs_and_views():
    dt = torch.float16
    big_q = torch.randn(4, 16, 64, device=DEV, dtype=dt)
    big_d = torch.randn(4, 4, 32, 64, device=DEV, dtype=dt)
    q_nc, d_nc = big_q[::2], big_d[::2]
    qlen = torch.full((2,), 16, dtype=torch.int32, device=DEV)
    dlen = torch.full((2, 4), 32, dtype=torch.int32, device=DEV)
    a = maxsim.score_candidates_padded(q_nc, d_nc, qlen, dlen)
    b = maxsim.score_candidates_padded(q_nc.contiguous(), d_nc.contiguous(), qlen, dlen)
    assert torch.equal(a, b)
    # a base pointer that is only 2-byte aligned takes the portable kernel
    flat = torch.randn(64 * 64 + 1, device=DEV, dtype=dt)
    docs = flat[1:].view(64, 64)
    off = torch.tensor([0, 20, 64], dtype=torch.int32, device=DEV)
    s = maxsim.score_contrastive(big_q[:2].contiguous(), docs, off)
    ws, _ = oracle.score_contrastive(f32(big_q[:2]), f32(docs), i64(off))
    assert_scores(f32(s), ws, "fp16")
