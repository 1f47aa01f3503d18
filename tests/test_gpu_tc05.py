"""The tcgen05 / TMEM contrastive forward (fp16 / bf16, Lq <= 64, dim a multiple
of 16 up to 128) against the oracle and against the streaming kernel: document
boundaries at every position relative to the 128-token tiles and the 16-column
groups of the fold, partial query groups, every lanes-per-query setting, exact
ties, maxima that take the exact walk (negative, large, non-finite)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from maxsim_b200 import workloads as W
from _util import NAME_OF, assert_argmax, assert_scores, f32, i64, oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _force_tc05():
    _ops.set_forward_path(3)  # error out instead of silently taking another kernel
    yield
    _ops.set_forward_path(0)
    assert _ops.device_status() == 0, "a bounded wait ran out"


def _make(Nq, d_lens, dtype, seed, Lq=32, dim=128, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (scale * torch.randn(Nq, Lq, dim, generator=g)).to(DEV, dtype)
    d = torch.randn(sum(d_lens), dim, generator=g).to(DEV, dtype)
    off = torch.zeros(len(d_lens) + 1, dtype=torch.int32)
    off[1:] = torch.tensor(d_lens, dtype=torch.int32).cumsum(0)
    return q, d, off.to(DEV)


def _check(q, d, off, dtype):
    name = NAME_OF[dtype]
    s = maxsim.score_contrastive(q, d, off)
    s2, a = maxsim.score_contrastive_with_argmax(q, d, off)
    ws, wa, gaps = oracle.score_contrastive(f32(q), f32(d), i64(off), want_gap=True)
    assert_scores(f32(s), ws, name)
    assert_scores(f32(s2), ws, name, "scores(with_argmax)")
    assert_argmax(a.cpu().numpy(), wa, gaps, name)
    return s2, a


SHAPES = [
    (8, [128]), (8, [1]), (8, [127, 129]), (8, [1, 1, 1, 1, 1]), (9, [40] * 7),
    (16, [31, 32, 33, 63, 64, 65, 95, 96, 97, 255, 256, 257]),
    (12, [600, 3, 1100, 17]), (70, [50, 60, 70, 80] * 5), (8, [5] * 100),
    (33, [200] * 40), (64, [300, 1, 299, 2, 512, 511, 513]),
]


@pytest.mark.parametrize("Nq,d_lens", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
# 3: tcgen05 kernel with the tiling chosen by document length, 8: every document tiled on
# its own, 9: 128-token tiles that ignore document boundaries
@pytest.mark.parametrize("path", [3, 8, 9])
def test_tc05_matches_oracle(Nq, d_lens, dtype, path):
    _ops.set_forward_path(path)
    q, d, off = _make(Nq, d_lens, dtype, 11)
    _check(q, d, off, dtype)


# query lengths on 16, 32 and 64 accumulator lanes (exact fits and zero-filled rows) and
# every dim the operand boxes cover (one box, a zero-filled second box, two boxes)
@pytest.mark.parametrize("Lq,dim", [(16, 128), (7, 64), (20, 96), (32, 64), (32, 96), (32, 16),
                                    (48, 128), (64, 128), (64, 96), (33, 48), (1, 32)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("path", [8, 9])
def test_tc05_query_lengths_and_dims(Lq, dim, dtype, path):
    _ops.set_forward_path(path)
    for Nq, d_lens in ((16, [31, 200, 128, 5, 129, 64, 1, 300]), (37, [90] * 9 + [17])):
        q, d, off = _make(Nq, d_lens, dtype, 17 + Lq, Lq=Lq, dim=dim)
        _check(q, d, off, dtype)


@pytest.mark.parametrize("Lq,dim", [(64, 96), (16, 64), (48, 128), (32, 128)])
@pytest.mark.parametrize("path", [8, 9])
def test_tc05_many_items_per_cta(Lq, dim, path):
    """More work items than SMs, several documents per item: every CTA walks its
    item loop many times (query block reloads, barrier phases that wrap, the
    hand-over ring of queries that span two warps)."""
    _ops.set_forward_path(path)
    g = torch.Generator().manual_seed(Lq + dim)
    d_lens = torch.randint(1, 90, (700,), generator=g).tolist()
    q, d, off = _make(640, d_lens, torch.bfloat16, 23, Lq=Lq, dim=dim)
    s, a = maxsim.score_contrastive_with_argmax(q, d, off)
    s0 = maxsim.score_contrastive(q, d, off)
    sel = torch.arange(0, 640, 97)
    ws, wa, gaps = oracle.score_contrastive(f32(q[sel]), f32(d), i64(off), want_gap=True)
    assert_scores(f32(s[sel]), ws, "bf16")
    assert_scores(f32(s0[sel]), ws, "bf16")
    assert_argmax(a[sel].cpu().numpy(), wa, gaps, "bf16")
    # every pair against the streaming kernel
    _ops.set_forward_path(2)
    s_mma, a_mma = maxsim.score_contrastive_with_argmax(q, d, off)
    torch.testing.assert_close(s, s_mma, rtol=1e-4, atol=2e-3)
    assert (a != a_mma).float().mean() < 2e-3


@pytest.mark.parametrize("path", [8, 9])
@pytest.mark.parametrize("Lq", [16, 32, 64])
def test_tc05_large_and_negative_maxima_take_the_exact_walk(path, Lq):
    _ops.set_forward_path(path)
    # similarities of magnitude well above 64: compared exactly, first index wins
    q, d, off = _make(16, [150, 40, 129, 256, 3], torch.bfloat16, 31, Lq=Lq, scale=8.0)
    s, a = _check(q, d, off, torch.bfloat16)
    assert float(s.abs().max()) > 64 * Lq / 4
    # every similarity negative: documents are copies of -q direction mixtures
    g = torch.Generator().manual_seed(5)
    base = torch.randn(1, 128, generator=g)
    qn = (base + 0.05 * torch.randn(16, Lq, 128, generator=g)).to(DEV, torch.float16)
    dn = (-base + 0.05 * torch.randn(400, 128, generator=g)).to(DEV, torch.float16)
    offn = torch.tensor([0, 130, 131, 300, 400], dtype=torch.int32, device=DEV)
    s, a = _check(qn, dn, offn, torch.float16)
    assert float(s.max()) < 0
    # duplicated tokens with a negative maximum: the first copy wins
    dn2 = dn.clone()
    dn2[200:300] = dn2[131:132]
    _, a2 = maxsim.score_contrastive_with_argmax(qn[:, :, :], dn2[131:300].contiguous(),
                                                 torch.tensor([0, 169], dtype=torch.int32, device=DEV))
    ws, wa, gaps = oracle.score_contrastive(f32(qn), f32(dn2[131:300]), np.array([0, 169]), want_gap=True)
    exact = gaps == 0
    assert np.array_equal(a2.cpu().numpy()[exact], wa[exact])


def test_tc05_agrees_with_streaming_kernel_bitwise_on_argmax():
    q, d, off = _make(24, [90, 130, 7, 256, 300, 64], torch.bfloat16, 12)
    s_tc, a_tc = maxsim.score_contrastive_with_argmax(q, d, off)
    _ops.set_forward_path(2)
    s_mma, a_mma = maxsim.score_contrastive_with_argmax(q, d, off)
    _ops.set_forward_path(3)
    torch.testing.assert_close(s_tc, s_mma, rtol=1e-4, atol=1e-4)
    assert (a_tc != a_mma).float().mean() < 1e-3


@pytest.mark.parametrize("path", [8, 9])
def test_tc05_exact_ties_and_duplicated_tokens(path):
    _ops.set_forward_path(path)
    wl = W.c5_contrastive_ties_bf16(seed=21, Nq=16, Nb=24, lo=20, hi=300, dup_frac=0.1)
    q = W.to_torch(wl.queries, "bf16", DEV)
    d = W.to_torch(wl.documents, "bf16", DEV)
    off = torch.from_numpy(wl.document_offsets).to(DEV)
    s, a = maxsim.score_contrastive_with_argmax(q, d, off)
    ws, wa, gaps = oracle.score_contrastive(f32(q), f32(d), wl.document_offsets, want_gap=True)
    assert_scores(f32(s), ws, "bf16")
    # duplicated tokens are exact ties: the lower index has to win every time
    exact = gaps == 0
    assert exact.sum() > 0
    assert np.array_equal(a.cpu().numpy()[exact], wa[exact])
    assert_argmax(a.cpu().numpy(), wa, gaps, "bf16")
    # all-identical documents: argmax 0 everywhere
    tok = torch.randn(1, 128, device=DEV).to(torch.float16)
    d2 = tok.expand(700, 128).contiguous()
    off2 = torch.tensor([0, 100, 357, 700], dtype=torch.int32, device=DEV)
    _, a2 = maxsim.score_contrastive_with_argmax(q.to(torch.float16), d2, off2)
    assert (a2 == 0).all()


@pytest.mark.parametrize("path", [8, 9])
def test_tc05_non_finite_contract(path):
    _ops.set_forward_path(path)
    q, d, off = _make(16, [64, 200, 33], torch.float16, 13)
    q[3, 5, 7] = float("nan")
    d[70, 1] = float("nan")
    s, a = maxsim.score_contrastive_with_argmax(q, d, off)
    assert torch.isinf(s[3]).all() and (s[3] < 0).all()
    ok = torch.ones(16, dtype=torch.bool)
    ok[3] = False
    assert torch.isfinite(s[ok]).all()
    assert (a[3, :, 5] == 0).all()
    assert (a[ok][:, 1, :] != 6).all()  # token 70 is index 6 of document 1
    ws, wa = oracle.score_contrastive(f32(q), f32(d), i64(off))
    assert_scores(f32(s), ws, "fp16")
    q2, d2, off2 = _make(8, [40, 40], torch.float16, 14)
    q2[0, 0] = float("inf")
    s2 = maxsim.score_contrastive(q2, d2.abs(), off2)
    assert torch.isinf(s2[0]).all() and (s2[0] > 0).all() and torch.isfinite(s2[1:]).all()


def test_tc05_train_step_backward():
    q, d, off = _make(16, [64, 200, 33, 128, 129], torch.bfloat16, 15)
    q.requires_grad_(True)
    d.requires_grad_(True)
    s = maxsim.score_contrastive_train(q, d, off)
    w = torch.randn_like(s)
    (s * w).sum().backward()
    _, a = maxsim.score_contrastive_with_argmax(q.detach(), d.detach(), off)
    wq, wd = oracle.contrastive_backward(f32(w), f32(q), f32(d), i64(off), a.cpu().numpy())
    from _util import assert_grads
    assert_grads(f32(q.grad), wq, "bf16")
    assert_grads(f32(d.grad), wd, "bf16")
