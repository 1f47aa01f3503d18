"""Non-finite contract (reference: tests/test_nan_inf.py:33-146): a NaN query
token gives -inf scores for every pair touching that query and nothing else; a
NaN document token is ignored; +inf propagates; a NaN forward gives non-finite
gradients.  Checked for every forward kernel family."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from _util import assert_scores, f32, i64, oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _reset():
    yield
    _ops.set_forward_path(0)
    assert _ops.device_status() == 0


@pytest.mark.parametrize("path", [0, 1, 2])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_nan_query_token_gives_neg_inf(path, dtype):
    if dtype == torch.float32 and path == 2:
        pytest.skip("fp32 always takes the portable kernel")
    _ops.set_forward_path(path)
    torch.manual_seed(0)
    B, C, Lq, Ld, D = 2, 3, 32, 40, 128
    q = torch.randn(B, Lq, D, device=DEV, dtype=dtype)
    d = torch.randn(B, C, Ld, D, device=DEV, dtype=dtype)
    qlen = torch.full((B,), Lq, dtype=torch.int32, device=DEV)
    dlen = torch.full((B, C), Ld, dtype=torch.int32, device=DEV)
    q[1, 0, 0] = float("nan")
    s, a = maxsim.score_candidates_padded_with_argmax(q, d, qlen, dlen)
    assert torch.isinf(s[1]).all() and (s[1] < 0).all()
    assert torch.isfinite(s[0]).all()
    assert (a[1, :, 0] == 0).all()
    ws, wa = oracle.score_candidates_padded(f32(q), f32(d), i64(qlen), i64(dlen))
    assert_scores(f32(s), ws, "fp16")

    docs = d.reshape(B * C * Ld, D)
    off = torch.arange(0, (B * C + 1) * Ld, Ld, dtype=torch.int32, device=DEV)
    s2 = maxsim.score_contrastive(q, docs, off)
    assert torch.isinf(s2[1]).all() and (s2[1] < 0).all() and torch.isfinite(s2[0]).all()

    qoff = torch.arange(0, (B + 1) * Lq, Lq, dtype=torch.int32, device=DEV)
    pq = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pd = torch.tensor([0, 0], dtype=torch.int32, device=DEV)
    s3 = maxsim.score_pairs_packed(q.reshape(B * Lq, D), qoff, docs, off, pq, pd, max_q_len=Lq)
    assert torch.isfinite(s3[0]) and torch.isinf(s3[1]) and s3[1] < 0


@pytest.mark.parametrize("path", [0, 1])
def test_nan_document_token_is_ignored(path):
    _ops.set_forward_path(path)
    torch.manual_seed(1)
    q = torch.randn(2, 32, 64, device=DEV, dtype=torch.float16)
    d = torch.randn(90, 64, device=DEV, dtype=torch.float16)
    off = torch.tensor([0, 30, 90], dtype=torch.int32, device=DEV)
    d[5, 3] = float("nan")
    s, a = maxsim.score_contrastive_with_argmax(q, d, off)
    assert torch.isfinite(s).all()
    assert (a[:, 0, :] != 5).all()
    ws, wa = oracle.score_contrastive(f32(q), f32(d), i64(off))
    assert_scores(f32(s), ws, "fp16")
    assert np.array_equal(a.cpu().numpy(), wa)


@pytest.mark.parametrize("path", [0, 1])
def test_pos_inf_propagates(path):
    _ops.set_forward_path(path)
    torch.manual_seed(2)
    q = torch.randn(1, 16, 64, device=DEV, dtype=torch.float16)
    d = torch.randn(64, 64, device=DEV, dtype=torch.float16).abs()
    off = torch.tensor([0, 32, 64], dtype=torch.int32, device=DEV)
    q[0, 0] = float("inf")
    s = maxsim.score_contrastive(q, d, off)
    assert torch.isinf(s).all() and (s > 0).all()


def test_nan_forward_gives_nonfinite_grads():
    torch.manual_seed(3)
    q = torch.randn(1, 16, 64, device=DEV, dtype=torch.float16, requires_grad=True)
    d = torch.randn(64, 64, device=DEV, dtype=torch.float16, requires_grad=True)
    off = torch.tensor([0, 32, 64], dtype=torch.int32, device=DEV)
    with torch.no_grad():
        q[0, 0, 0] = float("nan")
    maxsim.score_contrastive_train(q, d, off).sum().backward()
    assert not torch.isfinite(q.grad).all() or not torch.isfinite(d.grad).all()
