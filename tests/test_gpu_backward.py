"""Backward parity on the GPU (reference: tests/test_backward.py,
test_contrastive.py:98-167, test_packed_train.py, test_edge_shapes.py:74-116).

Gradients are compared with the oracle's routing through the argmax the kernel
itself produced, which keeps the check meaningful where a near-tie lets the
argmax legitimately differ; the argmax itself is checked against the oracle in
the forward tests."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from _util import NAME_OF, assert_grads, f32, i64, oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert _ops.device_status() == 0


PADDED = [(1, 1, 16, 16, 16), (1, 1, 16, 17, 16), (1, 1, 16, 32, 16), (1, 1, 16, 64, 16),
          (1, 1, 32, 1, 16), (4, 1, 16, 33, 64), (1, 8, 32, 50, 64), (3, 7, 32, 120, 128),
          (2, 3, 9, 20, 24), (2, 2, 40, 70, 96)]


@pytest.mark.parametrize("B,C,Lq,Ld,dim", PADDED)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_padded_backward(B, C, Lq, Ld, dim, dtype):
    g = torch.Generator().manual_seed(0)
    q = torch.randn(B, Lq, dim, generator=g).to(DEV, dtype).requires_grad_(True)
    d = torch.randn(B, C, Ld, dim, generator=g).to(DEV, dtype).requires_grad_(True)
    qlen = torch.randint(1, Lq + 1, (B,), generator=g, dtype=torch.int32).to(DEV)
    dlen = torch.randint(1, Ld + 1, (B, C), generator=g, dtype=torch.int32).to(DEV)
    w = torch.randn(B, C, generator=g).to(DEV)
    scores = maxsim.score_candidates_padded_train(q, d, qlen, dlen)
    (scores * w).sum().backward()
    assert q.grad.dtype == dtype and d.grad.dtype == dtype
    _, a = maxsim.score_candidates_padded_with_argmax(q.detach(), d.detach(), qlen, dlen)
    # the op-level gradients are fp32; compare those
    dq, dd = _ops.ops.maxsim_padded_backward(
        w.reshape(-1), q.detach().reshape(B * Lq, dim), d.detach().reshape(B * C * Ld, dim),
        qlen, dlen.reshape(-1), a.reshape(B * C, Lq), Lq, Ld, C)
    assert dq.dtype == torch.float32 and dd.dtype == torch.float32
    wq, wd = oracle.candidates_padded_backward(f32(w), f32(q), f32(d), i64(qlen), i64(dlen),
                                               a.cpu().numpy())
    name = NAME_OF[dtype]
    assert_grads(f32(dq).reshape(wq.shape), wq, name, "grad_queries")
    assert_grads(f32(dd).reshape(wd.shape), wd, name, "grad_documents")
    assert_grads(f32(q.grad), wq, "bf16" if dtype != torch.float32 else "fp32", "queries.grad")
    # rows past the lengths receive exactly zero
    for b in range(B):
        assert (dq.view(B, Lq, dim)[b, int(qlen[b]):] == 0).all()
        for c in range(C):
            assert (dd.view(B, C, Ld, dim)[b, c, int(dlen[b, c]):] == 0).all()


CONTRASTIVE = [(1, 16, [16], 16), (2, 16, [7, 8, 100], 32), (4, 32, [50, 50, 50, 50], 128),
               (6, 32, [1, 65, 64, 130, 300], 128), (3, 20, [33, 5], 96), (5, 32, [70] * 9, 64)]


@pytest.mark.parametrize("Nq,Lq,d_lens,dim", CONTRASTIVE)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_contrastive_backward(Nq, Lq, d_lens, dim, dtype):
    g = torch.Generator().manual_seed(1)
    q = torch.randn(Nq, Lq, dim, generator=g).to(DEV, dtype).requires_grad_(True)
    d = torch.randn(sum(d_lens), dim, generator=g).to(DEV, dtype).requires_grad_(True)
    off = torch.zeros(len(d_lens) + 1, dtype=torch.int32)
    off[1:] = torch.tensor(d_lens, dtype=torch.int32).cumsum(0)
    off = off.to(DEV)
    w = torch.randn(Nq, len(d_lens), generator=g).to(DEV)
    scores = maxsim.score_contrastive_train(q, d, off)
    (scores * w).sum().backward()
    _, a = maxsim.score_contrastive_with_argmax(q.detach(), d.detach(), off)
    dq, dd = _ops.ops.maxsim_contrastive_backward(w, q.detach(), d.detach(), off, a)
    wq, wd = oracle.contrastive_backward(f32(w), f32(q), f32(d), i64(off), a.cpu().numpy())
    name = NAME_OF[dtype]
    assert_grads(f32(dq), wq, name, "grad_queries")
    assert_grads(f32(dd), wd, name, "grad_documents")
    assert q.grad is not None and d.grad is not None
    assert_grads(f32(d.grad), wd, "bf16" if dtype != torch.float32 else "fp32", "documents.grad")


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_packed_backward_with_duplicate_pairs(dtype):
    g = torch.Generator().manual_seed(2)
    q_lens, d_lens, dim = [8, 32, 17, 9], [8, 200, 33, 120, 64], 96
    q = torch.randn(sum(q_lens), dim, generator=g).to(DEV, dtype).requires_grad_(True)
    d = torch.randn(sum(d_lens), dim, generator=g).to(DEV, dtype).requires_grad_(True)
    qoff = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=DEV)
    doff = torch.tensor(np.concatenate([[0], np.cumsum(d_lens)]), dtype=torch.int32, device=DEV)
    pq = torch.tensor([0, 1, 1, 2, 3, 1, 0, 1], dtype=torch.int32, device=DEV)
    pd = torch.tensor([0, 1, 1, 4, 2, 3, 0, 1], dtype=torch.int32, device=DEV)  # (1,1) x3, (0,0) x2
    w = torch.randn(pq.shape[0], generator=g).to(DEV)
    scores = maxsim.score_pairs_packed_train(q, qoff, d, doff, pq, pd)
    (scores * w).sum().backward()
    s2, a = maxsim.score_pairs_packed_with_argmax(q.detach(), qoff, d.detach(), doff, pq, pd)
    assert torch.equal(scores.detach(), s2)
    dq, dd = _ops.ops.maxsim_packed_backward(w, q.detach(), qoff, d.detach(), doff, pq, pd, a,
                                             a.shape[1])
    wq, wd = oracle.pairs_packed_backward(f32(w), f32(q), i64(qoff), f32(d), i64(doff), i64(pq),
                                          i64(pd), a.cpu().numpy())
    name = NAME_OF[dtype]
    assert_grads(f32(dq), wq, name, "grad_queries")
    assert_grads(f32(dd), wd, name, "grad_documents")


@pytest.mark.parametrize("api", ["padded", "contrastive", "packed"])
def test_zero_upstream_gradient_gives_exact_zeros(api):
    dt = torch.float16
    if api == "padded":
        q = torch.randn(2, 16, 64, device=DEV, dtype=dt, requires_grad=True)
        d = torch.randn(2, 3, 40, 64, device=DEV, dtype=dt, requires_grad=True)
        qlen = torch.full((2,), 16, dtype=torch.int32, device=DEV)
        dlen = torch.full((2, 3), 40, dtype=torch.int32, device=DEV)
        s = maxsim.score_candidates_padded_train(q, d, qlen, dlen)
    elif api == "contrastive":
        q = torch.randn(3, 16, 64, device=DEV, dtype=dt, requires_grad=True)
        d = torch.randn(100, 64, device=DEV, dtype=dt, requires_grad=True)
        off = torch.tensor([0, 30, 100], dtype=torch.int32, device=DEV)
        s = maxsim.score_contrastive_train(q, d, off)
    else:
        q = torch.randn(20, 64, device=DEV, dtype=dt, requires_grad=True)
        d = torch.randn(50, 64, device=DEV, dtype=dt, requires_grad=True)
        qoff = torch.tensor([0, 8, 20], dtype=torch.int32, device=DEV)
        doff = torch.tensor([0, 25, 50], dtype=torch.int32, device=DEV)
        ids = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
        s = maxsim.score_pairs_packed_train(q, qoff, d, doff, ids, ids)
    (s * 0.0).sum().backward()
    assert (q.grad == 0).all() and (d.grad == 0).all()


def test_autocast_compile_and_stability():
    dt = torch.bfloat16
    q = torch.randn(4, 16, 64, device=DEV, dtype=dt, requires_grad=True)
    d = torch.randn(128, 64, device=DEV, dtype=dt, requires_grad=True)
    off = torch.arange(0, 160, 32, dtype=torch.int32, device=DEV)
    with torch.autocast(device_type="cuda", dtype=dt):
        loss = maxsim.score_contrastive_train(q, d, off).sum()
    loss.backward()
    assert torch.isfinite(loss) and torch.isfinite(q.grad).all() and torch.isfinite(d.grad).all()

    def step(q, d):
        return maxsim.score_contrastive_train(q, d, off).sum()

    eager = step(q.detach(), d.detach())
    out = torch.compile(step, fullgraph=False)(q.detach(), d.detach())
    torch.testing.assert_close(out, eager, rtol=1e-3, atol=1e-3)

    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    for _ in range(100):
        q.grad = None
        d.grad = None
        maxsim.score_contrastive_train(q, d, off).sum().backward()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() - base < 20 * 2 ** 20
    assert torch.isfinite(q.grad).all()


def test_autocast_and_compile_on_the_padded_and_packed_train_paths():
    """The differentiable padded and packed operators under torch.autocast and
    torch.compile(fullgraph=False) (reference: tests/test_compat.py:36-152)."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(4)
    q = torch.randn(3, 16, 64, generator=g).to(DEV, dt).requires_grad_(True)
    d = torch.randn(3, 5, 40, 64, generator=g).to(DEV, dt).requires_grad_(True)
    qlen = torch.tensor([16, 9, 12], dtype=torch.int32, device=DEV)
    dlen = torch.randint(1, 41, (3, 5), generator=g, dtype=torch.int32).to(DEV)

    def padded_step(q, d):
        return maxsim.score_candidates_padded_train(q, d, qlen, dlen).sum()

    with torch.autocast(device_type="cuda", dtype=dt):
        loss = padded_step(q, d)
    loss.backward()
    assert torch.isfinite(loss) and torch.isfinite(q.grad).all() and torch.isfinite(d.grad).all()
    eager = padded_step(q.detach(), d.detach())
    out = torch.compile(padded_step, fullgraph=False)(q.detach(), d.detach())
    torch.testing.assert_close(out, eager, rtol=1e-3, atol=1e-3)

    qp = torch.randn(30, 64, generator=g).to(DEV, dt).requires_grad_(True)
    dp = torch.randn(90, 64, generator=g).to(DEV, dt).requires_grad_(True)
    qoff = torch.tensor([0, 7, 19, 30], dtype=torch.int32, device=DEV)
    doff = torch.tensor([0, 25, 26, 60, 90], dtype=torch.int32, device=DEV)
    pq = torch.tensor([0, 2, 1, 1, 0], dtype=torch.int32, device=DEV)
    pd = torch.tensor([3, 0, 1, 3, 3], dtype=torch.int32, device=DEV)

    def packed_step(q, d):
        return maxsim.score_pairs_packed_train(q, qoff, d, doff, pq, pd).sum()

    with torch.autocast(device_type="cuda", dtype=dt):
        loss = packed_step(qp, dp)
    loss.backward()
    assert torch.isfinite(loss) and torch.isfinite(qp.grad).all() and torch.isfinite(dp.grad).all()
    eager = packed_step(qp.detach(), dp.detach())
    out = torch.compile(packed_step, fullgraph=False)(qp.detach(), dp.detach())
    torch.testing.assert_close(out, eager, rtol=1e-3, atol=1e-3)
    # gradients through the compiled functions equal the eager ones
    q2 = q.detach().clone().requires_grad_(True)
    d2 = d.detach().clone().requires_grad_(True)
    torch.compile(padded_step, fullgraph=False)(q2, d2).backward()
    assert torch.equal(q2.grad, q.grad) and torch.equal(d2.grad, d.grad)


def test_training_reduces_contrastive_loss():
    """In-batch InfoNCE on the contrastive op converges (reference:
    tests/test_train_convergence.py:90-112)."""
    torch.manual_seed(0)
    Nq, Lq, Ld, D = 16, 16, 24, 64
    q = torch.nn.Parameter(torch.randn(Nq, Lq, D, device=DEV) * 0.5)
    d = torch.nn.Parameter(torch.randn(Nq * Ld, D, device=DEV) * 0.5)
    off = torch.arange(0, (Nq + 1) * Ld, Ld, dtype=torch.int32, device=DEV)
    opt = torch.optim.Adam([q, d], lr=5e-2)
    target = torch.arange(Nq, device=DEV)
    losses = []
    for _ in range(50):
        opt.zero_grad()
        qn = torch.nn.functional.normalize(q, dim=-1).half()
        dn = torch.nn.functional.normalize(d, dim=-1).half()
        s = maxsim.score_contrastive_train(qn, dn, off)
        loss = torch.nn.functional.cross_entropy(s / 0.5, target)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.7 * losses[0], losses[::10]


@pytest.mark.parametrize("temperature", [1.0, 0.05])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_contrastive_loss_matches_cross_entropy(temperature, dtype):
    """contrastive_loss == cross_entropy(score_contrastive_train / T, targets),
    values and gradients (the unfused expression is the one the reference's
    callers write, tests/test_train_convergence.py:34-45)."""
    g = torch.Generator().manual_seed(7)
    Nq, d_lens, dim = 24, [40, 7, 130, 64, 65] * 6, 128
    qn = torch.nn.functional.normalize(torch.randn(Nq, 32, dim, generator=g), dim=-1)
    dn = torch.nn.functional.normalize(torch.randn(sum(d_lens), dim, generator=g), dim=-1)
    off = torch.tensor(np.concatenate([[0], np.cumsum(d_lens)]), dtype=torch.int32, device=DEV)
    targets = torch.randint(0, len(d_lens), (Nq,), generator=g).to(DEV)
    q1 = qn.to(DEV, dtype).requires_grad_(True)
    d1 = dn.to(DEV, dtype).requires_grad_(True)
    q2 = q1.detach().clone().requires_grad_(True)
    d2 = d1.detach().clone().requires_grad_(True)
    fused = maxsim.contrastive_loss(q1, d1, off, targets, temperature=temperature)
    (fused * 3.0).backward()
    plain = torch.nn.functional.cross_entropy(
        maxsim.score_contrastive_train(q2, d2, off) / temperature, targets)
    (plain * 3.0).backward()
    torch.testing.assert_close(fused, plain, rtol=1e-5, atol=1e-5)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=1e-4, atol=1e-5)
    scale = max(1.0, float(q2.grad.float().abs().max()))
    torch.testing.assert_close(q1.grad.float() / scale, q2.grad.float() / scale, **tol)
    scale = max(1.0, float(d2.grad.float().abs().max()))
    torch.testing.assert_close(d1.grad.float() / scale, d2.grad.float() / scale, **tol)
    # default targets are the diagonal
    a = maxsim.contrastive_loss(q1.detach(), d1.detach(), off)
    b = torch.nn.functional.cross_entropy(maxsim.score_contrastive(q1.detach(), d1.detach(), off),
                                          torch.arange(Nq, device=DEV))
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError, match="temperature"):
        maxsim.contrastive_loss(q1, d1, off, temperature=0.0)
    with pytest.raises(ValueError, match="targets"):
        maxsim.contrastive_loss(q1, d1, off, targets[:3])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_grad_queries_alone_with_argmax_entries_outside_their_document(dtype):
    """grad_queries without grad_documents (what a rank of the sharded step
    computes), fp32 and in the leaf dtype, with many query rows, documents of
    very different lengths and argmax entries outside their document, which
    route nowhere."""
    g = torch.Generator().manual_seed(7)
    Nq, Lq, dim = 1250, 32, 128
    lens = [5, 1, 800, 300, 129, 1700, 64, 2, 33]
    q = torch.randn(Nq, Lq, dim, generator=g).to(DEV, dtype)
    d = torch.randn(sum(lens), dim, generator=g).to(DEV, dtype)
    off = torch.zeros(len(lens) + 1, dtype=torch.int32)
    off[1:] = torch.tensor(lens).cumsum(0)
    off = off.to(DEV)
    w = torch.randn(Nq, len(lens), generator=g).to(DEV)
    a = torch.stack([torch.randint(0, n, (Nq, Lq), generator=g) for n in lens], dim=1).to(DEV, torch.int32)
    a[3, 2, 5] = 10 ** 6
    a[7, 0, 1] = -4
    dq, none = _ops.contrastive_backward_part(w, q, d, off, a, want_queries=True, want_documents=False)
    assert none is None
    native = _ops.contrastive_backward_native(w, q, d, off, a, want_documents=False)
    assert native is not None and native[1] is None
    assert torch.equal(native[0], dq.to(dtype))
    sel = [0, 3, 7, 640, 1249]
    wq, _ = oracle.contrastive_backward(f32(w[sel]), f32(q[sel]), f32(d), i64(off), a.cpu().numpy()[sel])
    assert_grads(f32(dq[sel]), wq, NAME_OF[dtype])
    assert _ops.device_status() == 0


@pytest.mark.parametrize("dim", [96, 64, 32, 8])
@pytest.mark.parametrize("layout", ["contrastive", "padded"])
def test_grad_queries_with_32_or_more_routed_candidates_and_narrow_rows(dim, layout):
    """Blocks of 32 candidates that are all routed take a path of the gather
    kernel without per-row checks; with dim < 128 some lanes of a half-warp
    have no element of the row and must still take part in the warp vote."""
    g = torch.Generator().manual_seed(dim)
    dt = torch.bfloat16
    if layout == "contrastive":
        Nq, Lq, Nb = 6, 16, 70
        q = torch.randn(Nq, Lq, dim, generator=g).to(DEV, dt)
        lens = torch.randint(3, 40, (Nb,), generator=g)
        d = torch.randn(int(lens.sum()), dim, generator=g).to(DEV, dt)
        off = torch.zeros(Nb + 1, dtype=torch.int32)
        off[1:] = lens.cumsum(0)
        off = off.to(DEV)
        w = torch.randn(Nq, Nb, generator=g).to(DEV)
        _, a = maxsim.score_contrastive_with_argmax(q, d, off)
        dq, dd = _ops.ops.maxsim_contrastive_backward(w, q, d, off, a)
        wq, wd = oracle.contrastive_backward(f32(w), f32(q), f32(d), i64(off), a.cpu().numpy())
    else:
        B, C, Lq, Ld = 3, 65, 16, 30
        q = torch.randn(B, Lq, dim, generator=g).to(DEV, dt)
        d = torch.randn(B, C, Ld, dim, generator=g).to(DEV, dt)
        ql = torch.full((B,), Lq, dtype=torch.int32, device=DEV)
        dl = torch.randint(1, Ld + 1, (B, C), generator=g, dtype=torch.int32).to(DEV)
        w = torch.randn(B, C, generator=g).to(DEV)
        _, a = maxsim.score_candidates_padded_with_argmax(q, d, ql, dl)
        dq, dd = _ops.ops.maxsim_padded_backward(w.reshape(-1), q.reshape(B * Lq, dim),
                                                 d.reshape(B * C * Ld, dim), ql, dl.reshape(-1),
                                                 a.reshape(B * C, Lq), Lq, Ld, C)
        wq, wd = oracle.candidates_padded_backward(f32(w), f32(q), f32(d), i64(ql), i64(dl), a.cpu().numpy())
        dq, dd = dq.view(B, Lq, dim), dd.view(B, C, Ld, dim)
    assert_grads(f32(dq), wq, "bf16")
    assert_grads(f32(dd), wd, "bf16")
    assert _ops.device_status() == 0
