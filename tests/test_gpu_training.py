"""Training-loop behaviour the reference pins: hundreds of forward+backward
iterations stay finite and do not leak device memory on any of the three
surfaces (reference: tests/test_stability.py:44-134), and a model trained
through the kernels follows the loss curve of the same model trained through
an autograd einsum formulation (reference: tests/test_train_convergence.py:115-147)."""

from __future__ import annotations

import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(api, dtype):
    g = torch.Generator().manual_seed(5)
    if api == "padded":
        q = torch.randn(4, 32, 128, generator=g).to(DEV, dtype).requires_grad_(True)
        d = torch.randn(4, 8, 96, 128, generator=g).to(DEV, dtype).requires_grad_(True)
        qlen = torch.randint(8, 33, (4,), generator=g, dtype=torch.int32).to(DEV)
        dlen = torch.randint(16, 97, (4, 8), generator=g, dtype=torch.int32).to(DEV)
        return (q, d), lambda: maxsim.score_candidates_padded_train(q, d, qlen, dlen)
    if api == "contrastive":
        q = torch.randn(16, 32, 128, generator=g).to(DEV, dtype).requires_grad_(True)
        d = torch.randn(16 * 60, 128, generator=g).to(DEV, dtype).requires_grad_(True)
        off = torch.arange(0, 16 * 60 + 1, 60, dtype=torch.int32, device=DEV)
        return (q, d), lambda: maxsim.score_contrastive_train(q, d, off)
    q = torch.randn(10 * 20, 96, generator=g).to(DEV, dtype).requires_grad_(True)
    d = torch.randn(12 * 50, 96, generator=g).to(DEV, dtype).requires_grad_(True)
    qoff = torch.arange(0, 201, 20, dtype=torch.int32, device=DEV)
    doff = torch.arange(0, 601, 50, dtype=torch.int32, device=DEV)
    pq = torch.randint(0, 10, (64,), generator=g, dtype=torch.int32).to(DEV)
    pd = torch.randint(0, 12, (64,), generator=g, dtype=torch.int32).to(DEV)
    return (q, d), lambda: maxsim.score_pairs_packed_train(q, qoff, d, doff, pq, pd, max_q_len=20)


@pytest.mark.parametrize("api", ["padded", "contrastive", "packed"])
def test_two_hundred_steps_stay_finite_and_do_not_leak(api):
    (q, d), forward = _inputs(api, torch.float16)
    for _ in range(5):
        q.grad = d.grad = None
        forward().sum().backward()
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    for _ in range(200):
        q.grad = d.grad = None
        s = forward()
        s.sum().backward()
    torch.cuda.synchronize()
    assert torch.isfinite(s).all() and torch.isfinite(q.grad).all() and torch.isfinite(d.grad).all()
    assert torch.cuda.memory_allocated() - base < 20 * 2 ** 20
    assert _ops.device_status() == 0


def _einsum_scores(q, d, Ld):
    sim = torch.einsum("qid,njd->qnij", q, d.view(-1, Ld, d.shape[-1]))
    return sim.max(dim=-1).values.sum(dim=-1)


def test_kernel_trained_model_tracks_autograd_trained_model():
    torch.manual_seed(1)
    Nq, Lq, Ld, D = 16, 16, 24, 64
    q0 = torch.randn(Nq, Lq, D, device=DEV) * 0.5
    d0 = torch.randn(Nq * Ld, D, device=DEV) * 0.5
    off = torch.arange(0, (Nq + 1) * Ld, Ld, dtype=torch.int32, device=DEV)
    target = torch.arange(Nq, device=DEV)
    curves = []
    for use_kernel in (True, False):
        q = torch.nn.Parameter(q0.clone())
        d = torch.nn.Parameter(d0.clone())
        opt = torch.optim.SGD([q, d], lr=0.5)
        losses = []
        for _ in range(40):
            opt.zero_grad()
            qn = torch.nn.functional.normalize(q, dim=-1)
            dn = torch.nn.functional.normalize(d, dim=-1)
            if use_kernel:
                loss = maxsim.contrastive_loss(qn, dn, off, temperature=0.5)
            else:
                loss = torch.nn.functional.cross_entropy(_einsum_scores(qn, dn, Ld) / 0.5, target)
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
        curves.append(losses)
    kernel, plain = curves
    assert kernel[-1] < 0.7 * kernel[0]
    for a, b in zip(kernel, plain):
        assert abs(a - b) <= 5e-3 + 2e-2 * abs(b), (kernel[::8], plain[::8])
