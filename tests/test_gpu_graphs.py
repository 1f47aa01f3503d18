"""The operators inside CUDA graphs: every kernel is launched on the caller's
stream with caller-visible allocations only, and an index tensor that was
validated once is not synchronised on again, so a rerank call or a whole
contrastive train step can be captured and replayed."""

from __future__ import annotations

import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_rerank_call_replays_from_a_graph():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(8, 32, 128, generator=g).to(DEV, torch.float16)
    d = torch.randn(8, 40, 120, 128, generator=g).to(DEV, torch.float16)
    qlen = torch.randint(20, 33, (8,), generator=g, dtype=torch.int32).to(DEV)
    dlen = torch.randint(16, 121, (8, 40), generator=g, dtype=torch.int32).to(DEV)
    eager = maxsim.score_candidates_padded(q, d, qlen, dlen)  # also validates qlen / dlen once
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            maxsim.score_candidates_padded(q, d, qlen, dlen)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = maxsim.score_candidates_padded(q, d, qlen, dlen)
    d.copy_(torch.randn(d.shape, generator=g).to(DEV, torch.float16))  # new candidates, same buffers
    graph.replay()
    torch.cuda.synchronize()
    assert not torch.equal(out, eager)
    assert torch.equal(out, maxsim.score_candidates_padded(q, d, qlen, dlen))
    assert _ops.device_status() == 0


def test_contrastive_train_step_replays_from_a_graph():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(16, 32, 128, generator=g).to(DEV, torch.bfloat16).requires_grad_(True)
    d = torch.randn(16 * 50, 128, generator=g).to(DEV, torch.bfloat16).requires_grad_(True)
    off = torch.arange(0, 16 * 50 + 1, 50, dtype=torch.int32, device=DEV)

    def step():
        loss = maxsim.contrastive_loss(q, d, off, temperature=0.5)
        gq, gd = torch.autograd.grad(loss, (q, d))
        return loss, gq, gd

    # Warm up on a side stream and capture there.  (Running the step on the
    # default stream first would leave autograd nodes bound to that stream,
    # which a capture may not touch.)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        loss, gq, gd = step()
    graph.replay()
    torch.cuda.synchronize()
    want = [t.detach().clone() for t in step()]
    torch.testing.assert_close(loss, want[0], rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(gq, want[1], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(gd.float(), want[2].float(), rtol=2e-2, atol=1e-4)  # summation order
    with torch.no_grad():
        q.copy_(torch.randn(q.shape, generator=g).to(DEV, torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    fresh = step()
    torch.testing.assert_close(loss, fresh[0].detach(), rtol=1e-6, atol=1e-6)
    assert _ops.device_status() == 0


def test_packed_train_step_in_a_graph_follows_new_pair_ids():
    """The grouping of the pair list (by document and by query) must be part of
    the captured work: a replay after the id tensors were overwritten has to
    route the gradients of the NEW pairs."""
    from maxsim_b200 import workloads as W
    wl = W.c4_packed_grid_fp16(seed=9, n_queries=60, n_docs=200, n_pairs=4096, dim=96)
    assert wl.pair_query_ids.shape[0] >= _ops.GROUP_MIN_PAIRS
    q = W.to_torch(wl.queries, "fp16", DEV).requires_grad_(True)
    d = W.to_torch(wl.documents, "fp16", DEV).requires_grad_(True)
    qo = torch.from_numpy(wl.query_offsets).to(DEV)
    do = torch.from_numpy(wl.document_offsets).to(DEV)
    pq = torch.from_numpy(wl.pair_query_ids).to(DEV)
    pd = torch.from_numpy(wl.pair_document_ids).to(DEV)
    w = torch.from_numpy(wl.dscore).to(DEV)

    def step():
        s = maxsim.score_pairs_packed_train(q, qo, d, do, pq, pd, max_q_len=32)
        gq, gd = torch.autograd.grad(s, (q, d), w)
        return s, gq, gd

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        s, gq, gd = step()
    graph.replay()
    torch.cuda.synchronize()
    first = [t.detach().clone() for t in (s, gq, gd)]
    # new pair lists in the same tensors (ids stay in range, so the layout stays valid)
    gen = torch.Generator().manual_seed(3)
    pq.copy_(torch.randint(0, 60, (4096,), generator=gen, dtype=torch.int32))
    pd.copy_(torch.randint(0, 200, (4096,), generator=gen, dtype=torch.int32))
    graph.replay()
    torch.cuda.synchronize()
    assert not torch.equal(s, first[0])
    want = [t.detach() for t in step()]
    assert torch.equal(s, want[0])
    torch.testing.assert_close(gq.float(), want[1].float(), rtol=2e-2, atol=1e-3)
    torch.testing.assert_close(gd.float(), want[2].float(), rtol=2e-2, atol=1e-3)
    assert _ops.device_status() == 0


def test_graphed_contrastive_step_follows_batches_of_different_token_counts():
    torch.manual_seed(0)
    Nq, Lq, Nb, dim = 16, 32, 12, 128
    stepper = maxsim.GraphedContrastiveStep(Nq, Lq, Nb, dim, token_capacity=2000,
                                            dtype=torch.bfloat16, device=DEV, temperature=0.5)
    for it, hi in enumerate([20, 150, 60]):      # batches with different packed token counts
        lens = torch.randint(3, hi, (Nb,))
        off = torch.zeros(Nb + 1, dtype=torch.int32)
        off[1:] = lens.cumsum(0)
        q = torch.nn.functional.normalize(torch.randn(Nq, Lq, dim), dim=-1).to(DEV, torch.bfloat16)
        d = torch.nn.functional.normalize(torch.randn(int(off[-1]), dim), dim=-1).to(DEV, torch.bfloat16)
        targets = torch.randint(0, Nb, (Nq,), device=DEV) if it == 2 else None
        loss, gq, gd = stepper.step(q, d, off.to(DEV), targets)
        # the same step, eagerly
        qe, de = q.clone().requires_grad_(True), d.clone().requires_grad_(True)
        s = maxsim.score_contrastive_train(qe, de, off.to(DEV))
        want = torch.nn.functional.cross_entropy(
            s / 0.5, targets if targets is not None else torch.arange(Nq, device=DEV) % Nb)
        want.backward()
        torch.testing.assert_close(loss, want, rtol=1e-5, atol=1e-6)
        assert gd.shape == d.shape and gq.dtype == torch.bfloat16
        assert torch.equal(gq, qe.grad)
        torch.testing.assert_close(gd.float(), de.grad.float(), rtol=2.0 ** -6, atol=1e-4)
    with pytest.raises(ValueError, match="documents must be"):
        stepper.step(q, torch.zeros(2000, dim, device=DEV, dtype=torch.bfloat16), off.to(DEV))
    assert _ops.device_status() == 0
