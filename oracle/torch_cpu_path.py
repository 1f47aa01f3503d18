"""The reference's PyTorch CPU formulation of MaxSim -- TEST/BENCH INFRASTRUCTURE.

The reference's benchmark measures its kernels against "the natural way to
write MaxSim in PyTorch": one batched ``einsum`` that materialises the whole
similarity tensor, a mask, ``max(dim=-1)`` and a sum
(``scripts/bench_matrix.py:302-313`` for the contrastive layout and
``scripts/bench_matrix.py:402-413`` for the padded layout).  This file restates
those two expressions so that the benchmark can time them on the host cores as
the CPU baseline.  Queries are processed in chunks so that the similarity
tensor fits in host memory at the large configurations; the arithmetic per
pair is unchanged.

Only ``bench.py`` (CPU-baseline leg and ``--impl reference``) and the tests
use this module; the shipped package never imports it.
"""

from __future__ import annotations

import torch


def padded_scores(queries, documents, query_lengths, doc_lengths, chunk=4):
    """[B, C] scores; formulation of scripts/bench_matrix.py:402-413."""
    B, C, Ld, _ = documents.shape
    Lq = queries.shape[1]
    out = torch.empty((B, C), dtype=torch.float32)
    ar_q = torch.arange(Lq)
    ar_d = torch.arange(Ld)
    for b0 in range(0, B, chunk):
        b1 = min(B, b0 + chunk)
        q = queries[b0:b1].float()
        d = documents[b0:b1].float()
        sim = torch.einsum("bid,bcjd->bcij", q, d)
        q_mask = ar_q[None, :] < query_lengths[b0:b1, None]
        d_mask = ar_d[None, None, :] < doc_lengths[b0:b1, :, None]
        sim = sim.masked_fill(~d_mask[:, :, None, :], float("-inf"))
        per_q = sim.max(dim=-1).values
        per_q = per_q.masked_fill(~q_mask[:, None, :], 0.0)
        out[b0:b1] = per_q.sum(dim=-1)
    return out


def _pad_documents(documents, document_offsets):
    offs = document_offsets.to(torch.int64).tolist()
    lens = [offs[i + 1] - offs[i] for i in range(len(offs) - 1)]
    Ld = max(lens)
    padded = documents.new_zeros((len(lens), Ld, documents.shape[1]))
    mask = torch.zeros((len(lens), Ld), dtype=torch.bool)
    for i, n in enumerate(lens):
        padded[i, :n] = documents[offs[i]:offs[i + 1]]
        mask[i, :n] = True
    return padded, mask


def contrastive_scores(queries, documents, document_offsets, chunk=8):
    """[Nq, Nb] scores; formulation of scripts/bench_matrix.py:302-313, with
    the padding rows masked to -inf so ragged documents score exactly."""
    padded, mask = _pad_documents(documents, document_offsets)
    pf = padded.float()
    rows = []
    for q0 in range(0, queries.shape[0], chunk):
        sim = torch.einsum("qid,njd->qnij", queries[q0:q0 + chunk].float(), pf)
        sim = sim.masked_fill(~mask[None, :, None, :], float("-inf"))
        rows.append(sim.max(dim=-1).values.sum(dim=-1))
    return torch.cat(rows, dim=0)


def contrastive_train_step(queries, documents, document_offsets, chunk=8):
    """Forward + backward of the diagonal-target cross-entropy through the
    einsum formulation; returns (loss, grad_queries, grad_documents)."""
    q = queries.detach().float().requires_grad_(True)
    d = documents.detach().float().requires_grad_(True)
    offs = document_offsets.to(torch.int64).tolist()
    lens = [offs[i + 1] - offs[i] for i in range(len(offs) - 1)]
    Ld = max(lens)
    idx = torch.zeros((len(lens), Ld), dtype=torch.int64)
    mask = torch.zeros((len(lens), Ld), dtype=torch.bool)
    for i, n in enumerate(lens):
        idx[i, :n] = torch.arange(offs[i], offs[i + 1])
        mask[i, :n] = True
    pf = d[idx]                                   # differentiable gather-pad
    rows = []
    for q0 in range(0, q.shape[0], chunk):
        sim = torch.einsum("qid,njd->qnij", q[q0:q0 + chunk], pf)
        sim = sim.masked_fill(~mask[None, :, None, :], float("-inf"))
        rows.append(sim.max(dim=-1).values.sum(dim=-1))
    scores = torch.cat(rows, dim=0)
    target = torch.arange(scores.shape[0]) % scores.shape[1]
    loss = torch.nn.functional.cross_entropy(scores, target)
    loss.backward()
    return loss.detach(), q.grad, d.grad
