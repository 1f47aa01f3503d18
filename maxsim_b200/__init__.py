"""maxsim_b200 -- B200-native MaxSim (ColBERT late interaction) scoring.

    score(q, d) = sum_i max_j <q_i, d_j>

A drop-in for the operator surface of the reference package
(``torch-ext/maxsim/__init__.py:38-56``): the same nine public functions with
the same argument layouts, return shapes, dtypes, exceptions and autograd
behaviour, running on hand-written sm_100a kernels behind a C ABI.

* ``score_candidates_padded[_with_argmax|_train]`` -- padded reranking,
  ``queries [B, Lq, D]`` against ``documents [B, C, Ld, D]`` with prefix lengths.
* ``score_contrastive[_with_argmax|_train]`` -- every query against every
  packed document (``document_offsets`` CSR), the in-batch training layout.
* ``score_pairs_packed[_with_argmax|_train]`` -- arbitrary (query, document)
  pair grids over ragged packed tokens.

``score_padded*`` / ``score_packed*`` are short aliases.  Scores and gradients
are always fp32; argmax is int32 and document-local; the first token reaching
the maximum wins a tie; a NaN similarity never wins.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _ops
from . import _validate as _v
from ._ops import device_status, ops
from .graphed import GraphedContrastiveStep, GraphedShardedContrastiveStep
from .layout import (pack_padded, rerank_order, rerank_topk, score_candidates_padded_from_host,
                     unpack_packed)

__all__ = [
    "score_pairs_packed", "score_pairs_packed_with_argmax", "score_pairs_packed_train",
    "score_candidates_padded", "score_candidates_padded_with_argmax",
    "score_candidates_padded_train",
    "score_contrastive", "score_contrastive_with_argmax", "score_contrastive_train",
    "score_padded", "score_padded_with_argmax", "score_padded_train",
    "score_packed", "score_packed_with_argmax", "score_packed_train",
    "lengths_from_prefix_mask", "contrastive_loss",
    "pack_padded", "unpack_packed", "rerank_topk", "rerank_order",
    "score_candidates_padded_from_host", "GraphedContrastiveStep", "GraphedShardedContrastiveStep", "device_status",
]

__version__ = "0.1.0"

# The operators call into the library through ctypes, which a tracing compiler
# cannot see through.  Marking the public functions keeps them out of
# torch.compile graphs: a compiled caller breaks the graph around them and runs
# them eagerly, as the reference's tests require (tests/test_compat.py:111-152,
# fullgraph=False).
_eager = torch.compiler.disable


# ---------------------------------------------------------------------------
# Packed pair grids (torch-ext/maxsim/__init__.py:226-508)
# ---------------------------------------------------------------------------

def _packed_prologue(queries, query_offsets, documents, document_offsets,
                     pair_query_ids, pair_document_ids, max_q_len, verbose_shapes):
    _v.check_packed_types(queries, query_offsets, documents, document_offsets,
                          pair_query_ids, pair_document_ids, verbose_shapes=verbose_shapes)
    actual = _v.check_packed_layout(queries, query_offsets, documents, document_offsets,
                                    pair_query_ids, pair_document_ids)
    return _v.resolve_max_q_len(max_q_len, actual)


@_eager
def score_pairs_packed(queries, query_offsets, documents, document_offsets,
                       pair_query_ids, pair_document_ids, *,
                       max_q_len: Optional[int] = None) -> torch.Tensor:
    """``[num_pairs]`` fp32 scores for a packed ragged batch of pairs.

    ``queries [total_q_tokens, dim]`` / ``documents [total_d_tokens, dim]``
    (same float dtype), CSR ``*_offsets`` (start at 0, end at the token count,
    no empty segment), ``pair_*_ids [num_pairs]``.  ``max_q_len``, when given,
    must be at least the longest query segment.
    """
    mql = _packed_prologue(queries, query_offsets, documents, document_offsets,
                           pair_query_ids, pair_document_ids, max_q_len, True)
    return ops.maxsim_forward(queries.contiguous(), query_offsets.contiguous(),
                              documents.contiguous(), document_offsets.contiguous(),
                              pair_query_ids.contiguous(), pair_document_ids.contiguous(), mql)


@_eager
def score_pairs_packed_with_argmax(queries, query_offsets, documents, document_offsets,
                                   pair_query_ids, pair_document_ids, *,
                                   max_q_len: Optional[int] = None
                                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """As :func:`score_pairs_packed`, plus ``argmax [num_pairs, max_q_len]``
    int32 (slots past a pair's query length are 0)."""
    mql = _packed_prologue(queries, query_offsets, documents, document_offsets,
                           pair_query_ids, pair_document_ids, max_q_len, False)
    return ops.maxsim_packed_forward_with_argmax(
        queries.contiguous(), query_offsets.contiguous(), documents.contiguous(),
        document_offsets.contiguous(), pair_query_ids.contiguous(),
        pair_document_ids.contiguous(), mql)


class _PackedFn(torch.autograd.Function):
    """Forward saves the int32 argmax; backward routes the upstream gradient
    through it.  The operator returns fp32 gradients that autograd casts to the
    leaf dtype, as in torch-ext/maxsim/__init__.py:414-454; grouped lists of
    float16 / bfloat16 tensors get them from the kernels in that dtype directly
    (every row summed in fp32, rounded once)."""

    @staticmethod
    def forward(ctx, queries, query_offsets, documents, document_offsets,
                pair_query_ids, pair_document_ids, max_q_len):
        saved = (queries.contiguous(), query_offsets.contiguous(), documents.contiguous(),
                 document_offsets.contiguous(), pair_query_ids.contiguous(),
                 pair_document_ids.contiguous())
        scores, argmax = ops.maxsim_packed_forward_with_argmax(*saved, int(max_q_len))
        ctx.save_for_backward(*saved, argmax)
        ctx.max_q_len = int(max_q_len)
        return scores

    @staticmethod
    def backward(ctx, dscore):
        q, qoff, d, doff, pq, pd, argmax = ctx.saved_tensors
        g = dscore.contiguous().to(torch.float32)
        native = _ops.packed_backward_native(g, q, qoff, d, doff, pq, pd, argmax, ctx.max_q_len)
        if native is not None:  # grouped list of 16-bit tensors: gradients already in the leaf dtype
            dq, dd = native
        else:
            dq, dd = ops.maxsim_packed_backward(g, q, qoff, d, doff, pq, pd, argmax, ctx.max_q_len)
        return dq, None, dd, None, None, None, None


@_eager
def score_pairs_packed_train(queries, query_offsets, documents, document_offsets,
                             pair_query_ids, pair_document_ids, *,
                             max_q_len: Optional[int] = None) -> torch.Tensor:
    """Differentiable :func:`score_pairs_packed` (grads to queries / documents)."""
    mql = _packed_prologue(queries, query_offsets, documents, document_offsets,
                           pair_query_ids, pair_document_ids, max_q_len, False)
    return _PackedFn.apply(queries, query_offsets, documents, document_offsets,
                           pair_query_ids, pair_document_ids, mql)


# ---------------------------------------------------------------------------
# Padded candidates (torch-ext/maxsim/__init__.py:623-801)
# ---------------------------------------------------------------------------

def _flatten_padded(queries, documents, query_lengths, doc_lengths, B, C, Lq, Ld, D):
    return (queries.reshape(B * Lq, D).contiguous(),
            query_lengths.to(dtype=torch.int32).contiguous(),
            documents.reshape(B * C * Ld, D).contiguous(),
            doc_lengths.reshape(B * C).to(dtype=torch.int32).contiguous())


@_eager
def score_candidates_padded(queries, documents, query_lengths, doc_lengths) -> torch.Tensor:
    """``[B, C]`` fp32 scores of ``queries [B, Lq, D]`` against
    ``documents [B, C, Ld, D]``; only the first ``query_lengths[b]`` /
    ``doc_lengths[b, c]`` tokens take part."""
    B, C, Lq, Ld, D = _v.check_padded(queries, documents, query_lengths, doc_lengths)
    q, qlen, d, dlen = _flatten_padded(queries, documents, query_lengths, doc_lengths,
                                       B, C, Lq, Ld, D)
    return ops.maxsim_padded_forward(q, qlen, d, dlen, int(Lq), int(Ld), int(C)).view(B, C)


@_eager
def score_candidates_padded_with_argmax(queries, documents, query_lengths, doc_lengths
                                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """As :func:`score_candidates_padded`, plus ``argmax [B, C, Lq]`` int32
    (slots past ``query_lengths[b]`` are 0)."""
    B, C, Lq, Ld, D = _v.check_padded(queries, documents, query_lengths, doc_lengths)
    q, qlen, d, dlen = _flatten_padded(queries, documents, query_lengths, doc_lengths,
                                       B, C, Lq, Ld, D)
    s, a = ops.maxsim_padded_forward_with_argmax(q, qlen, d, dlen, int(Lq), int(Ld), int(C))
    return s.view(B, C), a.view(B, C, Lq)


class _PaddedFn(torch.autograd.Function):
    """torch-ext/maxsim/__init__.py:716-771."""

    @staticmethod
    def forward(ctx, queries, documents, query_lengths, doc_lengths):
        B, Lq, D = queries.shape
        _, C, Ld, _ = documents.shape
        q, qlen, d, dlen = _flatten_padded(queries, documents, query_lengths, doc_lengths,
                                           B, C, Lq, Ld, D)
        scores, argmax = ops.maxsim_padded_forward_with_argmax(q, qlen, d, dlen,
                                                               int(Lq), int(Ld), int(C))
        ctx.save_for_backward(q, d, qlen, dlen, argmax)
        ctx.shapes = (B, C, Lq, Ld, D)
        return scores.view(B, C)

    @staticmethod
    def backward(ctx, dscore):
        B, C, Lq, Ld, D = ctx.shapes
        q, d, qlen, dlen, argmax = ctx.saved_tensors
        g = dscore.reshape(B * C).contiguous().to(torch.float32)
        # 16-bit inputs: the kernels round each gradient row once on store, which is
        # what autograd's cast of the fp32 result would give, without the extra pass
        grads = _ops.padded_backward_native(g, q, d, qlen, dlen, argmax, int(Lq), int(Ld), int(C))
        if grads is None:
            grads = ops.maxsim_padded_backward(g, q, d, qlen, dlen, argmax,
                                               int(Lq), int(Ld), int(C))
        dq, dd = grads
        return dq.view(B, Lq, D), dd.view(B, C, Ld, D), None, None


@_eager
def score_candidates_padded_train(queries, documents, query_lengths, doc_lengths) -> torch.Tensor:
    """Differentiable :func:`score_candidates_padded`."""
    _v.check_padded(queries, documents, query_lengths, doc_lengths)
    return _PaddedFn.apply(queries, documents, query_lengths, doc_lengths)


# ---------------------------------------------------------------------------
# Contrastive all-pairs (torch-ext/maxsim/__init__.py:880-979)
# ---------------------------------------------------------------------------

@_eager
def score_contrastive(queries, documents, document_offsets) -> torch.Tensor:
    """``[Nq, Nb]`` fp32 scores of every query ``[Nq, Lq, D]`` against every
    packed document (``documents [total_d_tokens, D]``, ``document_offsets [Nb+1]``)."""
    _v.check_contrastive(queries, documents, document_offsets)
    return ops.maxsim_contrastive_forward(
        queries.contiguous(), documents.contiguous(),
        document_offsets.to(dtype=torch.int32).contiguous())


@_eager
def score_contrastive_with_argmax(queries, documents, document_offsets
                                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """As :func:`score_contrastive`, plus ``argmax [Nq, Nb, Lq]`` int32."""
    _v.check_contrastive(queries, documents, document_offsets)
    return ops.maxsim_contrastive_forward_with_argmax(
        queries.contiguous(), documents.contiguous(),
        document_offsets.to(dtype=torch.int32).contiguous())


class _ContrastiveFn(torch.autograd.Function):
    """torch-ext/maxsim/__init__.py:925-954."""

    @staticmethod
    def forward(ctx, queries, documents, document_offsets):
        q = queries.contiguous()
        d = documents.contiguous()
        off = document_offsets.to(dtype=torch.int32).contiguous()
        scores, argmax = ops.maxsim_contrastive_forward_with_argmax(q, d, off)
        ctx.save_for_backward(q, d, off, argmax)
        return scores

    @staticmethod
    def backward(ctx, dscore):
        q, d, off, argmax = ctx.saved_tensors
        g = dscore.contiguous().to(torch.float32)
        grads = _ops.contrastive_backward_native(g, q, d, off, argmax)
        if grads is None:
            grads = ops.maxsim_contrastive_backward(g, q, d, off, argmax)
        return grads[0], grads[1], None


@_eager
def score_contrastive_train(queries, documents, document_offsets) -> torch.Tensor:
    """Differentiable :func:`score_contrastive`."""
    _v.check_contrastive(queries, documents, document_offsets)
    return _ContrastiveFn.apply(queries, documents, document_offsets)


# ---------------------------------------------------------------------------
# Aliases and helpers
# ---------------------------------------------------------------------------

score_padded = score_candidates_padded
score_padded_with_argmax = score_candidates_padded_with_argmax
score_padded_train = score_candidates_padded_train
score_packed = score_pairs_packed
score_packed_with_argmax = score_pairs_packed_with_argmax
score_packed_train = score_pairs_packed_train


class _ContrastiveLossFn(torch.autograd.Function):
    """Forward: scores + argmax, then one kernel that produces the mean
    cross-entropy and the gradient with respect to the scores.  Backward: the
    saved score gradient, scaled by the upstream scalar, goes straight into the
    routing kernels -- no softmax / nll kernels and no [Nq, Nb] autograd graph."""

    @staticmethod
    def forward(ctx, queries, documents, document_offsets, targets, temperature):
        q = queries.contiguous()
        d = documents.contiguous()
        off = document_offsets.to(dtype=torch.int32).contiguous()
        scores, argmax = ops.maxsim_contrastive_forward_with_argmax(q, d, off)
        loss_rows, dscore = _ops.contrastive_ce(scores, targets, temperature,
                                                1.0 / max(1, scores.shape[0]), True)
        ctx.save_for_backward(q, d, off, argmax, dscore)
        return loss_rows.mean()

    @staticmethod
    def backward(ctx, grad_out):
        q, d, off, argmax, dscore = ctx.saved_tensors
        g = dscore * grad_out.to(torch.float32)
        grads = _ops.contrastive_backward_native(g, q, d, off, argmax)
        if grads is None:
            grads = ops.maxsim_contrastive_backward(g, q, d, off, argmax)
        return grads[0], grads[1], None, None, None


@_eager
def contrastive_loss(queries, documents, document_offsets, targets=None, *,
                     temperature: float = 1.0) -> torch.Tensor:
    """Mean in-batch cross-entropy of the contrastive score matrix, fused with
    the scoring operator (an extension; the reference has no such function).

    Equivalent to ``cross_entropy(score_contrastive_train(q, d, off) /
    temperature, targets)`` with ``targets`` defaulting to ``arange(Nq)``
    (query i's positive is document i); differentiable with respect to
    ``queries`` and ``documents``."""
    _v.check_contrastive(queries, documents, document_offsets)
    if not temperature > 0:
        raise ValueError(f"temperature must be > 0; got {temperature}")
    Nq, Nb = queries.shape[0], document_offsets.numel() - 1
    if targets is None:
        if Nq > Nb:
            raise ValueError(f"default diagonal targets need Nq <= Nb; got Nq={Nq}, Nb={Nb}")
        targets = torch.arange(Nq, device=queries.device)
    elif tuple(targets.shape) != (Nq,):
        raise ValueError(f"targets must have shape [Nq={Nq}]; got {tuple(targets.shape)}")
    return _ContrastiveLossFn.apply(queries, documents, document_offsets, targets, float(temperature))


def lengths_from_prefix_mask(mask: torch.Tensor) -> torch.Tensor:
    """Convert a boolean prefix mask ``[..., L]`` (True = real token, all real
    tokens first) into int32 lengths ``[...]``.  The operators take prefix
    lengths, not masks; this helper also verifies that the mask really is a
    prefix mask and raises ``ValueError`` otherwise."""
    if mask.dtype != torch.bool:
        raise TypeError(f"mask must be bool; got {mask.dtype}")
    lengths = mask.sum(dim=-1).to(torch.int32)
    ar = torch.arange(mask.shape[-1], device=mask.device)
    expect = ar < lengths.unsqueeze(-1)
    if not bool(torch.equal(expect, mask)):
        raise ValueError("mask is not a prefix mask (a masked token precedes a real one)")
    return lengths
