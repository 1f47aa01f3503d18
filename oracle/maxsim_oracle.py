"""CPU oracle for MaxSim late interaction -- TEST INFRASTRUCTURE, NOT PRODUCT.

This module is a numpy restatement of the reference's algorithm for the
MaxSim path.  It exists only so that tests, the smoke check and the
benchmark's CPU-baseline leg can check (or time) something that is *not* the
CUDA library.  Nothing in the shipped package imports it.

Parity status: PINNED.  ``tests/golden/*.npz`` hold outputs produced by the
reference's own pure-PyTorch implementation (``torch-ext/maxsim/reference.py``)
on seeded inputs; ``tests/test_oracle_golden.py`` checks every function here
against them.  ``tests/golden/make_golden.py`` is the script that made them.

What it follows (paths are relative to the reference checkout):

* pair score / argmax ............ ``torch-ext/maxsim/reference.py:20-47``
  (``q.float() @ d.float().T`` -> ``max(dim=-1)`` -> ``sum``; first index wins)
* packed pair grids .............. ``torch-ext/maxsim/reference.py:50-109``
* padded candidates .............. ``torch-ext/maxsim/reference.py:112-138, 326-361``
* contrastive all-pairs .......... ``torch-ext/maxsim/reference.py:232-281``
* backward routing ............... ``torch-ext/maxsim/reference.py:141-229, 284-323``

One deliberate difference, documented by the reference itself
(``tests/test_nan_inf.py:33-92``, ``README.md:557-562``): the reference
*kernels* never let a NaN similarity win a max (they start from -inf and
update with a strict ``>``), whereas ``torch.max`` propagates NaN.  The
kernel's tested contract is the one a drop-in has to meet, so this oracle
treats NaN similarities as "never wins": a NaN query token gives a -inf
row maximum with argmax 0, a NaN document token is ignored.  On finite
inputs both formulations agree exactly.

All functions take and return numpy arrays.  Token matrices are float32
arrays whose values already lie on the grid of the dtype under test (cast to
fp16/bf16 and back before calling), so the products formed here are the same
real numbers the tensor cores multiply.
"""

from __future__ import annotations

import numpy as np

__all__ = [
    "pair_score_argmax",
    "score_pairs_packed",
    "score_candidates_padded",
    "score_contrastive",
    "pairs_packed_backward",
    "candidates_padded_backward",
    "contrastive_backward",
    "top2_gap_pair",
    "argmax_mismatch_allowed",
]

_NEG_INF = np.float32(-np.inf)


def _sim(q: np.ndarray, d: np.ndarray) -> np.ndarray:
    """[Lq, Ld] float32 similarities (reference.py:30)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    d = np.ascontiguousarray(d, dtype=np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        return q @ d.T


def _rowmax_first(sim: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Row maximum with strict-greater-from-minus-infinity semantics.

    Mirrors ``sim.max(dim=-1)`` of reference.py:46 on finite data (first index
    wins) and the kernels' NaN contract otherwise (NaN never wins).
    """
    clean = np.where(np.isnan(sim), _NEG_INF, sim)
    idx = np.argmax(clean, axis=-1).astype(np.int32)  # first occurrence
    vals = np.take_along_axis(clean, idx[..., None].astype(np.int64), axis=-1)[..., 0]
    # A row that never rises above -inf keeps the initial index 0.
    idx = np.where(vals == _NEG_INF, np.int32(0), idx).astype(np.int32)
    return vals.astype(np.float32), idx


def _sum_rows(vals: np.ndarray) -> np.float32:
    with np.errstate(invalid="ignore", over="ignore"):
        return np.float32(np.sum(vals, dtype=np.float32))


def pair_score_argmax(q: np.ndarray, d: np.ndarray) -> tuple[np.float32, np.ndarray]:
    """One (query, document) pair: reference.py:34-47."""
    vals, idx = _rowmax_first(_sim(q, d))
    return _sum_rows(vals), idx


def top2_gap_pair(q: np.ndarray, d: np.ndarray) -> np.ndarray:
    """Per query token: best similarity minus the best similarity found at a
    *different* document index (inf when the document has one token).  Used by
    the tests to apply the argmax exemption for near-ties."""
    sim = _sim(q, d)
    clean = np.where(np.isnan(sim), _NEG_INF, sim)
    if clean.shape[1] < 2:
        return np.full(clean.shape[0], np.inf, dtype=np.float32)
    part = np.partition(clean, clean.shape[1] - 2, axis=1)
    with np.errstate(invalid="ignore"):
        gap = part[:, -1] - part[:, -2]
    return np.where(np.isnan(gap), 0.0, gap).astype(np.float32)


# ---------------------------------------------------------------------------
# Packed pair grids (reference.py:50-109)
# ---------------------------------------------------------------------------

def score_pairs_packed(queries, query_offsets, documents, document_offsets,
                       pair_query_ids, pair_document_ids, max_q_len=None,
                       want_gap=False):
    qoff = np.asarray(query_offsets, dtype=np.int64)
    doff = np.asarray(document_offsets, dtype=np.int64)
    qids = np.asarray(pair_query_ids, dtype=np.int64)
    dids = np.asarray(pair_document_ids, dtype=np.int64)
    n = qids.shape[0]
    if max_q_len is None:
        max_q_len = int(np.max(np.diff(qoff))) if qoff.size > 1 else 0
    scores = np.empty(n, dtype=np.float32)
    argmax = np.zeros((n, max_q_len), dtype=np.int32)
    gaps = np.full((n, max_q_len), np.inf, dtype=np.float32) if want_gap else None
    for k in range(n):
        q = queries[qoff[qids[k]]:qoff[qids[k] + 1]]
        d = documents[doff[dids[k]]:doff[dids[k] + 1]]
        s, a = pair_score_argmax(q, d)
        scores[k] = s
        argmax[k, :a.shape[0]] = a
        if want_gap:
            gaps[k, :a.shape[0]] = top2_gap_pair(q, d)
    if want_gap:
        return scores, argmax, gaps
    return scores, argmax


def pairs_packed_backward(dscore, queries, query_offsets, documents,
                          document_offsets, pair_query_ids, pair_document_ids,
                          argmax):
    """reference.py:186-229.  Duplicate pairs accumulate independently."""
    qoff = np.asarray(query_offsets, dtype=np.int64)
    doff = np.asarray(document_offsets, dtype=np.int64)
    qids = np.asarray(pair_query_ids, dtype=np.int64)
    dids = np.asarray(pair_document_ids, dtype=np.int64)
    q = np.asarray(queries, dtype=np.float32)
    d = np.asarray(documents, dtype=np.float32)
    g = np.asarray(dscore, dtype=np.float32)
    dq = np.zeros(q.shape, dtype=np.float64)
    dd = np.zeros(d.shape, dtype=np.float64)
    with np.errstate(invalid="ignore", over="ignore"):
        for k in range(qids.shape[0]):
            qs, qe = qoff[qids[k]], qoff[qids[k] + 1]
            ds, de = doff[dids[k]], doff[dids[k] + 1]
            lq, ld = qe - qs, de - ds
            a = np.asarray(argmax[k, :lq], dtype=np.int64)
            ok = (a >= 0) & (a < ld)
            rows = np.nonzero(ok)[0]
            np.add.at(dq, qs + rows, g[k] * d[ds + a[rows]])
            np.add.at(dd, ds + a[rows], g[k] * q[qs + rows])
    return dq.astype(np.float32), dd.astype(np.float32)


# ---------------------------------------------------------------------------
# Padded candidates (reference.py:112-138, 326-361)
# ---------------------------------------------------------------------------

def score_candidates_padded(queries, documents, query_lengths, doc_lengths,
                            want_gap=False):
    B, C = np.asarray(doc_lengths).shape
    Lq = queries.shape[1]
    qlen = np.asarray(query_lengths, dtype=np.int64)
    dlen = np.asarray(doc_lengths, dtype=np.int64)
    scores = np.empty((B, C), dtype=np.float32)
    argmax = np.zeros((B, C, Lq), dtype=np.int32)
    gaps = np.full((B, C, Lq), np.inf, dtype=np.float32) if want_gap else None
    for b in range(B):
        q = queries[b, :qlen[b]]
        for c in range(C):
            d = documents[b, c, :dlen[b, c]]
            s, a = pair_score_argmax(q, d)
            scores[b, c] = s
            argmax[b, c, :a.shape[0]] = a
            if want_gap:
                gaps[b, c, :a.shape[0]] = top2_gap_pair(q, d)
    if want_gap:
        return scores, argmax, gaps
    return scores, argmax


def candidates_padded_backward(dscore, queries, documents, query_lengths,
                               doc_lengths, argmax):
    """reference.py:141-183."""
    q = np.asarray(queries, dtype=np.float32)
    d = np.asarray(documents, dtype=np.float32)
    g = np.asarray(dscore, dtype=np.float32)
    B, C = np.asarray(doc_lengths).shape
    qlen = np.asarray(query_lengths, dtype=np.int64)
    dlen = np.asarray(doc_lengths, dtype=np.int64)
    dq = np.zeros(q.shape, dtype=np.float64)
    dd = np.zeros(d.shape, dtype=np.float64)
    with np.errstate(invalid="ignore", over="ignore"):
        for b in range(B):
            for c in range(C):
                a = np.asarray(argmax[b, c, :qlen[b]], dtype=np.int64)
                ok = (a >= 0) & (a < dlen[b, c])
                rows = np.nonzero(ok)[0]
                np.add.at(dq[b], rows, g[b, c] * d[b, c, a[rows]])
                np.add.at(dd[b, c], a[rows], g[b, c] * q[b, rows])
    return dq.astype(np.float32), dd.astype(np.float32)


# ---------------------------------------------------------------------------
# Contrastive all-pairs (reference.py:232-281), vectorised per query
# ---------------------------------------------------------------------------

def score_contrastive(queries, documents, document_offsets, want_gap=False):
    """Every query against every packed document.

    One [Lq, T_d] product per query followed by segmented max / first-argmax
    over ``document_offsets``; the same numbers as the reference's per-pair
    loop, arranged so that large batches finish in seconds.
    """
    q_all = np.asarray(queries, dtype=np.float32)
    docs = np.ascontiguousarray(documents, dtype=np.float32)
    offs = np.asarray(document_offsets, dtype=np.int64)
    Nq, Lq, _ = q_all.shape
    Nb = offs.shape[0] - 1
    lens = np.diff(offs)
    starts = offs[:-1]
    T = docs.shape[0]
    local = (np.arange(T, dtype=np.int64) - np.repeat(starts, lens)).astype(np.int32)
    big = np.int32(np.iinfo(np.int32).max)
    scores = np.empty((Nq, Nb), dtype=np.float32)
    argmax = np.zeros((Nq, Nb, Lq), dtype=np.int32)
    gaps = np.full((Nq, Nb, Lq), np.inf, dtype=np.float32) if want_gap else None
    for qi in range(Nq):
        sim = _sim(q_all[qi], docs)                          # [Lq, T]
        clean = np.where(np.isnan(sim), _NEG_INF, sim)
        segmax = np.maximum.reduceat(clean, starts, axis=1)  # [Lq, Nb]
        hit = clean == np.repeat(segmax, lens, axis=1)
        pos = np.where(hit, local[None, :], big)
        first = np.minimum.reduceat(pos, starts, axis=1)     # [Lq, Nb]
        first = np.where(segmax == _NEG_INF, 0, first).astype(np.int32)
        with np.errstate(invalid="ignore", over="ignore"):
            scores[qi] = np.sum(segmax, axis=0, dtype=np.float32)
        argmax[qi] = first.T
        if want_gap:
            masked = clean.copy()
            cols = (starts[None, :] + first).astype(np.int64)  # [Lq, Nb]
            np.put_along_axis(masked, cols, _NEG_INF, axis=1)
            second = np.maximum.reduceat(masked, starts, axis=1)
            with np.errstate(invalid="ignore"):
                gap = segmax - second
            gap = np.where(np.isnan(gap), 0.0, gap)
            gap = np.where(lens[None, :] < 2, np.inf, gap)
            gaps[qi] = gap.T.astype(np.float32)
    if want_gap:
        return scores, argmax, gaps
    return scores, argmax


def contrastive_backward(dscore, queries, documents, document_offsets, argmax):
    """reference.py:284-323."""
    q = np.asarray(queries, dtype=np.float32)
    d = np.asarray(documents, dtype=np.float32)
    g = np.asarray(dscore, dtype=np.float32)
    offs = np.asarray(document_offsets, dtype=np.int64)
    Nq, Lq, dim = q.shape
    Nb = offs.shape[0] - 1
    lens = np.diff(offs)
    dq = np.zeros(q.shape, dtype=np.float64)
    dd = np.zeros(d.shape, dtype=np.float64)
    a_all = np.asarray(argmax, dtype=np.int64)
    with np.errstate(invalid="ignore", over="ignore"):
        for qi in range(Nq):
            a = a_all[qi]                                   # [Nb, Lq]
            ok = (a >= 0) & (a < lens[:, None])
            rows = offs[:-1, None] + np.where(ok, a, 0)     # [Nb, Lq] global rows
            w = np.where(ok, g[qi][:, None], np.float32(0)).astype(np.float32)
            # dq[qi, i] += sum_d g[qi,d] * D[row(d,i)]
            picked = np.where(ok[:, :, None], d[rows], np.float32(0))
            dq[qi] += np.einsum("dl,dlk->lk", w.astype(np.float64),
                                picked.astype(np.float64))
            contrib = (w[:, :, None] * q[qi][None, :, :]).reshape(Nb * Lq, dim)
            flat_rows = rows.reshape(-1)
            keep = ok.reshape(-1)
            np.add.at(dd, flat_rows[keep], contrib[keep])
    return dq.astype(np.float32), dd.astype(np.float32)


def argmax_mismatch_allowed(got, want, gaps, tol):
    """True where the kernel's argmax equals the oracle's or where the oracle's
    top-2 similarities are closer than ``tol`` (1e-6 fp32, 1e-3 half)."""
    got = np.asarray(got)
    want = np.asarray(want)
    return (got == want) | (np.asarray(gaps) < tol)


# ---------------------------------------------------------------------------
# Either side of the operators: packing and ranking, as the reference's callers
# write them.
# ---------------------------------------------------------------------------

def pack_padded(padded, lengths):
    """``padded [N, L_max, ...]`` + prefix ``lengths [N]`` -> ``(packed [T, ...],
    offsets [N+1] int32)``: the slices ``padded[n, :lengths[n]]`` back to back
    (README.md:185-192 of the reference; the mask gather of
    torch-ext/maxsim/__init__.py:594-606 gives the same rows in the same order)."""
    padded = np.asarray(padded)
    lengths = np.asarray(lengths).astype(np.int64)
    offsets = np.zeros(lengths.shape[0] + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    parts = [padded[n, :lengths[n]] for n in range(lengths.shape[0])]
    packed = np.concatenate(parts, axis=0) if parts else padded.reshape((0,) + padded.shape[2:])
    return packed, offsets.astype(np.int32)


def unpack_packed(packed, offsets, L_max):
    """The reverse copy: ``out[n, j] = packed[offsets[n] + j]`` for ``j`` inside
    segment ``n`` (truncated at ``L_max``), zero elsewhere."""
    packed = np.asarray(packed)
    offsets = np.asarray(offsets).astype(np.int64)
    n_seg = offsets.shape[0] - 1
    out = np.zeros((n_seg, L_max) + packed.shape[1:], dtype=packed.dtype)
    for n in range(n_seg):
        ln = min(int(offsets[n + 1] - offsets[n]), L_max)
        out[n, :ln] = packed[offsets[n]:offsets[n] + ln]
    return out


def rank_rows(scores, k):
    """``scores [B, C]`` -> ``(values [B, k], indices [B, k] int64)``: each row in
    descending order (README.md:270-274 of the reference ranks candidates with
    ``argsort(descending=True)``), equal scores by ascending index, NaN first."""
    scores = np.asarray(scores, dtype=np.float32)
    B, C = scores.shape
    idx = np.empty((B, k), dtype=np.int64)
    for b in range(B):
        row = scores[b]
        order = sorted(range(C), key=lambda j: (0 if np.isnan(row[j]) else 1,
                                                -float(row[j]) if not np.isnan(row[j]) else 0.0, j))
        idx[b] = order[:k]
    vals = np.take_along_axis(scores, idx, axis=1) if k else np.empty((B, 0), np.float32)
    return vals, idx
