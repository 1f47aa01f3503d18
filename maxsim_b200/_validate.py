"""Input validation for the public scoring functions.

The checks, their order, the exception types and the message fragments follow
the reference's Python layer (``torch-ext/maxsim/__init__.py:63-223`` for the
padded and packed layouts, ``:812-877`` for the contrastive layout), because
its test-suite pins them (``tests/test_invalid_inputs.py``,
``tests/test_ragged.py:64-106``).  The mechanics differ: instead of copying
whole offset / id tensors to the host and looping over them in Python, each
layout is reduced on its own device to a handful of integers (first offset,
last offset, smallest and largest segment, smallest and largest id) that come
back in a single transfer.  Only when one of them is out of bounds is the
tensor inspected element by element to name the offending index.
"""

from __future__ import annotations

import weakref
from typing import Dict, Optional, Tuple

import torch

FLOAT_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
INDEX_DTYPES = (torch.int32, torch.int64)


def require_float(name: str, t: torch.Tensor) -> None:
    if t.dtype not in FLOAT_DTYPES:
        raise TypeError(f"{name} must be float32, float16, or bfloat16; got {t.dtype}")


def require_index(name: str, t: torch.Tensor) -> None:
    if t.dtype not in INDEX_DTYPES:
        raise TypeError(f"{name} must be int32 or int64; got {t.dtype}")


def require_same_device(tensors: Dict[str, torch.Tensor]) -> None:
    it = iter(tensors.items())
    first_name, first = next(it)
    for name, t in it:
        if t.device != first.device:
            raise RuntimeError(
                "all tensors must be on the same device; "
                f"{first_name} is on {first.device} but {name} is on {t.device}"
            )


def _host_ints(*scalars: torch.Tensor) -> list:
    """Bring a few 0-d integer tensors to the host in one transfer."""
    return torch.stack([s.to(torch.int64) for s in scalars]).tolist()


# ---------------------------------------------------------------------------
# Index-tensor statistics: one small device kernel per tensor, one transfer per
# call, and nothing at all for a tensor object that was already inspected and
# has not been written since (same Python object, same version counter).
# ---------------------------------------------------------------------------

_STATS_CACHE: Dict[int, tuple] = {}
_STATS_CACHE_LIMIT = 64


def _cache_get(t: torch.Tensor) -> Optional[tuple]:
    ent = _STATS_CACHE.get(id(t))
    if ent is not None and ent[0]() is t and ent[1] == t._version:
        return ent[2]
    return None


def _cache_put(t: torch.Tensor, stats: tuple) -> None:
    if len(_STATS_CACHE) >= _STATS_CACHE_LIMIT:
        _STATS_CACHE.clear()
    try:
        _STATS_CACHE[id(t)] = (weakref.ref(t), t._version, stats)
    except TypeError:
        pass


def _torch_stats(t: torch.Tensor, as_offsets: bool) -> tuple:
    flat = t.detach().reshape(-1).to(torch.int64)
    if as_offsets:
        seg = flat[1:] - flat[:-1]
        return tuple(_host_ints(flat[0], flat[-1], seg.min(), seg.max()))
    if flat.numel() == 0:
        return (0, 0)
    return tuple(_host_ints(flat.min(), flat.max()))


def index_stats(offsets=(), ids=()):
    """Statistics of CSR offset tensors -> ``(first, last, min_seg, max_seg)``
    and of id / length tensors -> ``(min, max)``, in argument order.  Offsets
    tensors need at least two elements; empty id tensors give ``(0, 0)``."""
    results: Dict[int, tuple] = {}
    todo = []
    for t, is_off in [(t, True) for t in offsets] + [(t, False) for t in ids]:
        hit = _cache_get(t)
        if hit is not None and len(hit) == (4 if is_off else 2):
            results[id(t)] = hit
        else:
            todo.append((t, is_off))
    cuda = [x for x in todo if x[0].device.type == "cuda" and x[0].numel() > 0]
    if cuda:
        from . import _ops
        rows = _ops.layout_stats([(t, None) if is_off else (None, t) for t, is_off in cuda])
        for (t, is_off), row in zip(cuda, rows):
            results[id(t)] = tuple(row[0:4]) if is_off else tuple(row[4:6])
    for t, is_off in todo:
        if id(t) not in results:
            results[id(t)] = _torch_stats(t, is_off)
    for t, _ in todo:
        _cache_put(t, results[id(t)])
    return [results[id(t)] for t in offsets], [results[id(t)] for t in ids]


# ---------------------------------------------------------------------------
# Padded layout
# ---------------------------------------------------------------------------

def _length_bounds(stats: tuple, numel: int, limit: int, name: str) -> None:
    if numel == 0:
        return
    lo, hi = stats
    if lo <= 0:
        raise ValueError(f"{name} must contain values > 0")
    if hi > limit:
        raise ValueError(f"{name} values must be <= padded length {limit}")


def check_padded(queries, documents, query_lengths, doc_lengths) -> Tuple[int, int, int, int, int]:
    """Returns ``(B, C, Lq_max, Ld_max, D)``; torch-ext/maxsim/__init__.py:101-152."""
    if queries.dim() != 3:
        raise ValueError(f"queries must be 3-D [B, Lq, D]; got shape {tuple(queries.shape)}")
    if documents.dim() != 4:
        raise ValueError(f"documents must be 4-D [B, C, Ld, D]; got shape {tuple(documents.shape)}")
    B, Lq_max, D = queries.shape
    Bd, C, Ld_max, Dd = documents.shape
    if B != Bd:
        raise ValueError(f"batch dim mismatch: queries B={B} but documents B={Bd}")
    if D != Dd:
        raise ValueError(f"embedding dim mismatch: queries D={D} but documents D={Dd}")
    if tuple(query_lengths.shape) != (B,):
        raise ValueError(f"query_lengths must have shape [B={B}]; got {tuple(query_lengths.shape)}")
    if tuple(doc_lengths.shape) != (B, C):
        raise ValueError(f"doc_lengths must have shape [B={B}, C={C}]; got {tuple(doc_lengths.shape)}")
    if queries.dtype != documents.dtype:
        raise TypeError(
            f"queries and documents must have the same dtype; got {queries.dtype} vs {documents.dtype}"
        )
    require_float("queries", queries)
    require_float("documents", documents)
    require_index("query_lengths", query_lengths)
    require_index("doc_lengths", doc_lengths)
    require_same_device(dict(queries=queries, documents=documents,
                             query_lengths=query_lengths, doc_lengths=doc_lengths))
    _, (qs, ds) = index_stats(ids=(query_lengths, doc_lengths))
    _length_bounds(qs, query_lengths.numel(), Lq_max, "query_lengths")
    _length_bounds(ds, doc_lengths.numel(), Ld_max, "doc_lengths")
    return B, C, Lq_max, Ld_max, D


# ---------------------------------------------------------------------------
# Packed layout
# ---------------------------------------------------------------------------

def check_packed_types(queries, query_offsets, documents, document_offsets,
                       pair_query_ids, pair_document_ids, *, verbose_shapes: bool) -> None:
    """Rank / dim / dtype / device checks (torch-ext/maxsim/__init__.py:256-293
    for the score-only entry, :325-363 for the argmax and train entries)."""
    if queries.dim() != 2:
        what = "2-D [total_q_tokens, dim]" if verbose_shapes else "2-D"
        raise ValueError(f"queries must be {what}; got shape {tuple(queries.shape)}")
    if documents.dim() != 2:
        what = "2-D [total_d_tokens, dim]" if verbose_shapes else "2-D"
        raise ValueError(f"documents must be {what}; got shape {tuple(documents.shape)}")
    if queries.shape[1] != documents.shape[1]:
        if verbose_shapes:
            raise ValueError("queries.dim and documents.dim must match; got "
                             f"{queries.shape[1]} vs {documents.shape[1]}")
        raise ValueError(f"queries.D ({queries.shape[1]}) must match documents.D "
                         f"({documents.shape[1]}); embedding dim differs")
    if queries.dtype != documents.dtype:
        if verbose_shapes:
            raise TypeError("queries and documents must have the same dtype; got "
                            f"{queries.dtype} vs {documents.dtype}")
        raise TypeError(f"queries and documents must share dtype; got {queries.dtype} "
                        f"vs {documents.dtype}")
    require_float("queries", queries)
    require_float("documents", documents)
    require_index("query_offsets", query_offsets)
    require_index("document_offsets", document_offsets)
    require_index("pair_query_ids", pair_query_ids)
    require_index("pair_document_ids", pair_document_ids)
    require_same_device(dict(queries=queries, query_offsets=query_offsets,
                             documents=documents, document_offsets=document_offsets,
                             pair_query_ids=pair_query_ids,
                             pair_document_ids=pair_document_ids))
    if pair_query_ids.shape != pair_document_ids.shape:
        raise ValueError("pair_query_ids and pair_document_ids must have the same shape; "
                         f"got {tuple(pair_query_ids.shape)} vs {tuple(pair_document_ids.shape)}")
    if pair_query_ids.dim() != 1:
        raise ValueError(f"pair_query_ids must be 1-D; got shape {tuple(pair_query_ids.shape)}")


def _first_index(mask: torch.Tensor) -> int:
    return int(torch.nonzero(mask.reshape(-1))[0].item())


def check_packed_layout(queries, query_offsets, documents, document_offsets,
                        pair_query_ids, pair_document_ids) -> int:
    """Offsets start at 0, end at the token count and have no empty segment;
    ids lie in range.  Returns the longest query segment.  Raises RuntimeError
    with the reference's wording (torch-ext/maxsim/__init__.py:170-223)."""
    for name, off in (("query_offsets", query_offsets), ("document_offsets", document_offsets)):
        if off.numel() < 2:
            raise RuntimeError(f"{name} must have length >= 2")
    (qo, do), (qi, di) = index_stats(offsets=(query_offsets, document_offsets),
                                     ids=(pair_query_ids, pair_document_ids))
    q0, qN, qmin, qmax = qo
    d0, dN, dmin, _dmax = do
    qid_lo, qid_hi = qi
    did_lo, did_hi = di

    def offsets_ok(name, off, first, last, smallest, total):
        if first != 0:
            raise RuntimeError(f"{name}[0] must equal 0, got {first}")
        if last != total:
            raise RuntimeError(f"{name}[-1] ({last}) must equal total token count ({total})")
        if smallest <= 0:
            o = off.detach().reshape(-1).to(torch.int64)
            i = _first_index((o[1:] - o[:-1]) <= 0)
            raise RuntimeError(f"empty segment in {name} at index {i}")

    offsets_ok("query_offsets", query_offsets, q0, qN, qmin, queries.shape[0])
    offsets_ok("document_offsets", document_offsets, d0, dN, dmin, documents.shape[0])

    def ids_ok(name, ids, lo, hi, upper):
        if ids.numel() and (lo < 0 or hi >= upper):
            flat = ids.detach().reshape(-1).to(torch.int64)
            i = _first_index((flat < 0) | (flat >= upper))
            raise RuntimeError(f"{name}[{i}] = {int(flat[i].item())} out of range [0, {upper})")

    ids_ok("pair_query_ids", pair_query_ids, qid_lo, qid_hi, query_offsets.numel() - 1)
    ids_ok("pair_document_ids", pair_document_ids, did_lo, did_hi, document_offsets.numel() - 1)
    return int(qmax)


def resolve_max_q_len(requested, actual: int) -> int:
    """torch-ext/maxsim/__init__.py:303-313."""
    if requested is None:
        return actual
    if requested <= 0:
        raise ValueError(f"max_q_len must be > 0; got {requested}")
    if requested < actual:
        raise ValueError(f"max_q_len ({requested}) must be >= actual max query "
                         f"segment length ({actual})")
    return int(requested)


# ---------------------------------------------------------------------------
# Contrastive layout
# ---------------------------------------------------------------------------

def check_contrastive(queries, documents, document_offsets) -> None:
    """torch-ext/maxsim/__init__.py:812-877 (ValueError for offset faults)."""
    require_float("queries", queries)
    require_float("documents", documents)
    require_index("document_offsets", document_offsets)
    if queries.dtype != documents.dtype:
        raise TypeError(f"queries and documents must share dtype; got {queries.dtype} "
                        f"and {documents.dtype}")
    if queries.dim() != 3:
        raise ValueError(f"queries must be [Nq, Lq, D]; got shape {tuple(queries.shape)}")
    if documents.dim() != 2:
        raise ValueError("documents must be [total_d_tokens, D] (packed); got shape "
                         f"{tuple(documents.shape)}")
    if document_offsets.dim() != 1:
        raise ValueError("document_offsets must be 1-D [Nb+1]; got shape "
                         f"{tuple(document_offsets.shape)}")
    if queries.shape[2] != documents.shape[1]:
        raise ValueError(f"queries.D ({queries.shape[2]}) must match documents.D "
                         f"({documents.shape[1]})")
    if queries.shape[1] <= 0:
        raise ValueError(f"Lq must be > 0; got {queries.shape[1]}")
    if queries.shape[2] <= 0:
        raise ValueError(f"dim must be > 0; got {queries.shape[2]}")
    if document_offsets.numel() < 2:
        raise ValueError("document_offsets must have length >= 2 (at least one doc); "
                         f"got {document_offsets.numel()}")
    require_same_device(dict(queries=queries, documents=documents,
                             document_offsets=document_offsets))
    ((first, last, smallest, _),), _ = index_stats(offsets=(document_offsets,))
    total = documents.shape[0]
    if first != 0:
        raise ValueError("document_offsets[0] must equal 0 (CSR offset convention); "
                         f"got {first}")
    if last != total:
        raise ValueError(f"document_offsets[-1] ({last}) must equal total doc tokens "
                         f"({total}). The packed documents tensor and the offsets must "
                         "agree on the total length.")
    if smallest <= 0:
        o = document_offsets.detach().to(torch.int64)
        i = _first_index((o[1:] - o[:-1]) <= 0)
        raise ValueError("document_offsets must be strictly increasing; got "
                         f"document_offsets[{i + 1}] ({int(o[i + 1])}) <= "
                         f"document_offsets[{i}] ({int(o[i])})")
