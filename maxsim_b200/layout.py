"""The steps either side of the operators: packing encoder outputs, unpacking
packed rows, ranking rerank scores.

The reference has no kernels for these.  Its callers pack with a Python loop of
slices and ``torch.cat`` (``README.md:185-192``) or a boolean-mask gather
(``torch-ext/maxsim/__init__.py:516-620``), both of which synchronise with the
host, and rank with ``scores.argsort(dim=1, descending=True)``
(``README.md:270-274``).  Here each is one kernel behind the C ABI:

* :func:`pack_padded` -- ``[N, L_max, D]`` + lengths -> packed ``[T, D]`` +
  int32 offsets; differentiable (the gradient is the reverse copy);
* :func:`unpack_packed` -- packed rows back to ``[N, L_max, D]`` with zero
  padding; differentiable;
* :func:`rerank_topk` -- the ``k`` best candidates of every row of a score
  matrix, best first, equal scores by ascending candidate index;
* :func:`score_candidates_padded_from_host` -- rerank a padded batch that
  lives in pinned host memory: a kernel reads only the valid token rows over
  PCIe (a padded batch is about one third padding), the scores go back to the
  host.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _ops
from . import _validate as _v

__all__ = ["pack_padded", "unpack_packed", "rerank_topk", "rerank_order",
           "score_candidates_padded_from_host"]

_eager = torch.compiler.disable


class _PackFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, padded, offsets, total):
        ctx.save_for_backward(offsets)
        ctx.L_max = padded.shape[1]
        return _ops.pack_rows(padded, offsets, total)

    @staticmethod
    def backward(ctx, grad_packed):
        (offsets,) = ctx.saved_tensors
        return _ops.unpack_rows(grad_packed, offsets, ctx.L_max), None, None


class _UnpackFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, offsets, L_max):
        ctx.save_for_backward(offsets)
        ctx.rows = packed.shape[0]
        return _ops.unpack_rows(packed, offsets, L_max)

    @staticmethod
    def backward(ctx, grad_padded):
        (offsets,) = ctx.saved_tensors
        return _ops.pack_rows(grad_padded, offsets, ctx.rows), None, None


@_eager
def pack_padded(padded: torch.Tensor, lengths: torch.Tensor, *,
                total_tokens: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Pack ``padded [N, L_max, D]`` (CUDA, any dtype) by prefix ``lengths [N]``.

    Returns ``(packed [T, D], offsets [N+1] int32)`` ready for
    ``score_contrastive*`` (documents) or ``score_pairs_packed*``.

    ``lengths`` may live on the host or on the device.  On the host the offsets
    are built there and nothing synchronises.  On the device a scan kernel
    builds them; ``T`` is then read back (one synchronisation) unless the
    caller passes ``total_tokens``, in which case nothing synchronises and the
    value is trusted to equal ``lengths.sum()`` (rows beyond it are dropped,
    never written out of bounds).

    Raises ``ValueError`` for a shape mismatch or, when the lengths are visible
    to the host, a length outside ``(0, L_max]``.
    """
    if padded.dim() < 2:
        raise ValueError(f"padded must be at least 2-D [N, L_max, ...]; got shape {tuple(padded.shape)}")
    if padded.device.type != "cuda":
        raise RuntimeError(f"padded must be a CUDA tensor (maxsim_b200 has no CPU path); got device {padded.device}")
    N, L_max = padded.shape[0], padded.shape[1]
    if tuple(lengths.shape) != (N,):
        raise ValueError(f"lengths must have shape [N={N}]; got {tuple(lengths.shape)}")
    if lengths.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"lengths must be int32 or int64; got {lengths.dtype}")
    if lengths.device.type == "cpu":
        if N and (int(lengths.min()) <= 0 or int(lengths.max()) > L_max):
            raise ValueError(f"lengths must be in (0, L_max={L_max}]")
        host = torch.zeros(N + 1, dtype=torch.int64)
        torch.cumsum(lengths, 0, out=host[1:])
        total = int(host[-1])
        if total >= 2 ** 31:
            raise ValueError("packed token count must fit int32 offsets")
        offsets = host.to(torch.int32).to(padded.device, non_blocking=True)
    else:
        offsets, total_dev = _ops.offsets_from_lengths(lengths, L_max)
        if total_tokens is None:
            total = int(total_dev.item())
            if total >= 2 ** 31:
                raise ValueError("packed token count must fit int32 offsets")
        else:
            total = int(total_tokens)
    if total_tokens is not None and int(total_tokens) != total:
        raise ValueError(f"total_tokens={int(total_tokens)} does not match lengths.sum()={total}")
    return _PackFn.apply(padded, offsets, total), offsets


@_eager
def unpack_packed(packed: torch.Tensor, offsets: torch.Tensor, L_max: int) -> torch.Tensor:
    """``packed [T, D]`` + ``offsets [N+1]`` -> ``[N, L_max, D]``, zero beyond
    each segment (segments longer than ``L_max`` are truncated)."""
    if packed.dim() < 1 or offsets.dim() != 1 or offsets.numel() < 1:
        raise ValueError("packed must be [T, ...] and offsets [N+1]")
    if int(L_max) < 0:
        raise ValueError("L_max must be >= 0")
    return _UnpackFn.apply(packed, offsets, int(L_max))


@_eager
def rerank_topk(scores: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The ``k`` best candidates per row of ``scores [B, C]``: returns
    ``(values [B, k] fp32, indices [B, k] int64)``, best first; equal scores
    are ordered by ascending candidate index; NaN ranks above ``+inf`` (the
    convention of ``torch.sort``).  ``C`` may be at most 16384."""
    if scores.dim() != 2:
        raise ValueError(f"scores must be 2-D [B, C]; got shape {tuple(scores.shape)}")
    if not 0 <= int(k) <= scores.shape[1]:
        raise ValueError(f"k must be in [0, C={scores.shape[1]}]; got {k}")
    return _ops.topk_rows(scores.detach(), int(k))


@_eager
def rerank_order(scores: torch.Tensor) -> torch.Tensor:
    """Full ranking: what ``scores.argsort(dim=1, descending=True)`` gives,
    with ties by ascending index."""
    return rerank_topk(scores, scores.shape[1])[1]


_STAGING = {}


def _staging_for(documents: torch.Tensor, device: torch.device) -> torch.Tensor:
    key = (tuple(documents.shape), documents.dtype, str(device))
    buf = _STAGING.get(key)
    if buf is None:
        _STAGING.clear()  # one batch shape at a time: these buffers are large
        buf = torch.empty(documents.shape, dtype=documents.dtype, device=device)
        _STAGING[key] = buf
    return buf


@_eager
def score_candidates_padded_from_host(queries: torch.Tensor, documents: torch.Tensor,
                                      query_lengths: torch.Tensor, doc_lengths: torch.Tensor, *,
                                      device, staging: Optional[torch.Tensor] = None,
                                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`maxsim_b200.score_candidates_padded` for a batch in host memory.

    ``queries [B, Lq, D]``, ``documents [B, C, Ld, D]`` and the two length
    tensors are CPU tensors.  When ``documents`` is pinned, a kernel on
    ``device`` reads each candidate's first ``doc_lengths[b, c]`` rows straight
    from it, so padding rows never cross PCIe; a pageable ``documents`` is
    copied whole.  ``staging`` is the device-side ``[B, C, Ld, D]`` landing
    buffer (one is kept per batch shape when not given; its padding rows hold
    whatever they held before, and no kernel reads them).  The kept buffer is
    shared by every call of that shape and is ordered only by the stream the
    calls run on: callers that use several streams pass their own ``staging``.

    Returns the ``[B, C]`` fp32 scores on the host.  With a pinned ``out`` the
    copy back is asynchronous on the current stream of ``device`` and ``out``
    is returned: synchronise that stream (or the device) before reading it.
    """
    for name, t in (("queries", queries), ("documents", documents),
                    ("query_lengths", query_lengths), ("doc_lengths", doc_lengths)):
        if t.device.type != "cpu":
            raise RuntimeError(f"{name} must be a CPU tensor; got device {t.device}")
    B, C, Lq, Ld, D = _v.check_padded(queries, documents, query_lengths, doc_lengths)
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"device must be a CUDA device (maxsim_b200 has no CPU path); got {device}")
    if device.index is None:  # "cuda" means the current device; tensors report an index
        device = torch.device("cuda", torch.cuda.current_device())
    documents = documents.contiguous()
    with torch.cuda.device(device):
        q = queries.contiguous().to(device, non_blocking=True)
        qlen = query_lengths.contiguous().to(device, non_blocking=True).to(torch.int32)
        dlen = doc_lengths.contiguous().to(device, non_blocking=True).to(torch.int32)
        if staging is None:
            staging = _staging_for(documents, device)
        elif (staging.shape != documents.shape or staging.dtype != documents.dtype
              or staging.device != device or not staging.is_contiguous()):
            raise ValueError("staging must be a contiguous tensor on `device` shaped and typed like documents")
        if documents.is_pinned():
            _ops.copy_valid_rows(documents.view(B * C, Ld, D), dlen.view(-1), staging.view(B * C, Ld, D))
        else:
            staging.copy_(documents)
        scores = _ops.ops.maxsim_padded_forward(q.view(B * Lq, D), qlen, staging.view(B * C * Ld, D),
                                                dlen.view(-1), int(Lq), int(Ld), int(C)).view(B, C)
        if out is not None:
            if tuple(out.shape) != (B, C) or out.dtype != torch.float32 or out.device.type != "cpu":
                raise ValueError(f"out must be a CPU float32 tensor of shape [B={B}, C={C}]")
            out.copy_(scores, non_blocking=True)
            return out
        return scores.cpu()
