"""The nine operators, as Python callables over the C ABI.

``ops`` exposes exactly the callables the reference's Python layer looks up on
``maxsim._ops.ops`` (``torch-ext/torch_binding.cpp:7-90``; the development
binding ``maxsim_cuda/dev_binding.cpp:82-104`` and ``tests/conftest.py:133-145``
build the same namespace): same names, positional arguments, return shapes and
dtypes.  Each callable allocates its outputs with torch, hands raw device
pointers and the current CUDA stream to ``libmaxsim_b200.so`` through ctypes
and raises ``RuntimeError`` on a non-zero status, the way ``TORCH_CHECK`` does
in the reference.

There is no CPU path: a tensor that is not on a CUDA device, or a missing
library, is an error.
"""

from __future__ import annotations

import ctypes
import os
import types
import weakref
from pathlib import Path
from ctypes import c_char_p, c_int, c_int64, c_void_p
from typing import Tuple

import torch

from . import _build

_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

_lib = None

_I64 = c_int64
_P = c_void_p

_SIGNATURES = {
    "maxsim_b200_version": (c_char_p, []),
    "maxsim_b200_last_error": (c_char_p, []),
    "maxsim_b200_device_status": (c_int, [_P]),
    "maxsim_b200_launch_count": (c_int64, []),
    "maxsim_b200_wait_probe": (c_int, [_I64, _P, _P]),
    "maxsim_b200_set_forward_path": (None, [c_int]),
    "maxsim_b200_layout_stats": (c_int, [_P, _I64, _P, _I64, c_int, _P, _P]),
    "maxsim_b200_contrastive_ce": (c_int, [_P] * 4 + [_I64] * 2 + [ctypes.c_float] * 2 + [_P]),
    "maxsim_b200_offsets_from_lengths": (c_int, [_P, _I64, _I64, _P, _P, _P]),
    "maxsim_b200_pack_rows": (c_int, [_P] * 3 + [_I64] * 4 + [_P]),
    "maxsim_b200_unpack_rows": (c_int, [_P] * 3 + [_I64] * 4 + [_P]),
    "maxsim_b200_topk_rows": (c_int, [_P] + [_I64] * 3 + [_P] * 3),
    "maxsim_b200_copy_valid_rows": (c_int, [_P, c_int, _P, _P] + [_I64] * 3 + [_P]),
    "maxsim_b200_group_pairs": (c_int, [_P, _I64, _I64, _P, _P, _P]),
    "maxsim_b200_group_pairs_static": (c_int, [_P, _I64, _I64, _P, _P]),
    "maxsim_forward_ordered": (c_int, [_P] * 8 + [_I64] * 7 + [c_int, _P]),
    "maxsim_packed_forward_with_argmax_ordered": (c_int, [_P] * 9 + [_I64] * 7 + [c_int, _P]),
    "maxsim_packed_backward_grouped": (c_int, [_P] * 14 + [_I64] * 7 + [c_int, _P]),
    "maxsim_packed_backward_grouped_native": (c_int, [_P] * 14 + [_I64] * 7 + [c_int, _P]),
    "maxsim_forward": (c_int, [_P] * 7 + [_I64] * 7 + [c_int, _P]),
    "maxsim_packed_forward_with_argmax": (c_int, [_P] * 8 + [_I64] * 7 + [c_int, _P]),
    "maxsim_packed_backward": (c_int, [_P] * 10 + [_I64] * 7 + [c_int, _P]),
    "maxsim_padded_forward": (c_int, [_P] * 5 + [_I64] * 5 + [c_int, _P]),
    "maxsim_padded_forward_with_argmax": (c_int, [_P] * 6 + [_I64] * 5 + [c_int, _P]),
    "maxsim_padded_backward": (c_int, [_P] * 8 + [_I64] * 5 + [c_int, _P]),
    "maxsim_contrastive_forward": (c_int, [_P] * 4 + [_I64] * 5 + [c_int, _P]),
    "maxsim_contrastive_forward_with_argmax": (c_int, [_P] * 5 + [_I64] * 5 + [c_int, _P]),
    "maxsim_contrastive_backward": (c_int, [_P] * 7 + [_I64] * 5 + [c_int, _P]),
    "maxsim_contrastive_forward_with_argmax_block": (c_int, [_P] * 5 + [_I64] * 9 + [c_int, _P]),
    "maxsim_b200_pack_owner_records": (c_int, [_P] * 3 + [_I64] * 4 + [_P, _P]),
    "maxsim_contrastive_backward_documents_from_records": (c_int, [_P] * 5 + [_I64] * 5 + [c_int, c_int, _P]),
    "maxsim_b200_pack_owner_records_to": (c_int, [_P] * 4 + [_I64] * 4 + [_P]),
    "maxsim_b200_peer_barrier": (c_int, [_P, _I64, _I64, _P, ctypes.c_uint32, _P]),
    "maxsim_b200_peer_gather": (c_int, [_P, _I64, _I64, _P, _P, _P]),
    "maxsim_b200_copy_many": (c_int, [_P, _P, _P, _I64, _P]),
    "maxsim_padded_backward_native": (c_int, [_P] * 8 + [_I64] * 5 + [c_int, _P]),
    "maxsim_contrastive_backward_native": (c_int, [_P] * 7 + [_I64] * 5 + [c_int, _P]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def load_library() -> ctypes.CDLL:
    """Load (building first if the sources changed and nvcc is present)."""
    global _lib
    if _lib is not None:
        return _lib
    override = os.environ.get("MAXSIM_B200_LIBRARY")  # an alternative build, for A/B comparisons
    path = _build.LIB_PATH if not override else Path(override)
    if not override and not _build.is_current():
        try:
            _build.build()
        except RuntimeError as exc:
            if not path.exists():
                raise RuntimeError(
                    f"libmaxsim_b200.so is not built and could not be built here: {exc}. "
                    "Run `python -m maxsim_b200._build` on a machine with nvcc."
                ) from exc
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in _SIGNATURES.items():
        if override and not hasattr(lib, name):
            continue  # an older build, loaded for comparison, may lack newer entry points
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def library_path() -> str:
    return str(_build.LIB_PATH)


def launch_count() -> int:
    return int(load_library().maxsim_b200_launch_count())


def set_forward_path(path: int) -> None:
    load_library().maxsim_b200_set_forward_path(int(path))


def device_status(device=None) -> int:
    """Synchronise the current stream and return the kernels' status word."""
    with torch.cuda.device(device):
        return int(load_library().maxsim_b200_device_status(_stream_ptr()))


def wait_probe(polls: int = 64, device=None) -> bool:
    """Launch the kernel whose only wait cannot be satisfied (see the header):
    returns True if it gave up after ``polls`` polls.  ``device_status()``
    reports the time-out bit afterwards, and clears it."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    flag = torch.zeros((1,), dtype=torch.int32, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_b200_wait_probe(int(polls), flag.data_ptr(), _stream_ptr())
    _check(rc, "maxsim_b200_wait_probe")
    return bool(flag.item())


def layout_stats(items) -> list:
    """``items``: list of ``(offsets or None, ids or None)`` index tensors on
    one CUDA device (each pair shares a dtype, int32 or int64).  Returns one
    list of eight ints per item -- first offset, last offset, smallest and
    largest segment, smallest and largest id, counts -- using one small kernel
    per item and a single device-to-host transfer for all of them."""
    lib = load_library()
    dev = next(t for pair in items for t in pair if t is not None).device
    out = torch.empty((len(items), 8), dtype=torch.int64, device=dev)
    keep = []
    with _on_device(dev):
        for row, (offsets, ids) in enumerate(items):
            ref = offsets if offsets is not None else ids
            o = offsets.detach().reshape(-1).contiguous() if offsets is not None else None
            i = ids.detach().reshape(-1).contiguous() if ids is not None else None
            if i is not None and o is not None and i.dtype != o.dtype:
                i = i.to(o.dtype)
            keep.append((o, i))
            rc = lib.maxsim_b200_layout_stats(
                _ptr(o) if o is not None else 0, o.numel() if o is not None else 0,
                _ptr(i) if i is not None else 0, i.numel() if i is not None else 0,
                ref.element_size(), out[row].data_ptr(), _stream_ptr())
            _check(rc, "maxsim_b200_layout_stats")
    return out.tolist()


def contrastive_ce(scores: torch.Tensor, targets: torch.Tensor, temperature: float,
                   grad_scale: float, want_grad: bool):
    """Row-wise cross-entropy of ``scores [Nq, Nb]`` (fp32, CUDA) against
    ``targets [Nq]``; returns ``(loss_rows [Nq], dscore [Nq, Nb] or None)``."""
    dev = _require_cuda(scores, targets)
    s = scores.contiguous().to(torch.float32)
    t = targets.contiguous().to(torch.int64)
    if s.dim() != 2 or t.dim() != 1 or t.shape[0] != s.shape[0]:
        raise RuntimeError("scores must be [Nq, Nb] and targets [Nq]")
    loss_rows = torch.empty((s.shape[0],), dtype=torch.float32, device=dev)
    dscore = torch.empty_like(s) if want_grad else None
    with _on_device(dev):
        rc = load_library().maxsim_b200_contrastive_ce(
            _ptr(s), _ptr(t), _ptr(loss_rows), _ptr(dscore) if dscore is not None else 0,
            s.shape[0], s.shape[1], float(temperature), float(grad_scale), _stream_ptr())
    _check(rc, "maxsim_b200_contrastive_ce")
    return loss_rows, dscore


def offsets_from_lengths(lengths: torch.Tensor, L_max: int):
    """``lengths [N]`` (CUDA, integer) -> ``(offsets [N+1] int32, total [1] int64)``,
    both on the device; lengths are clamped to ``[0, L_max]``."""
    dev = _require_cuda(lengths)
    ln = _i32(lengths.reshape(-1))
    offsets = torch.empty((ln.shape[0] + 1,), dtype=torch.int32, device=dev)
    total = torch.empty((1,), dtype=torch.int64, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_b200_offsets_from_lengths(
            _ptr(ln), ln.shape[0], int(L_max), offsets.data_ptr(), total.data_ptr(), _stream_ptr())
    _check(rc, "maxsim_b200_offsets_from_lengths")
    return offsets, total


def pack_rows(padded: torch.Tensor, offsets: torch.Tensor, packed_rows: int) -> torch.Tensor:
    """``padded [N, L_max, ...]`` -> ``packed [packed_rows, ...]``: segment ``n`` contributes its
    first ``offsets[n+1] - offsets[n]`` rows."""
    dev = _require_cuda(padded, offsets)
    src = padded.contiguous()
    off = _i32(offsets)
    n, L = src.shape[0], src.shape[1]
    packed = torch.empty((int(packed_rows),) + tuple(src.shape[2:]), dtype=src.dtype, device=dev)
    row_bytes = (src[0, 0].numel() if n and L else 1) * src.element_size()
    with _on_device(dev):
        rc = load_library().maxsim_b200_pack_rows(
            _ptr(src), _ptr(off), _ptr(packed), n, L, row_bytes, int(packed_rows), _stream_ptr())
    _check(rc, "maxsim_b200_pack_rows")
    return packed


def unpack_rows(packed: torch.Tensor, offsets: torch.Tensor, L_max: int) -> torch.Tensor:
    """``packed [T, ...]`` -> ``padded [N, L_max, ...]`` with zeros beyond each segment."""
    dev = _require_cuda(packed, offsets)
    src = packed.contiguous()
    off = _i32(offsets)
    n = off.shape[0] - 1
    padded = torch.empty((n, int(L_max)) + tuple(src.shape[1:]), dtype=src.dtype, device=dev)
    row_bytes = 1
    for extent in src.shape[1:]:
        row_bytes *= extent
    row_bytes *= src.element_size()
    if row_bytes == 0:
        return padded
    with _on_device(dev):
        rc = load_library().maxsim_b200_unpack_rows(
            _ptr(src), _ptr(off), _ptr(padded), n, int(L_max), row_bytes, src.shape[0],
            _stream_ptr())
    _check(rc, "maxsim_b200_unpack_rows")
    return padded


def copy_valid_rows(src: torch.Tensor, lengths: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """Copy the first ``lengths[n]`` rows of every segment of padded ``src
    [N, L_max, ...]`` into ``dst`` (same shape and dtype, on a CUDA device);
    padding rows of ``dst`` keep their contents.  ``src`` may be on the same
    device or in pinned host memory, which the kernel then reads over PCIe."""
    dev = _require_cuda(dst, lengths)
    if src.shape != dst.shape or src.dtype != dst.dtype:
        raise RuntimeError("src and dst must have the same shape and dtype")
    if not src.is_contiguous() or not dst.is_contiguous():
        raise RuntimeError("src and dst must be contiguous")
    host = src.device.type == "cpu"
    if host and not src.is_pinned():
        raise RuntimeError("a host source must be in pinned (page-locked) memory")
    if not host and src.device != dev:
        raise RuntimeError(f"all inputs must share a device; got {dev} and {src.device}")
    ln = _i32(lengths.reshape(-1))
    n, L = src.shape[0], src.shape[1]
    if ln.shape[0] != n:
        raise RuntimeError("lengths must have one entry per segment")
    row_bytes = (src[0, 0].numel() if n and L else 1) * src.element_size()
    with _on_device(dev):
        rc = load_library().maxsim_b200_copy_valid_rows(
            src.data_ptr(), 1 if host else 0, _ptr(ln), dst.data_ptr(), n, L, row_bytes,
            _stream_ptr())
    _check(rc, "maxsim_b200_copy_valid_rows")
    return dst


def topk_rows(scores: torch.Tensor, k: int):
    """``scores [rows, cols]`` fp32 -> ``(values [rows, k] fp32, indices [rows, k] int64)``."""
    dev = _require_cuda(scores)
    s = scores.contiguous().to(torch.float32)
    values = torch.empty((s.shape[0], int(k)), dtype=torch.float32, device=dev)
    indices = torch.empty((s.shape[0], int(k)), dtype=torch.int64, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_b200_topk_rows(
            _ptr(s), s.shape[0], s.shape[1], int(k), _ptr(values), _ptr(indices), _stream_ptr())
    _check(rc, "maxsim_b200_topk_rows")
    return values, indices


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_exchange_device = getattr(torch.cuda, "_exchange_device", None)


def _stream_ptr() -> int:
    """Handle of the current stream of the current device.  The raw query is
    about ten times cheaper than building a ``torch.cuda.Stream`` object,
    which matters for the small launch-bound shapes."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class _on_device:
    """``with _on_device(dev):`` makes ``dev`` current for the library call,
    like ``torch.cuda.device`` but without its argument parsing."""

    __slots__ = ("idx", "prev")

    def __init__(self, dev: torch.device):
        self.idx = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        if _exchange_device is not None:
            self.prev = _exchange_device(self.idx)
        else:
            self.prev = torch.cuda.current_device()
            if self.prev != self.idx:
                torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev != self.idx and self.prev >= 0:
            if _exchange_device is not None:
                _exchange_device(self.prev)
            else:
                torch.cuda.set_device(self.prev)
        return False


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr() if t.numel() else 0


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    if dev.type != "cuda":
        raise RuntimeError(
            f"queries must be a CUDA tensor (maxsim_b200 has no CPU path); got device {dev}")
    for t in tensors[1:]:
        if t.device != dev:
            raise RuntimeError(f"all inputs must share a device; got {dev} and {t.device}")
    return dev


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise RuntimeError(
            f"queries/documents dtype must be float32, float16, or bfloat16; got {t.dtype}") from None


def _check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load_library().maxsim_b200_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (status {rc}): {msg}")


def _i32(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().to(torch.int32)


def _same_float(q: torch.Tensor, d: torch.Tensor) -> None:
    if q.dtype != d.dtype:
        raise RuntimeError("queries and documents must have the same dtype")


# ---------------------------------------------------------------------------
# packed
# ---------------------------------------------------------------------------

# Pair lists at least this long are grouped by document (forward with argmax,
# backward) and by query (backward).
GROUP_MIN_PAIRS = 2048
_group_enabled = True
_GROUP_CACHE = {}
_GROUP_CACHE_LIMIT = 32


def set_pair_grouping(enabled: bool) -> None:
    """Switch the grouping of packed pair lists on or off (for A/B timing)."""
    global _group_enabled
    _group_enabled = bool(enabled)


def group_pairs(ids: torch.Tensor, n_bins: int):
    """Counting sort of a pair list by ``ids`` (document or query ids in
    ``[0, n_bins)``): returns ``(order, ends)``, int32 on the device --
    ``order`` a permutation of ``range(n_pairs)`` with equal ids adjacent,
    ``ends[b]`` the end of id ``b``'s group in it."""
    dev = _require_cuda(ids)
    flat = _i32(ids.reshape(-1))
    order = torch.empty((flat.shape[0],), dtype=torch.int32, device=dev)
    ends = torch.empty((max(int(n_bins), 1),), dtype=torch.int32, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_b200_group_pairs(
            _ptr(flat), flat.shape[0], max(int(n_bins), 1), ends.data_ptr(), _ptr(order),
            _stream_ptr())
    _check(rc, "maxsim_b200_group_pairs")
    return order, ends


def _groups(key: torch.Tensor, ids32: torch.Tensor, n_bins: int, build: bool = True):
    """``(order, ends)`` of a pair-id tensor, or None.  ``key`` is the tensor
    object the caller passed: its grouping is remembered until the tensor is
    written to or dies.  With ``build=False`` only a remembered grouping is
    returned.

    The memory trusts torch's version counter: a write that does not bump it
    (``tensor.data``, a DLPack / external-library view of the same storage)
    leaves a stale grouping behind; call :func:`forget_pair_groups` after such
    a write.  While a CUDA graph is being captured nothing is remembered or
    looked up: the grouping kernels are launched into the capture, so that a
    replay groups the pair ids that are in the tensors at replay time."""
    if not _group_enabled or ids32.shape[0] < GROUP_MIN_PAIRS or n_bins <= 0:
        return None
    if torch.cuda.is_current_stream_capturing():
        return group_pairs(ids32, n_bins) if build else None
    ent = _GROUP_CACHE.get(id(key))
    if ent is not None and ent[0]() is key and ent[1] == key._version and ent[2] == n_bins:
        return ent[3]
    if not build:
        return None
    groups = group_pairs(ids32, n_bins)
    if len(_GROUP_CACHE) >= _GROUP_CACHE_LIMIT:
        _GROUP_CACHE.clear()
    try:
        _GROUP_CACHE[id(key)] = (weakref.ref(key), key._version, n_bins, groups)
    except TypeError:
        pass
    return groups


def forget_pair_groups() -> None:
    """Drop every remembered grouping of a pair-id tensor."""
    _GROUP_CACHE.clear()


def _packed_args(queries, query_offsets, documents, document_offsets,
                 pair_query_ids, pair_document_ids):
    if queries.dim() != 2 or documents.dim() != 2:
        raise RuntimeError("queries/documents must be 2-D [tokens, dim]")
    if queries.shape[1] != documents.shape[1]:
        raise RuntimeError("queries.dim must match documents.dim")
    _same_float(queries, documents)
    q = queries.contiguous()
    d = documents.contiguous()
    return (q, _i32(query_offsets), d, _i32(document_offsets),
            _i32(pair_query_ids), _i32(pair_document_ids))


def maxsim_forward(queries, query_offsets, documents, document_offsets,
                   pair_query_ids, pair_document_ids, max_q_len) -> torch.Tensor:
    dev = _require_cuda(queries, query_offsets, documents, document_offsets,
                        pair_query_ids, pair_document_ids)
    q, qoff, d, doff, pq, pd = _packed_args(queries, query_offsets, documents,
                                            document_offsets, pair_query_ids, pair_document_ids)
    n_pairs = pq.shape[0]
    scores = torch.empty((n_pairs,), dtype=torch.float32, device=dev)
    if n_pairs == 0:
        return scores
    max_q_len = int(max_q_len)
    if max_q_len < 0:
        # the reference infers the bound from query_offsets when given a negative value
        max_q_len = int((qoff[1:] - qoff[:-1]).max().item())
    if max_q_len <= 0:
        raise RuntimeError(f"max_q_len must be > 0; got {max_q_len}")
    with _on_device(dev):
        # score-only calls use the document order only if it is already known
        by_doc = _groups(pair_document_ids, pd, doff.shape[0] - 1, build=False)
        rc = load_library().maxsim_forward_ordered(
            _ptr(q), _ptr(qoff), _ptr(d), _ptr(doff), _ptr(pq), _ptr(pd),
            _ptr(by_doc[0]) if by_doc is not None else 0, _ptr(scores),
            n_pairs, qoff.shape[0] - 1, doff.shape[0] - 1, q.shape[0], d.shape[0],
            q.shape[1], max_q_len, _code(q), _stream_ptr())
    _check(rc, "maxsim_forward")
    return scores


def maxsim_packed_forward_with_argmax(queries, query_offsets, documents, document_offsets,
                                      pair_query_ids, pair_document_ids,
                                      max_q_len) -> Tuple[torch.Tensor, torch.Tensor]:
    dev = _require_cuda(queries, query_offsets, documents, document_offsets,
                        pair_query_ids, pair_document_ids)
    q, qoff, d, doff, pq, pd = _packed_args(queries, query_offsets, documents,
                                            document_offsets, pair_query_ids, pair_document_ids)
    max_q_len = int(max_q_len)
    if max_q_len <= 0:
        raise RuntimeError(f"max_q_len must be > 0; got {max_q_len}")
    n_pairs = pq.shape[0]
    scores = torch.empty((n_pairs,), dtype=torch.float32, device=dev)
    argmax = torch.empty((n_pairs, max_q_len), dtype=torch.int32, device=dev)
    if n_pairs == 0:
        return scores, argmax
    with _on_device(dev):
        by_doc = _groups(pair_document_ids, pd, doff.shape[0] - 1)
        rc = load_library().maxsim_packed_forward_with_argmax_ordered(
            _ptr(q), _ptr(qoff), _ptr(d), _ptr(doff), _ptr(pq), _ptr(pd),
            _ptr(by_doc[0]) if by_doc is not None else 0, _ptr(scores), _ptr(argmax),
            n_pairs, qoff.shape[0] - 1, doff.shape[0] - 1, q.shape[0], d.shape[0],
            q.shape[1], max_q_len, _code(q), _stream_ptr())
    _check(rc, "maxsim_packed_forward_with_argmax")
    return scores, argmax


def maxsim_packed_backward(dscore, queries, query_offsets, documents, document_offsets,
                           pair_query_ids, pair_document_ids, argmax,
                           max_q_len) -> Tuple[torch.Tensor, torch.Tensor]:
    dev = _require_cuda(queries, dscore, query_offsets, documents, document_offsets,
                        pair_query_ids, pair_document_ids, argmax)
    q, qoff, d, doff, pq, pd = _packed_args(queries, query_offsets, documents,
                                            document_offsets, pair_query_ids, pair_document_ids)
    g = dscore.contiguous().to(torch.float32)
    a = argmax.contiguous().to(torch.int32)
    n_pairs = pq.shape[0]
    max_q_len = int(max_q_len)
    if g.numel() != n_pairs:
        raise RuntimeError("dscore must have one entry per pair")
    if tuple(a.shape) != (n_pairs, max_q_len):
        raise RuntimeError("argmax must have shape [num_pairs, max_q_len]")
    dq = torch.empty(q.shape, dtype=torch.float32, device=dev)
    dd = torch.empty(d.shape, dtype=torch.float32, device=dev)
    with _on_device(dev):
        by_doc = _groups(pair_document_ids, pd, doff.shape[0] - 1)
        by_query = _groups(pair_query_ids, pq, qoff.shape[0] - 1)
        grouped = by_doc is not None and by_query is not None
        rc = load_library().maxsim_packed_backward_grouped(
            _ptr(g), _ptr(q), _ptr(qoff), _ptr(d), _ptr(doff), _ptr(pq), _ptr(pd),
            _ptr(by_query[0]) if grouped else 0, by_query[1].data_ptr() if grouped else 0,
            _ptr(by_doc[0]) if grouped else 0, by_doc[1].data_ptr() if grouped else 0, _ptr(a),
            _ptr(dq), _ptr(dd),
            n_pairs, qoff.shape[0] - 1, doff.shape[0] - 1, q.shape[0], d.shape[0],
            q.shape[1], max(max_q_len, 1), _code(q), _stream_ptr())
    _check(rc, "maxsim_packed_backward")
    return dq, dd


def packed_backward_native(dscore, queries, query_offsets, documents, document_offsets,
                           pair_query_ids, pair_document_ids, argmax, max_q_len):
    """As ``maxsim_packed_backward`` with both gradients in the inputs' float16
    / bfloat16 type, every row summed in fp32 and rounded once.  None when the
    shape is not covered (short or ungrouped pair lists, fp32 inputs, dim not a
    multiple of 8); the caller then uses the fp32 operator."""
    if not _native_grads or queries.dtype not in (torch.float16, torch.bfloat16):
        return None
    dev = _require_cuda(queries, dscore, query_offsets, documents, document_offsets,
                        pair_query_ids, pair_document_ids, argmax)
    q, qoff, d, doff, pq, pd = _packed_args(queries, query_offsets, documents,
                                            document_offsets, pair_query_ids, pair_document_ids)
    g = dscore.contiguous().to(torch.float32)
    a = argmax.contiguous().to(torch.int32)
    n_pairs, max_q_len = pq.shape[0], int(max_q_len)
    if g.numel() != n_pairs or tuple(a.shape) != (n_pairs, max_q_len) or n_pairs == 0:
        return None
    with _on_device(dev):
        by_doc = _groups(pair_document_ids, pd, doff.shape[0] - 1)
        by_query = _groups(pair_query_ids, pq, qoff.shape[0] - 1)
        if by_doc is None or by_query is None:
            return None
        dq = torch.empty(q.shape, dtype=q.dtype, device=dev)
        dd = torch.empty(d.shape, dtype=d.dtype, device=dev)
        rc = load_library().maxsim_packed_backward_grouped_native(
            _ptr(g), _ptr(q), _ptr(qoff), _ptr(d), _ptr(doff), _ptr(pq), _ptr(pd),
            _ptr(by_query[0]), by_query[1].data_ptr(), _ptr(by_doc[0]), by_doc[1].data_ptr(), _ptr(a),
            _ptr(dq), _ptr(dd), n_pairs, qoff.shape[0] - 1, doff.shape[0] - 1, q.shape[0], d.shape[0],
            q.shape[1], max_q_len, _code(q), _stream_ptr())
    if rc == _EUNSUPPORTED:
        return None
    _check(rc, "maxsim_packed_backward_grouped_native")
    return dq, dd


# ---------------------------------------------------------------------------
# padded
# ---------------------------------------------------------------------------

def _padded_args(queries, query_lengths, documents, doc_lengths, Lq_max, Ld_max, C):
    if queries.dim() != 2 or documents.dim() != 2:
        raise RuntimeError("queries/documents must be 2-D")
    if queries.shape[1] != documents.shape[1]:
        raise RuntimeError("queries.dim must match documents.dim")
    _same_float(queries, documents)
    Lq_max, Ld_max, C = int(Lq_max), int(Ld_max), int(C)
    if Lq_max <= 0 or Ld_max <= 0 or C <= 0:
        raise RuntimeError("Lq_max/Ld_max/num_candidates must all be > 0")
    q = queries.contiguous()
    d = documents.contiguous()
    if q.shape[0] % Lq_max != 0:
        raise RuntimeError("queries rows must be a multiple of Lq_max")
    if d.shape[0] % Ld_max != 0:
        raise RuntimeError("documents rows must be a multiple of Ld_max")
    B = q.shape[0] // Lq_max
    if d.shape[0] // Ld_max != B * C:
        raise RuntimeError("documents shape inconsistent with B * num_candidates")
    qlen = _i32(query_lengths)
    dlen = _i32(doc_lengths)
    if qlen.numel() != B or dlen.numel() != B * C:
        raise RuntimeError("length tensors inconsistent with B and num_candidates")
    return q, qlen, d, dlen, B, C, Lq_max, Ld_max


def maxsim_padded_forward(queries, query_lengths, documents, doc_lengths,
                          Lq_max, Ld_max, num_candidates) -> torch.Tensor:
    dev = _require_cuda(queries, query_lengths, documents, doc_lengths)
    q, qlen, d, dlen, B, C, Lq_max, Ld_max = _padded_args(
        queries, query_lengths, documents, doc_lengths, Lq_max, Ld_max, num_candidates)
    scores = torch.empty((B * C,), dtype=torch.float32, device=dev)
    if B * C == 0:
        return scores
    with _on_device(dev):
        rc = load_library().maxsim_padded_forward(
            _ptr(q), _ptr(qlen), _ptr(d), _ptr(dlen), _ptr(scores),
            B, C, Lq_max, Ld_max, q.shape[1], _code(q), _stream_ptr())
    _check(rc, "maxsim_padded_forward")
    return scores


def maxsim_padded_forward_with_argmax(queries, query_lengths, documents, doc_lengths,
                                      Lq_max, Ld_max, num_candidates):
    dev = _require_cuda(queries, query_lengths, documents, doc_lengths)
    q, qlen, d, dlen, B, C, Lq_max, Ld_max = _padded_args(
        queries, query_lengths, documents, doc_lengths, Lq_max, Ld_max, num_candidates)
    scores = torch.empty((B * C,), dtype=torch.float32, device=dev)
    argmax = torch.empty((B * C, Lq_max), dtype=torch.int32, device=dev)
    if B * C == 0:
        return scores, argmax
    with _on_device(dev):
        rc = load_library().maxsim_padded_forward_with_argmax(
            _ptr(q), _ptr(qlen), _ptr(d), _ptr(dlen), _ptr(scores), _ptr(argmax),
            B, C, Lq_max, Ld_max, q.shape[1], _code(q), _stream_ptr())
    _check(rc, "maxsim_padded_forward_with_argmax")
    return scores, argmax


def maxsim_padded_backward(dscore, queries, documents, query_lengths, doc_lengths, argmax,
                           Lq_max, Ld_max, num_candidates):
    dev = _require_cuda(queries, dscore, documents, query_lengths, doc_lengths, argmax)
    q, qlen, d, dlen, B, C, Lq_max, Ld_max = _padded_args(
        queries, query_lengths, documents, doc_lengths, Lq_max, Ld_max, num_candidates)
    g = dscore.contiguous().to(torch.float32)
    a = argmax.contiguous().to(torch.int32)
    if g.numel() != B * C:
        raise RuntimeError("dscore must have B * num_candidates entries")
    if a.numel() != B * C * Lq_max:
        raise RuntimeError("argmax must have shape [B * num_candidates, Lq_max]")
    dq = torch.empty(q.shape, dtype=torch.float32, device=dev)
    dd = torch.empty(d.shape, dtype=torch.float32, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_padded_backward(
            _ptr(g), _ptr(q), _ptr(d), _ptr(qlen), _ptr(dlen), _ptr(a), _ptr(dq), _ptr(dd),
            B, C, Lq_max, Ld_max, q.shape[1], _code(q), _stream_ptr())
    _check(rc, "maxsim_padded_backward")
    return dq, dd


_EUNSUPPORTED = -2
_native_grads = True


def set_native_gradients(enabled: bool) -> None:
    """Let the autograd functions ask the kernels for gradients in the inputs'
    16-bit type (default) or always take the fp32 operators and autograd's cast."""
    global _native_grads
    _native_grads = bool(enabled)


def padded_backward_native(dscore, queries, documents, query_lengths, doc_lengths, argmax,
                           Lq_max, Ld_max, num_candidates):
    """As ``maxsim_padded_backward`` but with both gradients in the inputs'
    float16 / bfloat16 type (each row summed in fp32 and rounded once).
    Returns None when the shape is not covered; the caller then uses the fp32
    operator."""
    if not _native_grads or queries.dtype not in (torch.float16, torch.bfloat16):
        return None
    dev = _require_cuda(queries, dscore, documents, query_lengths, doc_lengths, argmax)
    q, qlen, d, dlen, B, C, Lq_max, Ld_max = _padded_args(
        queries, query_lengths, documents, doc_lengths, Lq_max, Ld_max, num_candidates)
    g = dscore.contiguous().to(torch.float32)
    a = argmax.contiguous().to(torch.int32)
    if g.numel() != B * C or tuple(a.shape) != (B * C, Lq_max) or B * C == 0:
        return None
    dq = torch.empty(q.shape, dtype=q.dtype, device=dev)
    dd = torch.empty(d.shape, dtype=d.dtype, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_padded_backward_native(
            _ptr(g), _ptr(q), _ptr(d), _ptr(qlen), _ptr(dlen), _ptr(a), _ptr(dq), _ptr(dd),
            B, C, Lq_max, Ld_max, q.shape[1], _code(q), _stream_ptr())
    if rc == _EUNSUPPORTED:
        return None
    _check(rc, "maxsim_padded_backward_native")
    return dq, dd


def contrastive_backward_native(dscore, queries, documents, document_offsets, argmax,
                                want_documents: bool = True):
    """As ``maxsim_contrastive_backward`` with gradients in the inputs' 16-bit
    type; None when the shape is not covered.  With ``want_documents=False``
    only grad_queries is computed (the second entry of the pair is None)."""
    if not _native_grads or queries.dtype not in (torch.float16, torch.bfloat16):
        return None
    dev = _require_cuda(queries, dscore, documents, document_offsets, argmax)
    q, d, off, Nq, Lq, Nb, dim = _contrastive_args(queries, documents, document_offsets)
    g = dscore.contiguous().to(torch.float32)
    a = argmax.contiguous().to(torch.int32)
    if tuple(g.shape) != (Nq, Nb) or tuple(a.shape) != (Nq, Nb, Lq) or Nq * Nb == 0:
        return None
    dq = torch.empty(q.shape, dtype=q.dtype, device=dev)
    dd = torch.empty(d.shape, dtype=d.dtype, device=dev) if want_documents else None
    with _on_device(dev):
        rc = load_library().maxsim_contrastive_backward_native(
            _ptr(g), _ptr(q), _ptr(d), _ptr(off), _ptr(a), _ptr(dq), _ptr(dd) if dd is not None else 0,
            Nq, Lq, Nb, dim, d.shape[0], _code(q), _stream_ptr())
    if rc == _EUNSUPPORTED:
        return None
    _check(rc, "maxsim_contrastive_backward_native")
    return dq, dd


# ---------------------------------------------------------------------------
# contrastive
# ---------------------------------------------------------------------------

def _contrastive_args(queries, documents, document_offsets):
    if queries.dim() != 3:
        raise RuntimeError("queries must be [Nq, Lq, D]")
    if documents.dim() != 2:
        raise RuntimeError("documents must be [total_d_tokens, D]")
    if document_offsets.dim() != 1:
        raise RuntimeError("document_offsets must be 1-D")
    if queries.shape[2] != documents.shape[1]:
        raise RuntimeError("queries.D must match documents.D")
    _same_float(queries, documents)
    q = queries.contiguous()
    d = documents.contiguous()
    off = _i32(document_offsets)
    Nq, Lq, dim = q.shape
    Nb = off.shape[0] - 1
    if Nb < 0:
        raise RuntimeError("document_offsets must have at least 1 element")
    if Lq <= 0:
        raise RuntimeError("Lq must be > 0")
    if dim <= 0:
        raise RuntimeError("dim must be > 0")
    return q, d, off, Nq, Lq, Nb, dim


def maxsim_contrastive_forward(queries, documents, document_offsets) -> torch.Tensor:
    dev = _require_cuda(queries, documents, document_offsets)
    q, d, off, Nq, Lq, Nb, dim = _contrastive_args(queries, documents, document_offsets)
    scores = torch.empty((Nq, Nb), dtype=torch.float32, device=dev)
    if Nq * Nb == 0:
        return scores
    with _on_device(dev):
        rc = load_library().maxsim_contrastive_forward(
            _ptr(q), _ptr(d), _ptr(off), _ptr(scores),
            Nq, Lq, Nb, dim, d.shape[0], _code(q), _stream_ptr())
    _check(rc, "maxsim_contrastive_forward")
    return scores


def maxsim_contrastive_forward_with_argmax(queries, documents, document_offsets):
    dev = _require_cuda(queries, documents, document_offsets)
    q, d, off, Nq, Lq, Nb, dim = _contrastive_args(queries, documents, document_offsets)
    scores = torch.empty((Nq, Nb), dtype=torch.float32, device=dev)
    argmax = torch.empty((Nq, Nb, Lq), dtype=torch.int32, device=dev)
    if Nq * Nb == 0:
        return scores, argmax
    with _on_device(dev):
        rc = load_library().maxsim_contrastive_forward_with_argmax(
            _ptr(q), _ptr(d), _ptr(off), _ptr(scores), _ptr(argmax),
            Nq, Lq, Nb, dim, d.shape[0], _code(q), _stream_ptr())
    _check(rc, "maxsim_contrastive_forward_with_argmax")
    return scores, argmax


def contrastive_forward_block(queries, documents, block_offsets, scores, argmax, col0: int,
                              block_tokens: int = 0, reserve_sms: int = 0) -> bool:
    """Scores ``queries [Nq, Lq, D]`` against the documents described by
    ``block_offsets [n + 1]`` (absolute token rows of the packed ``documents``)
    and writes them into columns ``[col0, col0 + n)`` of the caller's
    ``scores [Nq, Nb_total]`` fp32 and ``argmax [Nq, Nb_total, Lq]`` int32: several
    launches over different document ranges (or different ``documents``
    tensors) fill one score matrix.  ``block_tokens`` is the number of tokens
    in the block when known (it steers the choice of tiling); ``reserve_sms``
    SMs are left unused for a collective meant to run beside the launch (the
    kernel otherwise holds every SM until it ends).  Returns False
    when the shape is outside what the tcgen05 kernel covers (nothing was
    written); the caller then scores the block on its own and copies."""
    dev = _require_cuda(queries, documents, block_offsets, scores, argmax)
    q, d, off, Nq, Lq, n, dim = _contrastive_args(queries, documents, block_offsets)
    if scores.dtype != torch.float32 or argmax.dtype != torch.int32 or not scores.is_contiguous() \
            or not argmax.is_contiguous() or scores.dim() != 2 or scores.shape[0] != Nq \
            or tuple(argmax.shape) != (Nq, scores.shape[1], Lq):
        raise RuntimeError("scores must be contiguous [Nq, Nb_total] float32 and argmax [Nq, Nb_total, Lq] int32")
    if Nq * n == 0:
        return True
    with _on_device(dev):
        rc = load_library().maxsim_contrastive_forward_with_argmax_block(
            _ptr(q), _ptr(d), _ptr(off), scores.data_ptr(), argmax.data_ptr(),
            Nq, Lq, n, dim, d.shape[0], int(block_tokens), scores.shape[1], int(col0),
            int(reserve_sms), _code(q), _stream_ptr())
    if rc == _EUNSUPPORTED:
        return False
    _check(rc, "maxsim_contrastive_forward_with_argmax_block")
    return True


def pack_owner_records(argmax, dscore, col_start) -> torch.Tensor:
    """Regroups the pairs of this rank's queries by the rank that owns the
    document: ``argmax [Nq, Nb, Lq]`` int32 and ``dscore [Nq, Nb]`` fp32 become
    one int32 buffer in which owner ``o``'s block ``[Nq, n_o, Lq + 1]`` (the
    winning tokens, then the bits of the score gradient) starts at word
    ``col_start[o] * Nq * (Lq + 1)``; ``col_start [R + 1]`` int32 on the device
    holds the first column of every owner."""
    dev = _require_cuda(argmax, dscore, col_start)
    a = argmax.contiguous()
    g = dscore.contiguous().to(torch.float32)
    cs = _i32(col_start)
    Nq, Nb, Lq = a.shape
    send = torch.empty((Nq * Nb * (Lq + 1),), dtype=torch.int32, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_b200_pack_owner_records(
            _ptr(a), _ptr(g), _ptr(cs), cs.shape[0] - 1, Nq, Nb, Lq, _ptr(send), _stream_ptr())
    _check(rc, "maxsim_b200_pack_owner_records")
    return send


def pack_owner_records_to(argmax, dscore, col_start, owner_blocks) -> None:
    """:func:`pack_owner_records` without the send buffer: owner ``o``'s block
    is written to the address ``owner_blocks[o]`` (``[R]`` int64 on the device:
    pointers into the owners' memory as mapped in this process)."""
    dev = _require_cuda(argmax, dscore, col_start, owner_blocks)
    a = argmax.contiguous()
    g = dscore.contiguous().to(torch.float32)
    cs = _i32(col_start)
    if owner_blocks.dtype != torch.int64 or owner_blocks.numel() != cs.shape[0] - 1:
        raise ValueError("owner_blocks must hold one int64 address per owner")
    Nq, Nb, Lq = a.shape
    with _on_device(dev):
        rc = load_library().maxsim_b200_pack_owner_records_to(
            _ptr(a), _ptr(g), _ptr(cs), owner_blocks.data_ptr(), cs.shape[0] - 1, Nq, Nb, Lq,
            _stream_ptr())
    _check(rc, "maxsim_b200_pack_owner_records_to")


def peer_gather(table, max_bytes: int, dst0, dst1=None) -> None:
    """One launch that copies the segments listed in ``table`` (``[n, 4]`` int64
    on the device: source address, destination 0 / 1, byte offset there, bytes)
    out of peer-mapped memory into ``dst0`` / ``dst1``."""
    dev = _require_cuda(table, dst0)
    if table.dtype != torch.int64 or table.dim() != 2 or table.shape[1] != 4 or not table.is_contiguous():
        raise ValueError("table must be a contiguous [n, 4] int64 tensor")
    with _on_device(dev):
        rc = load_library().maxsim_b200_peer_gather(
            table.data_ptr(), table.shape[0], int(max_bytes), dst0.data_ptr(),
            dst1.data_ptr() if dst1 is not None else None, _stream_ptr())
    _check(rc, "maxsim_b200_peer_gather")


def copy_many(dst_addresses, src_addresses, sizes, device) -> None:
    """``len(sizes)`` asynchronous device-to-device copies on the current stream
    of ``device`` (addresses and byte counts as Python ints) with one call
    into the library."""
    n = len(sizes)
    if not (len(dst_addresses) == len(src_addresses) == n):
        raise ValueError("dst_addresses, src_addresses and sizes must have one entry per copy")
    if n == 0:
        return
    dst = (ctypes.c_void_p * n)(*dst_addresses)
    src = (ctypes.c_void_p * n)(*src_addresses)
    nbytes = (ctypes.c_int64 * n)(*sizes)
    with _on_device(torch.device(device)):
        rc = load_library().maxsim_b200_copy_many(dst, src, nbytes, n, _stream_ptr())
    _check(rc, "maxsim_b200_copy_many")


def peer_barrier(flags, rank: int, world: int, counter, polls: int = 0) -> None:
    """Stream-ordered barrier between the ranks of a node over flag words in
    peer-mapped memory (``flags``: ``[world]`` int64 addresses on the device,
    see the header); ``counter`` is this rank's one-word int32 tensor in which
    the kernel counts the barriers passed."""
    dev = _require_cuda(flags, counter)
    if counter.dtype != torch.int32 or counter.numel() != 1:
        raise ValueError("counter must be a one-element int32 tensor")
    with _on_device(dev):
        rc = load_library().maxsim_b200_peer_barrier(
            flags.data_ptr(), int(rank), int(world), counter.data_ptr(), int(polls), _stream_ptr())
    _check(rc, "maxsim_b200_peer_barrier")


def contrastive_backward_documents_from_records(records, queries, documents, document_offsets):
    """grad_documents of this rank's ``documents`` from ``records [Nq_all, Nb_own,
    Lq + 1]`` int32 (see :func:`pack_owner_records`) and the queries of all
    ranks ``[Nq_all, Lq, D]``.  The gradient comes back in the inputs' 16-bit
    type when the shape allows rounding once on store, else in fp32; None when
    the kernel does not cover the shape."""
    dev = _require_cuda(queries, records, documents, document_offsets)
    q, d, off, Nq, Lq, Nb, dim = _contrastive_args(queries, documents, document_offsets)
    r = records.contiguous()
    if r.dtype != torch.int32 or r.numel() != Nq * Nb * (Lq + 1):
        raise RuntimeError("records must be int32 [Nq, Nb, Lq + 1]")
    lib = load_library()
    for native in ((1, 0) if (_native_grads and q.dtype in (torch.float16, torch.bfloat16)) else (0,)):
        dd = torch.empty(d.shape, dtype=q.dtype if native else torch.float32, device=dev)
        with _on_device(dev):
            rc = lib.maxsim_contrastive_backward_documents_from_records(
                _ptr(r), _ptr(q), _ptr(d), _ptr(off), _ptr(dd), Nq, Lq, Nb, dim, d.shape[0],
                _code(q), native, _stream_ptr())
        if rc == 0:
            return dd
        if rc != _EUNSUPPORTED:
            _check(rc, "maxsim_contrastive_backward_documents_from_records")
    return None


def contrastive_backward_part(dscore, queries, documents, document_offsets, argmax, *,
                              want_queries: bool, want_documents: bool):
    """``maxsim_contrastive_backward`` computing only the requested gradients
    (fp32); the other entry of the returned pair is None."""
    dev = _require_cuda(queries, dscore, documents, document_offsets, argmax)
    q, d, off, Nq, Lq, Nb, dim = _contrastive_args(queries, documents, document_offsets)
    g = dscore.contiguous().to(torch.float32)
    a = argmax.contiguous().to(torch.int32)
    if tuple(g.shape) != (Nq, Nb):
        raise RuntimeError("dscore must have shape [Nq, Nb]")
    if tuple(a.shape) != (Nq, Nb, Lq):
        raise RuntimeError("argmax must have shape [Nq, Nb, Lq]")
    dq = torch.empty(q.shape, dtype=torch.float32, device=dev) if want_queries else None
    dd = torch.empty(d.shape, dtype=torch.float32, device=dev) if want_documents else None
    with _on_device(dev):
        rc = load_library().maxsim_contrastive_backward(
            _ptr(g), _ptr(q), _ptr(d), _ptr(off), _ptr(a),
            _ptr(dq) if dq is not None else 0, _ptr(dd) if dd is not None else 0,
            Nq, Lq, Nb, dim, d.shape[0], _code(q), _stream_ptr())
    _check(rc, "maxsim_contrastive_backward")
    return dq, dd


def maxsim_contrastive_backward(dscore, queries, documents, document_offsets, argmax):
    dev = _require_cuda(queries, dscore, documents, document_offsets, argmax)
    q, d, off, Nq, Lq, Nb, dim = _contrastive_args(queries, documents, document_offsets)
    g = dscore.contiguous().to(torch.float32)
    a = argmax.contiguous().to(torch.int32)
    if tuple(g.shape) != (Nq, Nb):
        raise RuntimeError("dscore must have shape [Nq, Nb]")
    if tuple(a.shape) != (Nq, Nb, Lq):
        raise RuntimeError("argmax must have shape [Nq, Nb, Lq]")
    dq = torch.empty(q.shape, dtype=torch.float32, device=dev)
    dd = torch.empty(d.shape, dtype=torch.float32, device=dev)
    with _on_device(dev):
        rc = load_library().maxsim_contrastive_backward(
            _ptr(g), _ptr(q), _ptr(d), _ptr(off), _ptr(a), _ptr(dq), _ptr(dd),
            Nq, Lq, Nb, dim, d.shape[0], _code(q), _stream_ptr())
    _check(rc, "maxsim_contrastive_backward")
    return dq, dd


ops = types.SimpleNamespace(
    maxsim_forward=maxsim_forward,
    maxsim_padded_forward=maxsim_padded_forward,
    maxsim_padded_forward_with_argmax=maxsim_padded_forward_with_argmax,
    maxsim_padded_backward=maxsim_padded_backward,
    maxsim_packed_forward_with_argmax=maxsim_packed_forward_with_argmax,
    maxsim_packed_backward=maxsim_packed_backward,
    maxsim_contrastive_forward=maxsim_contrastive_forward,
    maxsim_contrastive_forward_with_argmax=maxsim_contrastive_forward_with_argmax,
    maxsim_contrastive_backward=maxsim_contrastive_backward,
)
