"""Seeded synthetic workloads with the shapes and value distributions of the
five benchmark configurations.

The reference measures only on synthetic ``randn`` tensors
(``scripts/bench_matrix.py:291-299, 391-399``); no dataset is involved.  Every
token vector here is i.i.d. N(0,1) in fp32, L2-normalised, then cast to the
configuration's dtype.  Lengths follow the distribution each configuration
names.  All generators take explicit sizes so that the tests can run the same
distributions at sizes a CPU oracle finishes in seconds.

Two families:

* ``*_numpy`` -- ``numpy.random.Generator(PCG64)`` streams, bit-reproducible
  on any machine; used by the golden fixtures and the parity tests.
* ``*_device`` -- generated directly on a CUDA device with a per-query /
  per-document seed, so a shard generated on rank r equals the same rows of
  the unsharded tensor; used by the benchmark at full size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import numpy as np
import torch

_TORCH_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def _unit_rows(rng: np.random.Generator, n: int, dim: int) -> np.ndarray:
    x = rng.standard_normal((n, dim), dtype=np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return x


@dataclass
class PaddedWorkload:
    queries: np.ndarray        # [B, Lq, dim] fp32 unit rows
    documents: np.ndarray      # [B, C, Ld, dim] fp32 unit rows (padding rows are unit noise too)
    query_lengths: np.ndarray  # [B] int32
    doc_lengths: np.ndarray    # [B, C] int32
    dtype: str = "fp32"
    name: str = ""


@dataclass
class ContrastiveWorkload:
    queries: np.ndarray           # [Nq, Lq, dim]
    documents: np.ndarray         # [T_d, dim]
    document_offsets: np.ndarray  # [Nb+1] int32
    dtype: str = "bf16"
    name: str = ""


@dataclass
class PackedWorkload:
    queries: np.ndarray
    query_offsets: np.ndarray
    documents: np.ndarray
    document_offsets: np.ndarray
    pair_query_ids: np.ndarray
    pair_document_ids: np.ndarray
    dscore: np.ndarray            # [P] fp32 upstream gradient
    dtype: str = "fp16"
    name: str = ""


def _offsets(lengths: np.ndarray) -> np.ndarray:
    out = np.zeros(lengths.shape[0] + 1, dtype=np.int32)
    np.cumsum(lengths, out=out[1:])
    return out


def c1_padded_rerank_fp32(seed: int = 0, Nq: int = 16, Lq: int = 32, C: int = 32,
                          Ld: int = 300, dim: int = 128, lo: int = 64) -> PaddedWorkload:
    """Padded rerank forward, fp32; doc lengths uniform in [lo, Ld]."""
    rng = np.random.default_rng(seed)
    q = _unit_rows(rng, Nq * Lq, dim).reshape(Nq, Lq, dim)
    d = _unit_rows(rng, Nq * C * Ld, dim).reshape(Nq, C, Ld, dim)
    dlen = rng.integers(lo, Ld + 1, size=(Nq, C)).astype(np.int32)
    qlen = np.full(Nq, Lq, dtype=np.int32)
    return PaddedWorkload(q, d, qlen, dlen, "fp32", "c1_padded_rerank_fp32")


def c2_contrastive_train_bf16(seed: int = 1, Nq: int = 64, Nb: int = 64, Lq: int = 32,
                              dim: int = 128, lo: int = 32, hi: int = 256,
                              dtype: str = "bf16") -> ContrastiveWorkload:
    """Contrastive train, doc lengths uniform in [lo, hi], offsets by cumsum."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, size=Nb).astype(np.int32)
    q = _unit_rows(rng, Nq * Lq, dim).reshape(Nq, Lq, dim)
    d = _unit_rows(rng, int(lens.sum()), dim)
    return ContrastiveWorkload(q, d, _offsets(lens), dtype, "c2_contrastive_train")


def lognormal_lengths(rng: np.random.Generator, n, median: float, sigma: float,
                      lo: int, hi: int) -> np.ndarray:
    x = rng.lognormal(mean=np.log(median), sigma=sigma, size=n)
    return np.clip(np.rint(x), lo, hi).astype(np.int32)


def c3_large_rerank_fp16(seed: int = 2, Nq: int = 256, Lq: int = 32, C: int = 1000,
                         Ld: int = 300, dim: int = 128) -> PaddedWorkload:
    """Large padded rerank; lognormal(ln 180, 0.4) doc lengths clipped to
    [16, Ld]; the last 0-4 query tokens masked (query_lengths = Lq - U{0..4})."""
    rng = np.random.default_rng(seed)
    q = _unit_rows(rng, Nq * Lq, dim).reshape(Nq, Lq, dim)
    d = _unit_rows(rng, Nq * C * Ld, dim).reshape(Nq, C, Ld, dim)
    dlen = lognormal_lengths(rng, (Nq, C), 180.0, 0.4, min(16, Ld), Ld)
    qlen = (Lq - rng.integers(0, 5, size=Nq)).clip(1, Lq).astype(np.int32)
    return PaddedWorkload(q, d, qlen, dlen, "fp16", "c3_large_rerank_fp16")


def c4_packed_grid_fp16(seed: int = 3, n_queries: int = 2000, n_docs: int = 20000,
                        n_pairs: int = 65536, dim: int = 96) -> PackedWorkload:
    """Packed ragged pair grid; duplicates in the pair list are expected."""
    rng = np.random.default_rng(seed)
    qlens = rng.integers(8, 33, size=n_queries).astype(np.int32)
    dlens = lognormal_lengths(rng, n_docs, 120.0, 0.6, 8, 512)
    q = _unit_rows(rng, int(qlens.sum()), dim)
    d = _unit_rows(rng, int(dlens.sum()), dim)
    qids = rng.integers(0, n_queries, size=n_pairs).astype(np.int32)
    dids = rng.integers(0, n_docs, size=n_pairs).astype(np.int32)
    g = rng.standard_normal(n_pairs, dtype=np.float32)
    return PackedWorkload(q, _offsets(qlens), d, _offsets(dlens), qids, dids, g,
                          "fp16", "c4_packed_grid_fp16")


def c5_contrastive_ties_bf16(seed: int = 4, Nq: int = 1024, Nb: int = 1024, Lq: int = 32,
                             dim: int = 128, lo: int = 64, hi: int = 512,
                             dup_frac: float = 0.05) -> ContrastiveWorkload:
    """Contrastive train with 5% of every document's tokens overwritten by a
    verbatim copy of another token of the same document (forces exact ties)."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, size=Nb).astype(np.int32)
    offs = _offsets(lens)
    q = _unit_rows(rng, Nq * Lq, dim).reshape(Nq, Lq, dim)
    d = _unit_rows(rng, int(lens.sum()), dim)
    for i in range(Nb):
        n = int(lens[i])
        k = int(round(dup_frac * n))
        if k == 0 or n < 2:
            continue
        dst = rng.choice(n, size=k, replace=False)
        src = rng.integers(0, n, size=k)
        src = np.where(src == dst, (src + 1) % n, src)
        # copy from a snapshot so chains of copies stay verbatim copies of originals
        seg = d[offs[i]:offs[i + 1]]
        seg[dst] = seg.copy()[src]
    return ContrastiveWorkload(q, d, offs, "bf16", "c5_contrastive_ties_bf16")


def to_torch(x: np.ndarray, dtype: str, device="cpu") -> torch.Tensor:
    """Cast an fp32 numpy array onto the grid of ``dtype`` (round-to-nearest)."""
    return torch.from_numpy(np.ascontiguousarray(x)).to(device=device, dtype=_TORCH_DTYPES[dtype])


def on_grid(x: np.ndarray, dtype: str) -> np.ndarray:
    """The fp32 values of ``x`` after a round trip through ``dtype``."""
    return to_torch(x, dtype).float().numpy()


# ---------------------------------------------------------------------------
# Device-side generation for full-size benchmark runs
# ---------------------------------------------------------------------------

def _device_unit_rows(n: int, dim: int, seed: int, device, dtype) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = torch.randn((n, dim), generator=g, device=device, dtype=torch.float32)
    x = torch.nn.functional.normalize(x, dim=1)
    return x.to(dtype)


def c3_shard_lengths(q_begin: int, q_end: int, *, seed: int = 2, Lq: int = 32, C: int = 1000,
                     Ld: int = 300):
    """``(query_lengths [n], doc_lengths [n, C])`` (int32 numpy) of queries
    ``[q_begin, q_end)`` of the large rerank configuration: the lengths
    :func:`c3_device_shard` generates, without touching a device."""
    n = q_end - q_begin
    qlen = np.empty((n,), dtype=np.int32)
    dlen = np.empty((n, C), dtype=np.int32)
    for i, qi in enumerate(range(q_begin, q_end)):
        rng = np.random.default_rng([seed, qi])
        dlen[i] = lognormal_lengths(rng, C, 180.0, 0.4, min(16, Ld), Ld)
        qlen[i] = int(Lq - rng.integers(0, 5))
    return qlen, dlen


def c3_device_shard(q_begin: int, q_end: int, device, *, seed: int = 2, Lq: int = 32,
                    C: int = 1000, Ld: int = 300, dim: int = 128,
                    dtype: torch.dtype = torch.float16) -> Dict[str, torch.Tensor]:
    """Queries ``[q_begin, q_end)`` of the large rerank configuration, generated
    on ``device``.  Every query's tensors depend only on ``(seed, query index)``,
    so any sharding of the query range yields the same global data."""
    n = q_end - q_begin
    queries = torch.empty((n, Lq, dim), device=device, dtype=dtype)
    documents = torch.empty((n, C, Ld, dim), device=device, dtype=dtype)
    qlen_np, dlen_np = c3_shard_lengths(q_begin, q_end, seed=seed, Lq=Lq, C=C, Ld=Ld)
    qlen, dlen = torch.from_numpy(qlen_np), torch.from_numpy(dlen_np)
    for i, qi in enumerate(range(q_begin, q_end)):
        s = (seed * 1_000_003 + qi) * 2 + 1
        queries[i] = _device_unit_rows(Lq, dim, s, device, dtype).view(Lq, dim)
        documents[i] = _device_unit_rows(C * Ld, dim, s + 1, device, dtype).view(C, Ld, dim)
    return dict(queries=queries, documents=documents,
                query_lengths=qlen.to(device), doc_lengths=dlen.to(device))


def c5_device(device, *, seed: int = 4, Nq: int = 1024, Nb: int = 1024, Lq: int = 32,
              dim: int = 128, lo: int = 64, hi: int = 512, dup_frac: float = 0.05,
              dtype: torch.dtype = torch.bfloat16,
              q_begin: int = 0, q_end: Optional[int] = None,
              d_begin: int = 0, d_end: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Contrastive-with-ties configuration on ``device``.  ``q_begin:q_end`` and
    ``d_begin:d_end`` select a rank's query rows and documents; document lengths
    come from one global stream so every rank agrees on them."""
    q_end = Nq if q_end is None else q_end
    d_end = Nb if d_end is None else d_end
    lens_all = np.random.default_rng([seed, 0]).integers(lo, hi + 1, size=Nb).astype(np.int32)
    lens = lens_all[d_begin:d_end]
    offs = _offsets(lens)
    queries = torch.empty((q_end - q_begin, Lq, dim), device=device, dtype=dtype)
    for i, qi in enumerate(range(q_begin, q_end)):
        queries[i] = _device_unit_rows(Lq, dim, (seed * 1_000_003 + qi) * 2 + 1, device, dtype)
    docs = torch.empty((int(lens.sum()), dim), device=device, dtype=dtype)
    for i, di in enumerate(range(d_begin, d_end)):
        n = int(lens[i])
        seg = _device_unit_rows(n, dim, (seed * 1_000_003 + di) * 2 + 2, device, dtype)
        k = int(round(dup_frac * n))
        if k > 0 and n >= 2:
            rng = np.random.default_rng([seed, 1, di])
            dst = rng.choice(n, size=k, replace=False)
            src = rng.integers(0, n, size=k)
            src = np.where(src == dst, (src + 1) % n, src)
            snap = seg.clone()
            seg[torch.from_numpy(dst).to(device)] = snap[torch.from_numpy(src).to(device)]
        docs[int(offs[i]):int(offs[i + 1])] = seg
    return dict(queries=queries, documents=docs,
                document_offsets=torch.from_numpy(offs).to(device),
                doc_lengths_all=torch.from_numpy(lens_all))
