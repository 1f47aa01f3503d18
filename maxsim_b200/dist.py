"""Multi-GPU drivers: one process per GPU, ``torch.distributed`` for the plumbing.

The reference has no multi-device code at all; these two drivers sit *outside*
the operator boundary and only decide which rank scores what.

Rerank (padded / packed candidates)
    Pairs are independent, so queries -- with their candidate lists -- are
    split across ranks and each rank calls the ordinary operator on its shard.
    There is no collective on the data path (:func:`shard_range`,
    :func:`score_candidates_padded_sharded`).

Contrastive training
    Rank r owns ``Nq/R`` queries and ``Nb/R`` documents.  Forward: the packed
    document shards are all-gathered.  They are ragged, so each is padded to a
    common row count for the collective; the gathered buffer is never
    compacted -- it is handed to the operator as one packed tensor in which
    every rank's padding rows form one filler document whose score column is
    dropped.  One forward launch therefore scores the rank's queries against
    all documents.  Backward: one launch routes the gradient; the partial
    ``grad_documents`` of the whole buffer is reduce-scattered so each owner
    receives the sum for its shard; ``grad_queries`` stays local.  Scores come
    back as ``[Nq_local, Nb_total]`` with document columns in rank order, so
    diagonal targets are ``rank_query_offset + arange(Nq_local)``
    (:func:`score_contrastive_sharded`).

Both drivers take the operator namespace as a parameter so that their
sharding / reassembly logic can be exercised on CPU ``gloo`` ranks with a
stand-in scorer; the default is the CUDA library.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = [
    "shard_range", "score_candidates_padded_sharded", "score_contrastive_sharded",
    "contrastive_targets", "offsets_from_lengths",
]


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, as-even-as-possible split of ``range(n)``: the first
    ``n % world`` ranks get one extra element."""
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def offsets_from_lengths(lengths: torch.Tensor) -> torch.Tensor:
    off = torch.zeros(lengths.numel() + 1, dtype=torch.int32, device=lengths.device)
    off[1:] = torch.cumsum(lengths.to(torch.int64), 0).to(torch.int32)
    return off


def _default_ops():
    import types

    from . import _ops
    return types.SimpleNamespace(**vars(_ops.ops),
                                 contrastive_backward_part=_ops.contrastive_backward_part)


def _world(group) -> Tuple[int, int]:
    if not dist.is_available() or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


# ---------------------------------------------------------------------------
# Rerank: shard by query, no data-path collective
# ---------------------------------------------------------------------------

def score_candidates_padded_sharded(queries, documents, query_lengths, doc_lengths, *,
                                    group=None, gather: bool = False, scorer=None):
    """Score this rank's shard of queries (``[B_local, Lq, D]`` with their
    ``[B_local, C, Ld, D]`` candidates).  Returns ``[B_local, C]`` scores, or,
    with ``gather=True``, the ``[B_total, C]`` scores of all ranks in rank
    order (the only collective, and only for reporting)."""
    if scorer is None:
        from . import score_candidates_padded as scorer
    local = scorer(queries, documents, query_lengths, doc_lengths)
    rank, world = _world(group)
    if not gather or world == 1:
        return local
    counts = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    all_counts = [torch.zeros_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts, group=group)
    sizes = [int(c.item()) for c in all_counts]
    pad = max(sizes)
    buf = local.new_zeros((pad, local.shape[1]))
    buf[: local.shape[0]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)


# ---------------------------------------------------------------------------
# Contrastive training: all-gather documents, per-owner gradient reduction
# ---------------------------------------------------------------------------

def _gather_shards(documents: torch.Tensor, lengths: torch.Tensor, group, world: int,
                   n_queries: int = 0, shard_sizes=None):
    """All-gather ragged packed shards into one buffer.

    Every shard is padded to ``t_pad = longest shard + 1`` token rows, so the
    gathered buffer ``[world * t_pad, D]`` holds rank r's tokens at rows
    ``[r * t_pad, r * t_pad + T_r)`` followed by at least one padding row.  The
    buffer is then described to the operators as ONE packed document tensor:
    rank r's real documents followed by one filler document that covers its
    padding rows.  Returns the buffer, the combined int32 offsets, the column
    indices of the real (non-filler) documents, the number of columns, the
    per-rank ``(tokens, documents, queries)`` sizes and ``t_pad``."""
    dev = documents.device
    nccl = dist.get_backend(group) == "nccl"
    if shard_sizes is not None:
        # the caller already knows every rank's (tokens, documents, queries): no
        # exchange and, above all, no wait for the device on the host
        sizes = [(int(t), int(n), int(nq)) for t, n, nq in shard_sizes]
        rank = dist.get_rank(group)
        if len(sizes) != world or sizes[rank] != (documents.shape[0], lengths.numel(), n_queries):
            raise ValueError(f"shard_sizes[{rank}] = {sizes[rank] if len(sizes) == world else None} does not "
                             f"describe this rank's shard {(documents.shape[0], lengths.numel(), n_queries)}")
    else:
        meta = torch.tensor([documents.shape[0], lengths.numel(), n_queries], dtype=torch.int64, device=dev)
        metas = torch.empty((world, 3), dtype=torch.int64, device=dev)
        if nccl:
            dist.all_gather_into_tensor(metas, meta, group=group)
        else:
            dist.all_gather(list(metas.unbind(0)), meta, group=group)
        sizes = [(int(t), int(n), int(nq)) for t, n, nq in metas.tolist()]  # one transfer for all ranks
    t_pad = max(s[0] for s in sizes) + 1
    n_max = max(s[1] for s in sizes)

    doc_pad = documents.new_zeros((t_pad, documents.shape[1]))
    doc_pad[: documents.shape[0]] = documents
    doc_parts = torch.empty((world * t_pad, documents.shape[1]), dtype=documents.dtype, device=dev)
    if nccl:
        handle = dist.all_gather_into_tensor(doc_parts, doc_pad, group=group, async_op=True)
    else:
        handle = dist.all_gather(list(doc_parts.view(world, t_pad, -1).unbind(0)), doc_pad,
                                 group=group, async_op=True)

    len_pad = torch.zeros(n_max, dtype=torch.int32, device=dev)
    len_pad[: lengths.numel()] = lengths.to(torch.int32)
    len_all = torch.empty((world, n_max), dtype=torch.int32, device=dev)
    if nccl:
        dist.all_gather_into_tensor(len_all, len_pad, group=group)
    else:
        dist.all_gather(list(len_all.unbind(0)), len_pad, group=group)
    len_parts = len_all.unbind(0)

    # combined document list: real documents of rank r, then its filler.  The
    # column indices of the real documents are built on the host (the sizes are
    # already there), so selecting them later needs no device synchronisation.
    fillers = torch.tensor([t_pad - s[0] for s in sizes], dtype=torch.int32).to(dev, non_blocking=True)
    pieces, real_cols, base = [], [], 0
    for r in range(world):
        n_r = sizes[r][1]
        pieces.append(len_parts[r][:n_r])
        pieces.append(fillers[r:r + 1])
        real_cols.extend(range(base, base + n_r))
        base += n_r + 1
    offsets = offsets_from_lengths(torch.cat(pieces))
    real = torch.tensor(real_cols, dtype=torch.int64).to(dev, non_blocking=True)
    handle.wait()
    return doc_parts, offsets, real, base, sizes, t_pad


def _reduce_scatter_rows(full: torch.Tensor, world: int, rank: int, group) -> torch.Tensor:
    """Sum ``full [world * t_pad, D]`` over the ranks and return this rank's
    ``[t_pad, D]`` block.  NCCL does it in one reduce-scatter; backends without
    one (gloo, used by the CPU tests) all-reduce and slice."""
    t_pad = full.shape[0] // world
    if dist.get_backend(group) == "nccl":
        out = torch.empty((t_pad, full.shape[1]), dtype=full.dtype, device=full.device)
        dist.reduce_scatter_tensor(out, full, group=group)
        return out
    dist.all_reduce(full, group=group)
    return full[rank * t_pad:(rank + 1) * t_pad]


def _all_gather_rows(x: torch.Tensor, rows_per_rank: Sequence[int], group, world: int) -> torch.Tensor:
    """Concatenate every rank's ``x [rows_r, ...]`` along dim 0 (``rows_r`` may differ)."""
    n_max = max(rows_per_rank)
    pad = x
    if x.shape[0] != n_max:
        pad = x.new_zeros((n_max,) + tuple(x.shape[1:]))
        pad[: x.shape[0]] = x
    out = torch.empty((world * n_max,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, pad.contiguous(), group=group)
    else:
        dist.all_gather(list(out.view((world, n_max) + tuple(x.shape[1:])).unbind(0)), pad.contiguous(),
                        group=group)
    if all(n == n_max for n in rows_per_rank):
        return out
    parts = out.view((world, n_max) + tuple(x.shape[1:]))
    return torch.cat([parts[r, : rows_per_rank[r]] for r in range(world)], dim=0)


def _columns_to_owners(x: torch.Tensor, docs_per_rank: Sequence[int], queries_per_rank: Sequence[int],
                       rank: int, group) -> torch.Tensor:
    """``x [Nq_local, Nb_total, W]`` holds, for this rank's queries, one record
    of W ints per document column (columns in rank order).  Every owner gets
    the records of its own documents from all ranks: returns
    ``[Nq_total, Nb_own, W]`` with queries in rank order."""
    nq_local, _, width = x.shape
    send = x.transpose(0, 1).contiguous().view(-1)                 # [Nb_total, Nq_local, W]
    in_splits = [n * nq_local * width for n in docs_per_rank]
    n_own = docs_per_rank[rank]
    out_splits = [n_own * nq * width for nq in queries_per_rank]
    recv = torch.empty((sum(out_splits),), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, send, out_splits, in_splits, group=group)
    blocks, at = [], 0
    for nq, n in zip(queries_per_rank, out_splits):
        blocks.append(recv[at:at + n].view(n_own, nq, width).transpose(0, 1))
        at += n
    return torch.cat(blocks, dim=0).contiguous()


class _ShardedContrastive(torch.autograd.Function):
    @staticmethod
    def forward(ctx, queries, documents, doc_lengths, group, ops, exchange, shard_sizes):
        rank, world = _world(group)
        q = queries.contiguous()
        d_local = documents.contiguous()
        lens_local = doc_lengths.to(torch.int32).contiguous()
        sizes = None
        if world == 1:
            docs_all, offsets, real, n_cols = d_local, offsets_from_lengths(lens_local), None, 0
            t_pad = d_local.shape[0]
        else:
            docs_all, offsets, real, n_cols, sizes, t_pad = _gather_shards(
                d_local, lens_local, group, world, n_queries=q.shape[0], shard_sizes=shard_sizes)
        scores_all, argmax = ops.maxsim_contrastive_forward_with_argmax(q, docs_all, offsets)
        ctx.save_for_backward(q, docs_all, offsets, argmax, d_local, lens_local)
        ctx.real, ctx.n_cols, ctx.sizes = real, n_cols, sizes
        ctx.group, ctx.ops, ctx.rank, ctx.world = group, ops, rank, world
        ctx.t_local, ctx.t_pad, ctx.exchange = d_local.shape[0], t_pad, exchange
        return scores_all if real is None else scores_all.index_select(1, real)

    @staticmethod
    def backward(ctx, dscore):
        q, docs_all, offsets, argmax, d_local, lens_local = ctx.saved_tensors
        ops, group, rank, world = ctx.ops, ctx.group, ctx.rank, ctx.world
        part = getattr(ops, "contrastive_backward_part", None)
        g = dscore.contiguous().to(torch.float32)
        if world == 1:
            dq, dd_all = ops.maxsim_contrastive_backward(g, q, docs_all, offsets, argmax)
            return dq, dd_all, None, None, None, None, None
        # filler documents receive no gradient
        g_all = torch.zeros((g.shape[0], ctx.n_cols), dtype=torch.float32, device=g.device)
        g_all.index_copy_(1, ctx.real, g)

        if ctx.exchange == "reduce_scatter":
            dq, dd_all = ops.maxsim_contrastive_backward(g_all, q, docs_all, offsets, argmax)
            mine = _reduce_scatter_rows(dd_all, world, rank, group)
            return dq, mine[: ctx.t_local].contiguous(), None, None, None, None, None

        # "owner": grad_queries is computed here, where the queries are.  For
        # grad_documents every rank sends each owner the argmax and the score
        # gradient of that owner's documents (one int32 record of Lq + 1 words
        # per pair) and the queries are all-gathered; each owner then computes
        # the gradient of its own documents from all queries.  This moves
        # 4 * (Lq + 1) bytes per pair instead of 4 * dim bytes per document
        # token per rank, and no partial sums.
        if part is not None:
            dq = part(g_all, q, docs_all, offsets, argmax, want_queries=True, want_documents=False)[0]
        else:
            dq = ops.maxsim_contrastive_backward(g_all, q, docs_all, offsets, argmax)[0]
        docs_per_rank = [s[1] for s in ctx.sizes]
        queries_per_rank = [s[2] for s in ctx.sizes]
        record = torch.cat([argmax.index_select(1, ctx.real).to(torch.int32),
                            g.view(torch.int32).unsqueeze(-1)], dim=2)      # [Nq_local, Nb_total, Lq + 1]
        mine = _columns_to_owners(record, docs_per_rank, queries_per_rank, rank, group)
        a_own = mine[:, :, :-1].contiguous()
        g_own = mine[:, :, -1].contiguous().view(torch.float32)
        q_all = _all_gather_rows(q, queries_per_rank, group, world)
        off_local = offsets_from_lengths(lens_local)
        if part is not None:
            dd = part(g_own, q_all, d_local, off_local, a_own, want_queries=False, want_documents=True)[1]
        else:
            dd = ops.maxsim_contrastive_backward(g_own, q_all, d_local, off_local, a_own)[1]
        return dq, dd, None, None, None, None, None


def score_contrastive_sharded(queries, documents, doc_lengths, *, group=None, ops=None,
                              exchange: str = "owner", shard_sizes=None):
    """Differentiable contrastive scores of this rank's queries against the
    documents of all ranks.

    Args:
        queries: ``[Nq_local, Lq, D]`` -- this rank's queries.
        documents: ``[T_local, D]`` packed -- this rank's documents.
        doc_lengths: ``[Nb_local]`` int -- their lengths (offsets are rebuilt
            per shard by cumulative sum).
    Returns:
        ``[Nq_local, Nb_total]`` fp32, document columns in rank order.  The
        gradient reaching ``documents`` is the sum over all ranks' queries.

    ``shard_sizes``, when given, is the list of every rank's ``(document
    tokens, documents, queries)`` in rank order (a data pipeline can exchange
    these numbers ahead of the step): the driver then neither exchanges them
    nor waits for the device, so the host keeps launching ahead of the GPU.

    ``exchange`` selects how the backward pass gets that sum to the owner:
    ``"owner"`` (default) sends each owner the argmax and score gradient of its
    documents and lets it compute the gradient from the all-gathered queries;
    ``"reduce_scatter"`` has every rank compute a partial gradient for all
    documents and reduce-scatters the partial sums.
    """
    if ops is None:
        ops = _default_ops()
    if doc_lengths.dim() != 1:
        raise ValueError(f"doc_lengths must be 1-D [Nb_local]; got shape {tuple(doc_lengths.shape)}")
    if int(doc_lengths.numel()) == 0:
        raise ValueError("every rank must own at least one document")
    if queries.dim() != 3 or documents.dim() != 2 or queries.shape[2] != documents.shape[1]:
        raise ValueError("queries must be [Nq, Lq, D] and documents [T, D] with matching D")
    if queries.dtype != documents.dtype:
        raise TypeError(f"queries and documents must share dtype; got {queries.dtype} and {documents.dtype}")
    if exchange not in ("owner", "reduce_scatter"):
        raise ValueError(f"exchange must be 'owner' or 'reduce_scatter'; got {exchange!r}")
    return _ShardedContrastive.apply(queries, documents, doc_lengths, group, ops, exchange, shard_sizes)


def contrastive_targets(n_queries_local: int, *, group=None, device=None,
                        docs_per_rank: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Column index of the positive document of each local query when query i
    of rank r is paired with document i of rank r (in-batch negatives)."""
    rank, world = _world(group)
    if docs_per_rank is None:
        if world == 1:
            start = 0
        else:
            raise ValueError("docs_per_rank is required when more than one rank takes part")
    else:
        start = int(sum(docs_per_rank[:rank]))
    return start + torch.arange(n_queries_local, device=device)
