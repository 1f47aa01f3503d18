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
    document shards are all-gathered (they are ragged, so each is padded to the
    longest shard for the collective and never compacted afterwards); the rank
    scores its queries against one source shard at a time, starting with its
    own shard while the gather is still in flight.  Backward: for every owner
    rank the partial ``grad_documents`` of that owner's shard is reduced to the
    owner as soon as the chunk is computed, overlapping with the next chunk;
    ``grad_queries`` stays local.  Scores come back as ``[Nq_local, Nb_total]``
    with document columns in rank order, so diagonal targets are
    ``rank_query_offset + arange(Nq_local)`` (:func:`score_contrastive_sharded`).

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
    from ._ops import ops
    return ops


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

def _gather_shards(documents: torch.Tensor, lengths: torch.Tensor, group, world: int):
    """All-gather ragged packed shards.  Returns (per-rank token buffers, per-
    rank int32 length vectors, async handle of the big gather or None)."""
    dev = documents.device
    meta = torch.tensor([documents.shape[0], lengths.numel()], dtype=torch.int64, device=dev)
    metas = [torch.zeros_like(meta) for _ in range(world)]
    dist.all_gather(metas, meta, group=group)
    sizes = [(int(m[0].item()), int(m[1].item())) for m in metas]
    t_max = max(s[0] for s in sizes)
    n_max = max(s[1] for s in sizes)

    len_pad = torch.zeros(n_max, dtype=torch.int32, device=dev)
    len_pad[: lengths.numel()] = lengths.to(torch.int32)
    len_parts = [torch.empty_like(len_pad) for _ in range(world)]
    dist.all_gather(len_parts, len_pad, group=group)

    doc_pad = documents.new_zeros((t_max, documents.shape[1]))
    doc_pad[: documents.shape[0]] = documents
    doc_parts = [torch.empty_like(doc_pad) for _ in range(world)]
    handle = dist.all_gather(doc_parts, doc_pad, group=group, async_op=True)
    shards = [(doc_parts[r], len_parts[r][: sizes[r][1]], sizes[r][0]) for r in range(world)]
    return shards, handle


class _ShardedContrastive(torch.autograd.Function):
    @staticmethod
    def forward(ctx, queries, documents, doc_lengths, group, ops):
        rank, world = _world(group)
        q = queries.contiguous()
        d_local = documents.contiguous()
        lens_local = doc_lengths.to(torch.int32).contiguous()
        if world == 1:
            shards = [(d_local, lens_local, d_local.shape[0])]
            handle = None
        else:
            shards, handle = _gather_shards(d_local, lens_local, group, world)

        order = [rank] + [r for r in range(world) if r != rank]  # own shard first
        cols: List[Optional[torch.Tensor]] = [None] * world
        saved = []
        for step, r in enumerate(order):
            if step == 1 and handle is not None:
                handle.wait()  # remote shards are needed from here on
            if r == rank:
                d_r, lens_r, t_r = d_local, lens_local, d_local.shape[0]
            else:
                buf, lens_r, t_r = shards[r]
                d_r = buf[:t_r]
            off_r = offsets_from_lengths(lens_r)
            s_r, a_r = ops.maxsim_contrastive_forward_with_argmax(q, d_r, off_r)
            cols[r] = s_r
            saved.append((r, d_r, off_r, a_r))
        ctx.saved_chunks = saved
        ctx.q = q
        ctx.group = group
        ctx.ops = ops
        ctx.rank, ctx.world = rank, world
        ctx.col_sizes = [c.shape[1] for c in cols]
        return torch.cat(cols, dim=1)

    @staticmethod
    def backward(ctx, dscore):
        ops, group, rank, world = ctx.ops, ctx.group, ctx.rank, ctx.world
        g = dscore.contiguous().to(torch.float32)
        starts = [0]
        for n in ctx.col_sizes:
            starts.append(starts[-1] + n)
        by_rank = {r: (d_r, off_r, a_r) for r, d_r, off_r, a_r in ctx.saved_chunks}
        dq_total = None
        dd_local = None
        pending = []
        # Collectives must be issued in the same order on every rank: owner 0, 1, ...
        for r in range(world):
            d_r, off_r, a_r = by_rank[r]
            g_r = g[:, starts[r]:starts[r + 1]].contiguous()
            dq_r, dd_r = ops.maxsim_contrastive_backward(g_r, ctx.q, d_r, off_r, a_r)
            dq_total = dq_r if dq_total is None else dq_total.add_(dq_r)
            if world > 1:
                pending.append(dist.reduce(dd_r, dst=dist.get_global_rank(group, r) if group else r,
                                           group=group, async_op=True))
            if r == rank:
                dd_local = dd_r
        for h in pending:
            h.wait()
        return dq_total, dd_local, None, None, None


def score_contrastive_sharded(queries, documents, doc_lengths, *, group=None, ops=None):
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
    return _ShardedContrastive.apply(queries, documents, doc_lengths, group, ops)


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
