"""Multi-GPU drivers: one process per GPU, ``torch.distributed`` for the plumbing.

The reference has no multi-device code at all; these two drivers sit *outside*
the operator boundary and only decide which rank scores what.

Rerank (padded / packed candidates)
    Pairs are independent, so queries -- with their candidate lists -- are
    split across ranks and each rank calls the ordinary operator on its shard.
    There is no collective on the data path (:func:`shard_range`,
    :func:`score_candidates_padded_sharded`).

Contrastive training
    Rank r owns ``Nq/R`` queries and ``Nb/R`` documents.

    Forward: the packed document shards (ragged) are gathered straight into
    one packed buffer ``[T_total, D]`` in rank order -- no padding rows, no
    compaction -- by one broadcast per owner, together with their lengths.
    While the transfers run, the rank's queries are scored against its OWN
    documents, then against every other shard as soon as it has landed.  All
    launches write into one ``[Nq_local, Nb_total]`` score matrix (document
    columns in rank order, so diagonal targets are ``rank_query_offset +
    arange``).

    Backward, ``exchange="owner"`` (default): ``grad_queries`` is computed
    where the queries are.  For ``grad_documents`` one kernel regroups the
    pairs' records -- the Lq winning tokens and the score gradient -- by
    owning rank, one all-to-all delivers every owner the records of its
    documents from all ranks (while ``grad_queries`` is being computed), the
    queries were all-gathered during the forward pass, and each owner computes
    the gradient of its own documents from all queries.  4 (Lq + 1) bytes per
    pair cross the links instead of 4 D bytes per document token per rank.

    ``exchange="reduce_scatter"``: every rank routes a partial
    ``grad_documents`` for the whole buffer and the sums are reduce-scattered.

    The transfers only overlap with the kernels if their own kernels find free
    SMs: forward launches that run beside a transfer leave ``COLLECTIVE_SMS``
    SMs unused; a process group created with
    ``opts = ProcessGroupNCCL.Options(is_high_priority_stream=True);
    opts.config.max_ctas = COLLECTIVE_SMS`` keeps its collectives within them.

    ``peer=`` (a :class:`maxsim_b200.peer.PeerExchange`) replaces the
    collectives by the node's peer-mapped memory: shards are fetched by the
    copy engines out of the owners' buffers while forward launches keep every
    SM, the regrouping kernel stores each owner's records into that owner's
    memory, and one small barrier kernel per pass orders the two.

Both drivers take the operator namespace as a parameter so that their
sharding / reassembly logic can be exercised on CPU ``gloo`` ranks with a
stand-in scorer; the default is the CUDA library, whose extra entry points
(column blocks of a score matrix, record packing, gradients from records) are
used when the namespace has them.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = [
    "shard_range", "score_candidates_padded_sharded", "score_contrastive_sharded",
    "contrastive_targets", "offsets_from_lengths", "fetch_schedule",
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
    return types.SimpleNamespace(
        **vars(_ops.ops),
        contrastive_backward_part=_ops.contrastive_backward_part,
        contrastive_backward_native=_ops.contrastive_backward_native,
        contrastive_forward_block=_ops.contrastive_forward_block,
        pack_owner_records=_ops.pack_owner_records,
        contrastive_backward_documents_from_records=_ops.contrastive_backward_documents_from_records,
        offsets_from_lengths=lambda lengths: _ops.offsets_from_lengths(lengths, 2 ** 31 - 1)[0])


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

# SMs a forward launch leaves to the kernels of the transfers that run beside it.  A process
# group whose collectives use more CTAs than this (ProcessGroupNCCL.Options().config.max_ctas)
# still makes progress, with the CTAs that found room.
COLLECTIVE_SMS = 8

_INT_TABLES = {}


def _device_ints(values: Sequence[int], device) -> torch.Tensor:
    """A small int32 table on ``device``.  Tables are kept: a training loop asks
    for the same shard boundaries every step, and a host-to-device copy from
    pageable memory makes the host wait for the stream."""
    key = (str(device), tuple(values))
    table = _INT_TABLES.get(key)
    if table is None:
        if len(_INT_TABLES) > 64:
            _INT_TABLES.clear()
        table = torch.tensor(list(values), dtype=torch.int32, device=device)
        _INT_TABLES[key] = table
    return table


class _Done:
    """Stands in for the handle of an exchange that has already completed."""

    def wait(self):
        return True


class _AfterBarrier:
    """Handle of an exchange made of stores to peer memory: it is complete on
    every rank once the group's barrier has been passed on the stream."""

    def __init__(self, peer):
        self.peer = peer

    def wait(self):
        self.peer.barrier()
        return True


def _exchange_sizes(documents, lengths, n_queries, group, world, shard_sizes):
    """Every rank's ``(document tokens, documents, queries)`` in rank order."""
    if shard_sizes is not None:
        # the caller already knows them: no exchange and, above all, no wait for
        # the device on the host
        sizes = [(int(t), int(n), int(nq)) for t, n, nq in shard_sizes]
        rank = dist.get_rank(group)
        mine = (documents.shape[0], lengths.numel(), n_queries)
        if len(sizes) != world or sizes[rank] != mine:
            raise ValueError(f"shard_sizes[{rank}] = {sizes[rank] if len(sizes) == world else None} does not "
                             f"describe this rank's shard {mine}")
        return sizes
    dev = documents.device
    meta = torch.tensor([documents.shape[0], lengths.numel(), n_queries], dtype=torch.int64, device=dev)
    metas = torch.empty((world, 3), dtype=torch.int64, device=dev)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(metas, meta, group=group)
    else:
        dist.all_gather(list(metas.unbind(0)), meta, group=group)
    return [(int(t), int(n), int(nq)) for t, n, nq in metas.tolist()]  # one transfer for all ranks


def _all_gather_rows(out: torch.Tensor, local: torch.Tensor, counts: Sequence[int], group, rank: int):
    """Start gathering every rank's ``local [counts[r], ...]`` into ``out
    [sum(counts), ...]`` in rank order; returns a handle to ``wait()`` on.  The
    pieces land in place: ragged shards need neither padding nor compaction."""
    views = list(out.split(list(counts), dim=0))
    local = local.contiguous()
    if dist.get_backend(group) == "nccl":
        if all(c == counts[0] for c in counts):
            return dist.all_gather_into_tensor(out, local, group=group, async_op=True)
        return dist.all_gather(views, local, group=group, async_op=True)  # uneven pieces are supported
    if all(c == counts[0] for c in counts):
        return dist.all_gather(views, local, group=group, async_op=True)
    # backends whose all-gather wants equal pieces: one broadcast per rank
    world = len(counts)
    for r in range(world):
        if r == rank:
            views[r].copy_(local)
        if counts[r]:
            dist.broadcast(views[r], src=dist.get_global_rank(group, r) if group is not None else r,
                           group=group)
    return _Done()


def _broadcast_rows(out: torch.Tensor, local: torch.Tensor, counts: Sequence[int], group, rank: int):
    """Gather every rank's ``local [counts[r], ...]`` into ``out [sum(counts),
    ...]`` in rank order as one broadcast per rank, issued in rank order on
    every rank; returns the handles in rank order, so that a consumer can wait
    for one piece at a time.  The own piece is copied."""
    views = list(out.split(list(counts), dim=0))
    local = local.contiguous()
    handles = []
    for r in range(len(counts)):
        src = dist.get_global_rank(group, r) if group is not None else r
        if counts[r] == 0:
            handles.append(_Done())
        elif r == rank:
            handles.append(dist.broadcast(local, src=src, group=group, async_op=True))
            views[r].copy_(local)
        else:
            handles.append(dist.broadcast(views[r], src=src, group=group, async_op=True))
    return handles


def _reduce_scatter_rows(full: torch.Tensor, counts: Sequence[int], rank: int, group) -> torch.Tensor:
    """Sum ``full [sum(counts), D]`` over the ranks and return this rank's rows
    ``[counts[rank], D]``.  NCCL reduce-scatters (ragged shards through a padded
    copy); backends without a reduce-scatter (gloo, used by the CPU tests)
    all-reduce and slice."""
    world = len(counts)
    begin = sum(counts[:rank])
    if dist.get_backend(group) != "nccl":
        dist.all_reduce(full, group=group)
        return full[begin:begin + counts[rank]].contiguous()
    t_max = max(counts)
    if all(c == t_max for c in counts):
        src = full
    else:
        src = full.new_zeros((world * t_max, full.shape[1]))
        for r, piece in enumerate(full.split(list(counts), dim=0)):
            src[r * t_max:r * t_max + counts[r]].copy_(piece)
    out = torch.empty((t_max, full.shape[1]), dtype=full.dtype, device=full.device)
    dist.reduce_scatter_tensor(out, src, group=group)
    return out[:counts[rank]].contiguous() if counts[rank] != t_max else out


def _offsets(ops, lengths: torch.Tensor) -> torch.Tensor:
    fn = getattr(ops, "offsets_from_lengths", None)
    return fn(lengths) if fn is not None and lengths.is_cuda else offsets_from_lengths(lengths)


def fetch_schedule(rank: int, tokens: Sequence[int], n_queries_local: int, lq: int, dim: int,
                   itemsize: int) -> List[Tuple[int, int]]:
    """Which fetched shards a rank scores with which launch, for the peer
    transport: contiguous rank ranges ``(first, last)`` in the order the shards
    are fetched (the ranks after ``rank``, then those before it).

    Every launch pays a ramp-up and a tail, so few launches are better -- as
    long as none waits for its data.  The shards arrive one after the other
    while the rank's own block and then the earlier ranges are being scored;
    the schedule is what a greedy consumer would do: each launch takes every
    shard that has landed by the time the previous launch ends (at least one).
    With shards that arrive faster than they are scored (4 GPUs on config 5:
    30 us against 185 us) that is one launch for everything fetched; with
    many small shards (8 GPUs: the seven copies take 180 us, a block 45 us)
    it is a short first launch followed by longer ones.  The rates are the
    measured ones of this library on a B200 (copy-engine fetch over NVLink,
    forward with argmax); they only steer the grouping."""
    world = len(tokens)
    order = [(rank + k) % world for k in range(1, world)]
    copy_rate, copy_latency = 4.0e11, 2.0e-6        # bytes/s per fetch, s per copy
    score_rate, launch_cost = 1.0e15, 12.0e-6       # flop/s of forward + argmax, s per launch
    per_token = 2.0 * n_queries_local * lq * dim / score_rate
    landed, t = [], 0.0
    for r in order:
        t += tokens[r] * dim * itemsize / copy_rate + copy_latency
        landed.append(t)
    now = tokens[rank] * per_token + launch_cost   # the own block ends
    groups, k = [], 0
    while k < len(order):
        n = max(1, sum(1 for x in landed[k:] if x <= now))
        group = order[k:k + n]
        now = max(now, landed[k + n - 1]) + sum(tokens[r] for r in group) * per_token + launch_cost
        groups.append(group)
        k += n
    ranges = []
    for group in groups:  # a group that wraps around the last rank is two column ranges
        first = prev = group[0]
        for r in group[1:]:
            if r != prev + 1:
                ranges.append((first, prev + 1))
                first = r
            prev = r
        ranges.append((first, prev + 1))
    return ranges


class _ShardedContrastive(torch.autograd.Function):
    @staticmethod
    def forward(ctx, queries, documents, doc_lengths, group, ops, exchange, shard_sizes, records_group,
                peer=None):
        rank, world = _world(group)
        q = queries.contiguous()
        d_local = documents.contiguous()
        lens_local = doc_lengths.to(torch.int32).contiguous()
        ctx.group, ctx.ops, ctx.rank, ctx.world, ctx.exchange = group, ops, rank, world, exchange
        ctx.records_group = records_group if records_group is not None else group
        if world == 1:
            offsets = _offsets(ops, lens_local)
            scores, argmax = ops.maxsim_contrastive_forward_with_argmax(q, d_local, offsets)
            ctx.save_for_backward(q, d_local, offsets, argmax)
            return scores
        dev = q.device
        sizes = _exchange_sizes(d_local, lens_local, q.shape[0], group, world, shard_sizes)
        tokens = [s[0] for s in sizes]
        n_docs = [s[1] for s in sizes]
        n_queries = [s[2] for s in sizes]
        col0 = [sum(n_docs[:r]) for r in range(world + 1)]
        nb_total, t_total = col0[-1], sum(tokens)
        ctx.peer, ctx.sizes = peer, sizes
        if peer is not None:
            return _ShardedContrastive._forward_peer(ctx, q, d_local, lens_local, ops, peer, sizes, col0)

        # start the exchanges: the documents' lengths, the documents themselves -- one
        # broadcast per owner, so that every shard can be scored as soon as it has landed --
        # and (for the owner exchange of the backward pass) the queries
        docs_all = torch.empty((t_total, d_local.shape[1]), dtype=d_local.dtype, device=dev)
        lens_all = torch.empty((nb_total,), dtype=torch.int32, device=dev)
        h_lens = _all_gather_rows(lens_all, lens_local, n_docs, group, rank)
        h_docs = _broadcast_rows(docs_all, d_local, tokens, group, rank)
        q_all, h_q = None, None
        if exchange == "owner":
            q_all = torch.empty((sum(n_queries),) + tuple(q.shape[1:]), dtype=q.dtype, device=dev)
            h_q = _all_gather_rows(q_all, q, n_queries, group, rank)

        # This rank's own documents are scored while the exchange runs, then every other
        # rank's shard as it arrives.  The forward kernel is persistent: it leaves a few SMs
        # unused while transfers are still under way, or their kernels would only start
        # when it ends.
        block = getattr(ops, "contrastive_forward_block", None)
        off_local = _offsets(ops, lens_local)
        scores = argmax = None
        if block is not None and q.is_cuda:
            scores = torch.empty((q.shape[0], nb_total), dtype=torch.float32, device=dev)
            argmax = torch.empty((q.shape[0], nb_total, q.shape[1]), dtype=torch.int32, device=dev)
            if not block(q, d_local, off_local, scores, argmax, col0[rank], tokens[rank],
                         reserve_sms=COLLECTIVE_SMS):
                scores = argmax = None  # shape outside the kernel: one ordinary call below
        h_lens.wait()
        offsets = _offsets(ops, lens_all)
        others = [r for r in range(world) if r != rank and n_docs[r] > 0]
        if scores is None:
            for h in h_docs:
                h.wait()
            scores, argmax = ops.maxsim_contrastive_forward_with_argmax(q, docs_all, offsets)
        else:
            for k, r in enumerate(others):
                h_docs[r].wait()
                last = k + 1 == len(others)
                block(q, docs_all, offsets[col0[r]:col0[r + 1] + 1], scores, argmax, col0[r], tokens[r],
                      reserve_sms=0 if last else COLLECTIVE_SMS)
            for h in h_docs:
                h.wait()  # (shards without documents)
        ctx.save_for_backward(q, docs_all, offsets, argmax, d_local, off_local)
        ctx.q_all, ctx.h_q = q_all, h_q
        ctx.tokens, ctx.n_docs, ctx.n_queries, ctx.col0 = tokens, n_docs, n_queries, col0
        return scores

    @staticmethod
    def _forward_peer(ctx, q, d_local, lens_local, ops, peer, sizes, col0):
        """The forward pass over peer-mapped buffers (maxsim_b200.peer): no
        collective; copies by the copy engines beside forward launches that keep
        every SM."""
        rank, world = ctx.rank, ctx.world
        dev = q.device
        tokens = [s[0] for s in sizes]
        n_docs = [s[1] for s in sizes]
        n_queries = [s[2] for s in sizes]
        peer.check_fits(sizes, q.shape[1], q.shape[2], q.dtype)
        docs_all = torch.empty((sum(tokens), d_local.shape[1]), dtype=d_local.dtype, device=dev)
        lens_all = torch.empty((col0[-1],), dtype=torch.int32, device=dev)
        q_all = torch.empty((sum(n_queries),) + tuple(q.shape[1:]), dtype=q.dtype, device=dev)
        ranges = fetch_schedule(rank, tokens, q.shape[0], q.shape[1], q.shape[2], q.element_size())
        landed, everything = peer.gather(d_local, lens_local, q, sizes, docs_all, lens_all, q_all, ranges)
        off_local = _offsets(ops, lens_local)
        offsets = _offsets(ops, lens_all)
        scores = torch.empty((q.shape[0], col0[-1]), dtype=torch.float32, device=dev)
        argmax = torch.empty((q.shape[0], col0[-1], q.shape[1]), dtype=torch.int32, device=dev)
        blocks = ops.contrastive_forward_block(q, d_local, off_local, scores, argmax, col0[rank],
                                               tokens[rank])
        if blocks:
            # every range of fetched shards is a contiguous range of columns and gets one
            # launch, as soon as its last shard has landed (see fetch_schedule)
            for (first, last), handle in zip(ranges, landed):
                handle.wait()
                if col0[last] == col0[first]:
                    continue
                ops.contrastive_forward_block(q, docs_all, offsets[col0[first]:col0[last] + 1], scores,
                                              argmax, col0[first], sum(tokens[first:last]))
            everything.wait()  # every read of a peer's buffers is ordered before what follows
        else:  # shape outside the block kernel: one ordinary call over all shards
            everything.wait()
            scores, argmax = ops.maxsim_contrastive_forward_with_argmax(q, docs_all, offsets)
        ctx.save_for_backward(q, docs_all, offsets, argmax, d_local, off_local)
        ctx.q_all, ctx.h_q = q_all, _Done()
        ctx.tokens, ctx.n_docs, ctx.n_queries, ctx.col0 = tokens, n_docs, n_queries, col0
        return scores

    @staticmethod
    def backward(ctx, dscore):
        ops, group, rank, world = ctx.ops, ctx.group, ctx.rank, ctx.world
        g = dscore.contiguous().to(torch.float32)
        no_grad = (None,) * 7
        if world == 1:
            q, d_local, offsets, argmax = ctx.saved_tensors
            dq, dd = ops.maxsim_contrastive_backward(g, q, d_local, offsets, argmax)
            return (dq, dd) + no_grad
        q, docs_all, offsets, argmax, d_local, off_local = ctx.saved_tensors
        if ctx.exchange == "reduce_scatter":
            dq, dd_all = ops.maxsim_contrastive_backward(g, q, docs_all, offsets, argmax)
            return (dq, _reduce_scatter_rows(dd_all, ctx.tokens, rank, group)) + no_grad

        # "owner".  The records of this rank's pairs go to the owners of the documents ...
        n_docs, n_queries, col0 = ctx.n_docs, ctx.n_queries, ctx.col0
        nq_local, lq = q.shape[0], q.shape[1]
        pack = getattr(ops, "pack_owner_records", None)
        width = lq + 1
        peer = getattr(ctx, "peer", None)
        if peer is not None:
            # the regrouping kernel stores each owner's block in that owner's memory
            recv = peer.send_records(argmax, g, _device_ints(col0, g.device), ctx.sizes)
            h_rec = _AfterBarrier(peer)
        else:
            if pack is not None and g.is_cuda:
                send = pack(argmax, g, _device_ints(col0, g.device))
            else:
                record = torch.cat([argmax.to(torch.int32), g.view(torch.int32).unsqueeze(-1)], dim=2)
                send = torch.cat([record[:, col0[o]:col0[o + 1]].reshape(-1) for o in range(world)])
            in_splits = [n * nq_local * width for n in n_docs]
            out_splits = [n_docs[rank] * nq * width for nq in n_queries]
            recv = torch.empty((sum(out_splits),), dtype=torch.int32, device=g.device)
            h_rec = dist.all_to_all_single(recv, send, out_splits, in_splits, group=ctx.records_group,
                                           async_op=True)

        # ... while grad_queries is computed here, where the queries are
        native = getattr(ops, "contrastive_backward_native", None)
        part = getattr(ops, "contrastive_backward_part", None)
        dq = None
        if native is not None:
            got = native(g, q, docs_all, offsets, argmax, want_documents=False)
            dq = got[0] if got is not None else None
        if dq is None and part is not None:
            dq = part(g, q, docs_all, offsets, argmax, want_queries=True, want_documents=False)[0]
        if dq is None:
            dq = ops.maxsim_contrastive_backward(g, q, docs_all, offsets, argmax)[0]

        # every owner now holds [all queries, own documents, Lq + 1] and all queries
        h_rec.wait()
        ctx.h_q.wait()
        q_all = ctx.q_all
        from_records = getattr(ops, "contrastive_backward_documents_from_records", None)
        dd = from_records(recv, q_all, d_local, off_local) if from_records is not None and g.is_cuda else None
        if dd is None:
            rec = recv.view(q_all.shape[0], n_docs[rank], width)
            a_own = rec[:, :, :lq].contiguous()
            g_own = rec[:, :, lq].contiguous().view(torch.float32)
            if part is not None:
                dd = part(g_own, q_all, d_local, off_local, a_own, want_queries=False, want_documents=True)[1]
            else:
                dd = ops.maxsim_contrastive_backward(g_own, q_all, d_local, off_local, a_own)[1]
        return (dq, dd) + no_grad


def score_contrastive_sharded(queries, documents, doc_lengths, *, group=None, ops=None,
                              exchange: str = "owner", shard_sizes=None, records_group=None, peer=None):
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

    ``records_group``, when given, is a second process group over the same
    ranks that carries the all-to-all of the backward pass.  The forward
    transfers run beside kernels and want a group limited to a few CTAs (see
    the module text); the all-to-all has little to run beside and is fastest
    on a group with NCCL's default CTA count.

    ``peer``, when given, is a :class:`maxsim_b200.peer.PeerExchange` built
    for this group: the shards then travel as copies out of peer-mapped
    buffers (copy engines; the forward launches keep every SM) and the argmax
    records as stores of the regrouping kernel into the owners' memory, with
    one barrier kernel per pass instead of collectives.  Needs
    ``shard_sizes`` and ``exchange="owner"``.

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
    if peer is not None:
        if exchange != "owner" or shard_sizes is None:
            raise ValueError("the peer transport needs exchange='owner' and shard_sizes")
        if not hasattr(ops, "contrastive_forward_block"):
            raise ValueError("the peer transport needs the CUDA library's operators")
    return _ShardedContrastive.apply(queries, documents, doc_lengths, group, ops, exchange, shard_sizes,
                                     records_group, peer)


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
