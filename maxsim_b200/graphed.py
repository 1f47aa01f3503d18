"""A contrastive training step captured once in a CUDA graph and replayed.

At the batch sizes the reference publishes (32 to 64 queries and documents,
``README.md:405-442``) a contrastive train step is a few tens of microseconds
of GPU work behind a few hundred microseconds of Python, autograd and launch
overhead; the reference's own figures (0.26-0.32 ms on an H200) are that
overhead.  Replaying the step from a graph removes it.

A graph needs static shapes, and packed documents change their token count
from batch to batch.  :class:`GraphedContrastiveStep` therefore owns a
document buffer of a fixed token capacity; the rows a batch does not use are
described to the kernels as one extra "filler" document whose score column is
dropped before the loss, so the offsets -- device data the kernels read at run
time -- are the only thing that changes between replays.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

__all__ = ["GraphedContrastiveStep", "GraphedShardedContrastiveStep"]


class GraphedContrastiveStep:
    """In-batch contrastive loss and its gradients for batches of a fixed
    ``(n_queries, q_len, n_documents, dim)`` and at most ``token_capacity - 1``
    document tokens.

    ``step(queries, documents, document_offsets, targets=None)`` copies the
    batch into the static buffers, replays the graph and returns
    ``(loss, grad_queries, grad_documents)``: the mean cross-entropy of
    ``score_contrastive(q, d, off) / temperature`` against ``targets``
    (default: query i's positive is document i) and its gradients in the
    inputs' dtype.  The returned tensors are views of static buffers: they are
    overwritten by the next ``step``.
    """

    def __init__(self, n_queries: int, q_len: int, n_documents: int, dim: int, token_capacity: int,
                 *, dtype=torch.bfloat16, device="cuda", temperature: float = 1.0):
        import maxsim_b200 as maxsim

        if min(n_queries, q_len, n_documents, dim) <= 0 or token_capacity < n_documents + 1:
            raise ValueError("sizes must be positive and token_capacity > n_documents")
        if not temperature > 0:
            raise ValueError(f"temperature must be > 0; got {temperature}")
        self.device = torch.device(device)
        self.n_queries, self.n_documents, self.capacity = n_queries, n_documents, int(token_capacity)
        self.temperature = float(temperature)
        dev = self.device
        self._q = torch.zeros((n_queries, q_len, dim), dtype=dtype, device=dev, requires_grad=True)
        self._d = torch.zeros((self.capacity, dim), dtype=dtype, device=dev, requires_grad=True)
        # n_documents real documents of one token each, then the filler
        off = list(range(n_documents + 1)) + [self.capacity]
        self._off = torch.tensor(off, dtype=torch.int32, device=dev)
        self._targets = (torch.arange(n_queries, device=dev) % n_documents).to(torch.int64)

        def body():
            scores = maxsim.score_contrastive_train(self._q, self._d, self._off)[:, :n_documents]
            loss = torch.nn.functional.cross_entropy(scores / self.temperature, self._targets)
            gq, gd = torch.autograd.grad(loss, (self._q, self._d))
            return loss, gq, gd

        # warm up on a side stream (this also validates the offsets tensor once, so
        # nothing synchronises during capture), then capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                body()
        torch.cuda.current_stream(dev).wait_stream(side)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._loss, self._gq, self._gd = body()

    def step(self, queries: torch.Tensor, documents: torch.Tensor, document_offsets: torch.Tensor,
             targets: Optional[torch.Tensor] = None
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        T = documents.shape[0]
        if tuple(queries.shape) != tuple(self._q.shape):
            raise ValueError(f"queries must have shape {tuple(self._q.shape)}; got {tuple(queries.shape)}")
        if documents.dim() != 2 or documents.shape[1] != self._d.shape[1] or not 0 < T < self.capacity:
            raise ValueError(f"documents must be [T, {self._d.shape[1]}] with 0 < T < {self.capacity}; "
                             f"got {tuple(documents.shape)}")
        if document_offsets.numel() != self.n_documents + 1:
            raise ValueError(f"document_offsets must have {self.n_documents + 1} elements")
        if document_offsets.device.type == "cpu":
            # offsets on the host cost nothing to check; device offsets are the caller's
            # contract (first 0, strictly increasing, last == T), as for the C ABI
            off = document_offsets.to(torch.int64)
            if int(off[0]) != 0 or int(off[-1]) != T or bool((off[1:] <= off[:-1]).any()):
                raise ValueError("document_offsets must start at 0, increase strictly and end at "
                                 f"the token count {T}")
        with torch.no_grad():
            self._q.copy_(queries, non_blocking=True)
            self._d[:T].copy_(documents, non_blocking=True)
            self._off[: self.n_documents + 1].copy_(document_offsets, non_blocking=True)
            if targets is not None:
                self._targets.copy_(targets, non_blocking=True)
        self._graph.replay()
        return self._loss, self._gq, self._gd[:T]


class GraphedShardedContrastiveStep:
    """The sharded contrastive train step (``maxsim_b200.dist``) over
    peer-mapped buffers, captured in CUDA graphs and replayed.

    With the problem split over the GPUs of a node each rank's share of a step
    is a few hundred microseconds of kernels, the same order as the Python,
    autograd and launch work that enqueues it; the slowest host then sets the
    pace of all ranks (they meet at two barriers per step).  The peer transport
    consists of kernels, copies and events only, so the whole step -- publish,
    barrier, fetches on the side streams, forward launches, loss, record
    stores, barrier, both gradients -- can be captured and replayed with one
    host call.  The barrier counts its epochs on the device, and the exchange
    buffers alternate between two slots, so two graphs are captured (one per
    slot) and replayed in turn.

    Every rank builds the object with the same ``shard_sizes`` (list of every
    rank's ``(document tokens, documents, queries)``), which are fixed for its
    lifetime (batches packed to a fixed token count per rank; a rank with fewer
    tokens pads its last document).  ``step(queries, documents, doc_lengths)``
    copies this rank's shard into static buffers, replays, and returns ``(loss,
    grad_queries, grad_documents)``: this rank's part of the global mean
    cross-entropy of ``scores / temperature`` against in-batch targets (query i
    of rank r is paired with document i of rank r) and the gradients of the
    global loss with respect to this rank's shard.  The returned tensors are
    static buffers, overwritten two steps later.  All ranks must call ``step``
    the same number of times.
    """

    def __init__(self, peer, shard_sizes, *, temperature: float = 1.0):
        from . import dist as mdist

        if not temperature > 0:
            raise ValueError(f"temperature must be > 0; got {temperature}")
        self.peer = peer
        self.sizes = [(int(t), int(n), int(nq)) for t, n, nq in shard_sizes]
        peer.check_fits(self.sizes, peer.lq, peer.dim, peer.dtype)
        rank, dev = peer.rank, peer.device
        tokens, n_docs, n_queries = self.sizes[rank]
        self.temperature = float(temperature)
        n_total = sum(s[2] for s in self.sizes)
        self._q = torch.zeros((n_queries, peer.lq, peer.dim), dtype=peer.dtype, device=dev, requires_grad=True)
        self._d = torch.zeros((tokens, peer.dim), dtype=peer.dtype, device=dev, requires_grad=True)
        # one token per document and the rest in the last one: valid lengths until the first step
        lens = [1] * n_docs
        lens[-1] = tokens - (n_docs - 1)
        self._lens = torch.tensor(lens, dtype=torch.int32, device=dev)
        self._targets = mdist.contrastive_targets(n_queries, group=peer.group, device=dev,
                                                  docs_per_rank=[s[1] for s in self.sizes])

        def body():
            scores = mdist.score_contrastive_sharded(self._q, self._d, self._lens, group=peer.group,
                                                     shard_sizes=self.sizes, peer=peer)
            loss = torch.nn.functional.cross_entropy(scores / self.temperature, self._targets,
                                                     reduction="sum") / n_total
            gq, gd = torch.autograd.grad(loss, (self._q, self._d))
            return loss, gq, gd

        # Warm up on a side stream: an even number of steps, so that the capture of the first
        # graph meets slot 0 again, and every table the step needs exists before capture.
        with torch.cuda.device(dev):
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    body()
            torch.cuda.current_stream(dev).wait_stream(side)
            self._graphs, self._outs = [], []
            for _ in range(2):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out = body()
                self._graphs.append(graph)
                self._outs.append(out)
        self._k = 0

    def step(self, queries: torch.Tensor, documents: torch.Tensor, doc_lengths: torch.Tensor
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if tuple(queries.shape) != tuple(self._q.shape) or tuple(documents.shape) != tuple(self._d.shape):
            raise ValueError(f"this rank's shard must be queries {tuple(self._q.shape)} and documents "
                             f"{tuple(self._d.shape)}; got {tuple(queries.shape)} and {tuple(documents.shape)}")
        if doc_lengths.numel() != self._lens.numel():
            raise ValueError(f"doc_lengths must have {self._lens.numel()} elements")
        with torch.no_grad():
            self._q.copy_(queries, non_blocking=True)
            self._d.copy_(documents, non_blocking=True)
            self._lens.copy_(doc_lengths, non_blocking=True)
        k = self._k & 1
        self._k += 1
        self._graphs[k].replay()
        return self._outs[k]
