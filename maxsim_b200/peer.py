"""Exchange buffers of the sharded contrastive step in peer-mapped memory.

The GPUs of one node can map each other's memory (NVLink / NVSwitch).  A
:class:`PeerExchange` owns one such allocation per rank, laid out identically
on all ranks, and gives :func:`maxsim_b200.dist.score_contrastive_sharded` a
transport that needs no collective library on the data path:

* forward: every rank *publishes* its document shard, lengths and queries in
  its own buffer, a barrier kernel follows, and every rank *fetches* the other
  shards with plain device-to-device copies on side streams -- copy engines,
  no SM is taken from the forward kernel, one event per shard so that each
  shard is scored as soon as it has landed;
* backward: the kernel that regroups the argmax records by owner stores each
  owner's block straight into that owner's buffer; a second barrier tells the
  owners their records are complete.

Buffers that a peer reads or writes exist twice and alternate from step to
step, so that one barrier per phase is enough: a rank can only reach the
barrier of step n + 1 after its own reads of step n, hence nobody overwrites
a slot that is still being read.

The allocation and the mapping come from ``torch.distributed._symmetric_memory``
(CUDA virtual-memory handles exchanged between the processes of the group); the
barrier and the record stores are this library's kernels
(``maxsim_b200_peer_barrier``, ``maxsim_b200_pack_owner_records_to``).  The
memory is not bound to a multicast object (``TORCH_SYMM_MEM_DISABLE_MULTICAST``
is set before the first allocation unless the caller has set it).
"""

from __future__ import annotations

import os
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _ops

__all__ = ["PeerExchange"]


def _round_up(n: int, to: int = 256) -> int:
    return (n + to - 1) // to * to


class PeerExchange:
    """Peer-mapped exchange buffers for one process group (one node).

    Args:
        group: the process group (``None``: the default group); every rank
            constructs the object with the same arguments (collective).
        max_doc_tokens, max_docs, max_queries: the largest document shard
            (tokens, documents) and query shard any rank will bring.
        lq, dim, dtype: query tokens per query, embedding width, element type.
        wait_polls: polls a barrier waits for each peer before it gives up and
            sets the status bit (0: the library's default, about ten seconds).
    """

    def __init__(self, group=None, *, max_doc_tokens: int, max_docs: int, max_queries: int,
                 lq: int, dim: int, dtype: torch.dtype, device=None, wait_polls: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.lq, self.dim, self.dtype = int(lq), int(dim), dtype
        self.max_doc_tokens, self.max_docs, self.max_queries = int(max_doc_tokens), int(max_docs), int(max_queries)
        self.wait_polls = int(wait_polls)
        item = torch.empty((), dtype=dtype).element_size()
        self._item = item

        # layout, in bytes (every region starts on a 256-byte boundary)
        cursor = 0

        def region(nbytes: int) -> int:
            nonlocal cursor
            at = cursor
            cursor = _round_up(cursor + max(nbytes, 4))
            return at

        self._flags_at = region(4 * self.world)
        self._docs_at = [region(self.max_doc_tokens * self.dim * item) for _ in range(2)]
        self._q_at = [region(self.max_queries * self.lq * self.dim * item) for _ in range(2)]
        self._lens_at = [region(4 * self.max_docs) for _ in range(2)]
        rec_words = self.world * self.max_queries * self.max_docs * (self.lq + 1)
        self._rec_at = [region(4 * rec_words) for _ in range(2)]
        self.nbytes = cursor

        with torch.cuda.device(self.device):
            self._buf = symm_mem.empty(self.nbytes // 4, dtype=torch.int32, device=self.device)
            self._buf.zero_()
            torch.cuda.synchronize()
            self._handle = symm_mem.rendezvous(self._buf, self.group)
            dist.barrier(self.group)  # every rank's flags are zero before anyone signals
            bases = [int(p) for p in self._handle.buffer_ptrs]
            self._bases = bases
            self._flags = torch.tensor([b + self._flags_at for b in bases], dtype=torch.int64, device=self.device)
            self._fetch_small = torch.cuda.Stream(self.device)
            self._fetch_docs = torch.cuda.Stream(self.device)
        self._epoch = 0
        self._fwd_steps = 0
        self._bwd_steps = 0
        self._tables = {}

    # -- views ---------------------------------------------------------------

    def _view(self, rank: int, at: int, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        size = torch.empty((), dtype=dtype).element_size()
        return self._handle.get_buffer(rank, tuple(shape), dtype, at // size)

    def check_fits(self, sizes: Sequence[Tuple[int, int, int]], lq: int, dim: int, dtype) -> None:
        if len(sizes) != self.world:
            raise ValueError(f"shard_sizes describes {len(sizes)} ranks, the exchange has {self.world}")
        if (lq, dim, dtype) != (self.lq, self.dim, self.dtype):
            raise ValueError(f"the exchange was built for Lq={self.lq}, D={self.dim}, {self.dtype}; "
                             f"got Lq={lq}, D={dim}, {dtype}")
        for r, (t, n, nq) in enumerate(sizes):
            if t > self.max_doc_tokens or n > self.max_docs or nq > self.max_queries:
                raise ValueError(f"rank {r}'s shard ({t} tokens, {n} documents, {nq} queries) exceeds the "
                                 f"exchange's capacity ({self.max_doc_tokens}, {self.max_docs}, {self.max_queries})")

    # -- synchronisation -----------------------------------------------------

    def barrier(self) -> None:
        """Stream-ordered barrier of the group on the current stream."""
        self._epoch += 1
        _ops.peer_barrier(self._flags, self.rank, self.world, self._epoch, self.wait_polls)

    # -- forward -------------------------------------------------------------

    def gather(self, documents, lengths, queries, sizes, docs_all, lens_all, q_all):
        """Publish this rank's shard and start fetching all others into the
        rank-ordered ``docs_all [T_total, D]``, ``lens_all [Nb_total]`` and
        ``q_all [Nq_total, Lq, D]``.  Returns ``(lens_event, doc_events, q_event,
        order)``: ``lens_event`` fires when all lengths are there,
        ``doc_events[r]`` when rank r's documents have landed, ``q_event`` when
        everything has (all queries and this rank's own rows of ``docs_all``
        included); ``order`` lists the other ranks in the order their documents
        are fetched.  The caller's tensors must stay untouched until
        ``q_event`` has been waited for."""
        rank, world = self.rank, self.world
        tokens = [s[0] for s in sizes]
        n_docs = [s[1] for s in sizes]
        n_queries = [s[2] for s in sizes]
        slot = self._fwd_steps & 1
        self._fwd_steps += 1
        main = torch.cuda.current_stream(self.device)

        self._view(rank, self._docs_at[slot], (tokens[rank], self.dim), self.dtype).copy_(documents)
        self._view(rank, self._lens_at[slot], (n_docs[rank],), torch.int32).copy_(lengths)
        self._view(rank, self._q_at[slot], (n_queries[rank], self.lq, self.dim), self.dtype).copy_(queries)
        self.barrier()
        ready = torch.cuda.Event()
        ready.record(main)

        d_views = list(docs_all.split(tokens, dim=0))
        l_views = list(lens_all.split(n_docs, dim=0))
        q_views = list(q_all.split(n_queries, dim=0))

        order = [(rank + k) % world for k in range(1, world)]
        with torch.cuda.stream(self._fetch_small):
            self._fetch_small.wait_event(ready)
            l_views[rank].copy_(lengths)
            for r in order:
                if n_docs[r]:
                    l_views[r].copy_(self._view(r, self._lens_at[slot], (n_docs[r],), torch.int32))
            lens_event = torch.cuda.Event()
            lens_event.record(self._fetch_small)
            for r in order:
                if n_queries[r]:
                    q_views[r].copy_(self._view(r, self._q_at[slot], (n_queries[r], self.lq, self.dim), self.dtype))
            # this rank's own pieces: needed by the backward pass only
            q_views[rank].copy_(queries)
            d_views[rank].copy_(documents)
            q_event = torch.cuda.Event()
            q_event.record(self._fetch_small)
        doc_events: List[torch.cuda.Event] = [None] * world
        with torch.cuda.stream(self._fetch_docs):
            self._fetch_docs.wait_event(ready)
            for r in order:
                if tokens[r]:
                    d_views[r].copy_(self._view(r, self._docs_at[slot], (tokens[r], self.dim), self.dtype))
                ev = torch.cuda.Event()
                ev.record(self._fetch_docs)
                doc_events[r] = ev
        return lens_event, doc_events, q_event, order

    # -- backward ------------------------------------------------------------

    def send_records(self, argmax, dscore, col_start, sizes) -> torch.Tensor:
        """Store every owner's block of this rank's argmax records in that
        owner's buffer (see ``pack_owner_records``).  Returns this rank's own
        receive buffer ``[Nq_total * n_docs_own * (Lq + 1)]`` int32, complete
        once :meth:`barrier` has been passed on the same stream."""
        rank = self.rank
        n_docs = [s[1] for s in sizes]
        n_queries = [s[2] for s in sizes]
        slot = self._bwd_steps & 1
        self._bwd_steps += 1
        key = (slot, tuple(n_docs), tuple(n_queries))
        table = self._tables.get(key)
        if table is None:
            if len(self._tables) > 64:
                self._tables.clear()
            q_before = sum(n_queries[:rank])
            width = self.lq + 1
            table = torch.tensor(
                [self._bases[o] + self._rec_at[slot] + 4 * q_before * n_docs[o] * width
                 for o in range(self.world)], dtype=torch.int64, device=self.device)
            self._tables[key] = table
        _ops.pack_owner_records_to(argmax, dscore, col_start, table)
        words = sum(n_queries) * n_docs[rank] * (self.lq + 1)
        return self._view(rank, self._rec_at[slot], (words,), torch.int32)
