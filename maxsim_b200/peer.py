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
from typing import Sequence, Tuple

import torch
import torch.distributed as dist

from . import _ops

__all__ = ["PeerExchange"]


class _StreamWait:
    """Handle of work on a side stream: ``wait()`` makes the current stream
    wait for the event recorded behind it (no host wait)."""

    def __init__(self, event, device):
        self.event, self.device = event, device

    def wait(self):
        torch.cuda.current_stream(self.device).wait_event(self.event)
        return True


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
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)
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
        _ops.peer_barrier(self._flags, self.rank, self.world, self._counter, self.wait_polls)

    # -- forward -------------------------------------------------------------

    def gather(self, documents, lengths, queries, sizes, docs_all, lens_all, q_all, ranges=None):
        """Publish this rank's shard and gather all shards into the
        rank-ordered ``docs_all [T_total, D]``, ``lens_all [Nb_total]`` and
        ``q_all [Nq_total, Lq, D]``.

        The lengths are complete on the current stream when this returns (one
        small kernel reads them out of the peers' buffers).  The documents
        travel as one copy-engine copy per owner on a side stream, range by
        range: ``ranges`` lists contiguous rank ranges ``(first, last)`` in the
        order to fetch them (default: the ranks after this one, then those
        before it); the queries and this rank's own rows follow on a second
        side stream.  The copies of a range are issued by one call into the
        library.  Returns ``(landed, everything)``: one handle per range and
        one for all transfers, whose ``wait()`` orders the current stream
        behind them.  The caller's tensors must stay untouched until
        ``everything`` has been waited for."""
        rank, world = self.rank, self.world
        tokens = [s[0] for s in sizes]
        n_docs = [s[1] for s in sizes]
        n_queries = [s[2] for s in sizes]
        slot = self._fwd_steps & 1
        self._fwd_steps += 1
        main = torch.cuda.current_stream(self.device)
        plan = self._plan(slot, tuple(tokens), tuple(n_docs), tuple(n_queries))

        item = self._item
        dev = self.device
        if not (documents.is_contiguous() and lengths.is_contiguous() and queries.is_contiguous()):
            raise ValueError("the peer transport takes contiguous tensors")
        # publish: this rank's rows into its own peer-visible buffer
        _ops.copy_many(plan["own_dst"], [documents.data_ptr(), lengths.data_ptr(), queries.data_ptr()],
                       plan["own_bytes"], dev)
        self.barrier()
        ready = plan["events"][0]
        ready.record(main)
        _ops.peer_gather(plan["lens_table"], plan["lens_max"], lens_all)

        row_bytes = self.dim * item
        d_base, q_base = docs_all.data_ptr(), q_all.data_ptr()
        row, q0 = plan["row0"], plan["q0"]
        q_bytes = self.lq * row_bytes
        if ranges is None:
            ranges = [(rank + 1, world), (0, rank)]
        covered = sorted(r for first, last in ranges for r in range(first, last))
        if covered != [r for r in range(world) if r != rank]:
            raise ValueError(f"ranges {ranges} must cover every rank but {rank} exactly once")
        events = plan["events"]
        while len(events) < 2 + len(ranges):
            events.append(torch.cuda.Event())
        landed = []
        with torch.cuda.stream(self._fetch_docs):
            self._fetch_docs.wait_event(ready)
            for k, (first, last) in enumerate(ranges):
                span = range(first, last)
                _ops.copy_many([d_base + row[r] * row_bytes for r in span],
                               [plan["docs_src"][r] for r in span],
                               [tokens[r] * row_bytes for r in span], dev)
                events[2 + k].record(self._fetch_docs)
                landed.append(_StreamWait(events[2 + k], dev))
            last_docs = events[2 + len(ranges) - 1] if ranges else ready
        with torch.cuda.stream(self._fetch_small):
            # needed by the backward pass only: all queries, this rank's own document rows.
            # Behind the documents: the copy engine serves one peer copy at a time, and the
            # forward launches wait for the documents.
            self._fetch_small.wait_event(last_docs)
            others = [r for r in range(world) if r != rank]
            _ops.copy_many(
                [q_base + q0[r] * q_bytes for r in others] + [q_base + q0[rank] * q_bytes,
                                                             d_base + row[rank] * row_bytes],
                [plan["q_src"][r] for r in others] + [queries.data_ptr(), documents.data_ptr()],
                [n_queries[r] * q_bytes for r in others] + [n_queries[rank] * q_bytes,
                                                            tokens[rank] * row_bytes], dev)
            all_event = events[1]
            all_event.record(self._fetch_small)
        return landed, _StreamWait(all_event, dev)

    def _plan(self, slot, tokens, n_docs, n_queries):
        """Views, tables and events of one (slot, shard sizes) combination;
        built once, a training loop asks for the same two every step."""
        key = ("fwd", slot, tokens, n_docs, n_queries)
        plan = self._tables.get(key)
        if plan is not None:
            return plan
        if len(self._tables) > 64:
            self._tables.clear()
        rank, world = self.rank, self.world
        item = self._item
        row0 = [sum(tokens[:r]) for r in range(world + 1)]
        doc0 = [sum(n_docs[:r]) for r in range(world + 1)]
        q0 = [sum(n_queries[:r]) for r in range(world + 1)]
        q_bytes = self.lq * self.dim * item
        lens_rows = [[self._bases[r] + self._lens_at[slot], 0, 4 * doc0[r], 4 * n_docs[r]]
                     for r in range(world) if n_docs[r]]
        plan = {
            "own_dst": [self._bases[rank] + self._docs_at[slot], self._bases[rank] + self._lens_at[slot],
                        self._bases[rank] + self._q_at[slot]],
            "own_bytes": [tokens[rank] * self.dim * item, 4 * n_docs[rank], n_queries[rank] * q_bytes],
            "docs_src": [self._bases[r] + self._docs_at[slot] for r in range(world)],
            "q_src": [self._bases[r] + self._q_at[slot] for r in range(world)],
            "row0": row0,
            "q0": q0,
            "lens_table": torch.tensor(lens_rows, dtype=torch.int64, device=self.device).reshape(len(lens_rows), 4),
            "lens_max": max([4 * n for n in n_docs] + [0]),
            "events": [torch.cuda.Event() for _ in range(2)],  # ready, everything; one per range follows
        }
        self._tables[key] = plan
        return plan

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
