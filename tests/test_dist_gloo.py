"""The multi-rank drivers on CPU ``gloo`` ranks (world size 2 and 3), with the
CPU oracle standing in for the CUDA operators: shard arithmetic, ragged shard
gathering, column order, per-owner gradient reduction, and a rank that fails
before the exchange."""

from __future__ import annotations

import os
import socket
import sys
import types
from datetime import timedelta
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from maxsim_b200 import dist as mdist  # noqa: E402
from maxsim_b200 import workloads as W  # noqa: E402


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_ops():
    from oracle import maxsim_oracle as oracle

    def fwd(q, d, off):
        s, a = oracle.score_contrastive(q.float().numpy(), d.float().numpy(), off.numpy())
        return torch.from_numpy(s), torch.from_numpy(a)

    def bwd(g, q, d, off, a):
        dq, dd = oracle.contrastive_backward(g.numpy(), q.float().numpy(), d.float().numpy(),
                                             off.numpy(), a.numpy())
        return torch.from_numpy(dq), torch.from_numpy(dd)

    return types.SimpleNamespace(maxsim_contrastive_forward_with_argmax=fwd,
                                 maxsim_contrastive_backward=bwd)


def _oracle_ops_with_blocks():
    """The stand-in operators plus the column-block forward the peer transport
    drives (same contract as the CUDA entry point: the block's offsets are rows
    of ``d``, its columns start at ``col0`` of the wider outputs)."""
    from oracle import maxsim_oracle as oracle
    ops = _oracle_ops()

    def block(q, d, block_offsets, scores, argmax, col0, block_tokens=0, reserve_sms=0):
        off = block_offsets.numpy().astype(np.int64)
        n = off.size - 1
        rows = d.float().numpy()[off[0]:off[-1]]
        s, a = oracle.score_contrastive(q.float().numpy(), rows, (off - off[0]).astype(np.int32))
        scores[:, col0:col0 + n] = torch.from_numpy(s)
        argmax[:, col0:col0 + n] = torch.from_numpy(a)
        return True

    ops.contrastive_forward_block = block
    return ops


class _HostPeer:
    """What ``maxsim_b200.peer.PeerExchange`` does, with gloo collectives in
    place of peer-mapped memory: the driver's use of the transport (which
    columns are scored from which rows, where each rank's records land) runs
    on CPU ranks."""

    class _Done:
        def wait(self):
            return True

    def __init__(self, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.barriers = 0

    def check_fits(self, sizes, lq, dim, dtype):
        assert len(sizes) == self.world

    def barrier(self):
        self.barriers += 1
        dist.barrier(self.group)

    def gather(self, documents, lengths, queries, sizes, docs_all, lens_all, q_all, ranges=None):
        others = sorted(r for first, last in ranges for r in range(first, last))
        assert others == [r for r in range(self.world) if r != self.rank]
        self.ranges = list(ranges)
        for out, local, col in ((docs_all, documents, 0), (lens_all, lengths, 1), (q_all, queries, 2)):
            mdist._all_gather_rows(out, local.detach(), [s[col] for s in sizes], self.group, self.rank).wait()
        return [self._Done() for _ in ranges], self._Done()

    def send_records(self, argmax, dscore, col_start, sizes):
        n_docs, n_queries = [s[1] for s in sizes], [s[2] for s in sizes]
        col0 = col_start.tolist()
        record = torch.cat([argmax.to(torch.int32), dscore.contiguous().view(torch.int32).unsqueeze(-1)], dim=2)
        send = torch.cat([record[:, col0[o]:col0[o + 1]].reshape(-1) for o in range(self.world)])
        width = argmax.shape[2] + 1
        in_splits = [n * argmax.shape[0] * width for n in n_docs]
        out_splits = [n_docs[self.rank] * nq * width for nq in n_queries]
        recv = torch.empty((sum(out_splits),), dtype=torch.int32)
        dist.all_to_all_single(recv, send, out_splits, in_splits, group=self.group)
        return recv


def _padded_scorer(q, d, ql, dl):
    from oracle import maxsim_oracle as oracle
    s, _ = oracle.score_candidates_padded(q.float().numpy(), d.float().numpy(), ql.numpy(), dl.numpy())
    return torch.from_numpy(s)


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=timedelta(seconds=timeout_s))


def _contrastive_worker(rank, world, port, out_dir, exchange):
    _init(rank, world, port)
    try:
        wl = W.c5_contrastive_ties_bf16(seed=31, Nq=12, Nb=11, Lq=16, dim=32, lo=3, hi=40)
        lens = np.diff(wl.document_offsets).astype(np.int32)
        q0, q1 = mdist.shard_range(12, rank, world)
        d0, d1 = mdist.shard_range(11, rank, world)
        t0, t1 = int(wl.document_offsets[d0]), int(wl.document_offsets[d1])
        q = torch.from_numpy(wl.queries[q0:q1]).requires_grad_(True)
        d = torch.from_numpy(wl.documents[t0:t1]).requires_grad_(True)
        sizes = None
        if exchange == "owner" and world == 3:  # also the path where the caller supplies the shard sizes
            sizes = []
            for r in range(world):
                a0, a1 = mdist.shard_range(11, r, world)
                b0, b1 = mdist.shard_range(12, r, world)
                sizes.append((int(wl.document_offsets[a1] - wl.document_offsets[a0]), a1 - a0, b1 - b0))
        peer = None
        if exchange == "peer":  # the owner exchange over the transport object
            exchange, peer = "owner", _HostPeer()
            sizes = []
            for r in range(world):
                a0, a1 = mdist.shard_range(11, r, world)
                b0, b1 = mdist.shard_range(12, r, world)
                sizes.append((int(wl.document_offsets[a1] - wl.document_offsets[a0]), a1 - a0, b1 - b0))
        s = mdist.score_contrastive_sharded(q, d, torch.from_numpy(lens[d0:d1]),
                                            ops=_oracle_ops_with_blocks() if peer else _oracle_ops(),
                                            exchange=exchange, shard_sizes=sizes, peer=peer)
        g = torch.from_numpy(np.random.default_rng(5).standard_normal((12, 11)).astype(np.float32))
        (s * g[q0:q1]).sum().backward()
        docs_per_rank = [mdist.shard_range(11, r, world)[1] - mdist.shard_range(11, r, world)[0]
                         for r in range(world)]
        tgt = mdist.contrastive_targets(q1 - q0, docs_per_rank=docs_per_rank)
        if peer is not None:
            assert peer.barriers == 1  # the backward pass orders the records with one barrier
        np.savez(Path(out_dir) / f"r{rank}.npz", s=s.detach().numpy(), dq=q.grad.numpy(),
                 dd=d.grad.numpy(), tgt=tgt.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,exchange", [(2, "owner"), (3, "owner"), (5, "owner"),  # 5: uneven query shards
                                            (2, "reduce_scatter"), (3, "reduce_scatter"),
                                            (2, "peer"), (3, "peer"), (5, "peer")])
def test_contrastive_sharded_matches_unsharded(world, exchange, tmp_path):
    from oracle import maxsim_oracle as oracle
    port = _free_port()
    mp.spawn(_contrastive_worker, args=(world, port, str(tmp_path), exchange), nprocs=world, join=True)
    wl = W.c5_contrastive_ties_bf16(seed=31, Nq=12, Nb=11, Lq=16, dim=32, lo=3, hi=40)
    ws, wa = oracle.score_contrastive(wl.queries, wl.documents, wl.document_offsets)
    g = np.random.default_rng(5).standard_normal((12, 11)).astype(np.float32)
    wq, wd = oracle.contrastive_backward(g, wl.queries, wl.documents, wl.document_offsets, wa)
    for rank in range(world):
        r = np.load(tmp_path / f"r{rank}.npz")
        q0, q1 = mdist.shard_range(12, rank, world)
        d0, d1 = mdist.shard_range(11, rank, world)
        t0, t1 = int(wl.document_offsets[d0]), int(wl.document_offsets[d1])
        np.testing.assert_allclose(r["s"], ws[q0:q1], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(r["dq"], wq[q0:q1], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(r["dd"], wd[t0:t1], rtol=1e-5, atol=1e-5)
        assert r["tgt"].tolist() == list(range(d0, d0 + (q1 - q0)))


def _rerank_worker(rank, world, port, out_dir):
    _init(rank, world, port)
    try:
        wl = W.c3_large_rerank_fp16(seed=32, Nq=5, C=6, Ld=40, dim=32)
        b0, b1 = mdist.shard_range(5, rank, world)
        args = [torch.from_numpy(x[b0:b1]) for x in (wl.queries, wl.documents, wl.query_lengths,
                                                     wl.doc_lengths)]
        local = mdist.score_candidates_padded_sharded(*args, scorer=_padded_scorer)
        full = mdist.score_candidates_padded_sharded(*args, scorer=_padded_scorer, gather=True)
        np.savez(Path(out_dir) / f"r{rank}.npz", local=local.numpy(), full=full.numpy())
    finally:
        dist.destroy_process_group()


def test_rerank_sharded_by_query(tmp_path):
    from oracle import maxsim_oracle as oracle
    world, port = 2, _free_port()
    mp.spawn(_rerank_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    wl = W.c3_large_rerank_fp16(seed=32, Nq=5, C=6, Ld=40, dim=32)
    ws, _ = oracle.score_candidates_padded(wl.queries, wl.documents, wl.query_lengths, wl.doc_lengths)
    for rank in range(world):
        r = np.load(tmp_path / f"r{rank}.npz")
        b0, b1 = mdist.shard_range(5, rank, world)
        np.testing.assert_allclose(r["local"], ws[b0:b1], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(r["full"], ws, rtol=1e-6, atol=1e-6)


def test_shard_range_covers_everything():
    for n in (0, 1, 7, 256, 1000):
        for world in (1, 2, 3, 8):
            spans = [mdist.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def _failing_worker(rank, world, port, out_dir):
    _init(rank, world, port, timeout_s=5)
    status = "no error"
    try:
        if rank == 1:
            raise RuntimeError("rank 1 fails before the exchange")  # never joins the gather
        q = torch.randn(2, 4, 8)
        d = torch.randn(6, 8)
        mdist.score_contrastive_sharded(q, d, torch.tensor([2, 4]), ops=_oracle_ops())
    except Exception as exc:  # the surviving rank must get an exception, not hang
        status = type(exc).__name__
    Path(out_dir, f"r{rank}.txt").write_text(status)
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_rank_that_never_joins_surfaces_as_an_error(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_failing_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "r1.txt").read_text() == "RuntimeError"
    assert (tmp_path / "r0.txt").read_text() != "no error"


def test_argument_checks():
    q = torch.randn(2, 4, 8)
    d = torch.randn(6, 8)
    with pytest.raises(ValueError, match="1-D"):
        mdist.score_contrastive_sharded(q, d, torch.tensor([[2, 4]]), ops=_oracle_ops())
    with pytest.raises(ValueError, match="at least one document"):
        mdist.score_contrastive_sharded(q, d, torch.tensor([], dtype=torch.int32), ops=_oracle_ops())
    with pytest.raises(TypeError, match="share dtype"):
        mdist.score_contrastive_sharded(q, d.half(), torch.tensor([2, 4]), ops=_oracle_ops())
    # world size 1 needs no process group
    s = mdist.score_contrastive_sharded(q, d, torch.tensor([2, 4]), ops=_oracle_ops())
    assert s.shape == (2, 2)


def test_fetch_schedule_covers_every_other_rank_in_fetch_order():
    # many small shards: several launches, the first ones short; few large ones: one launch
    for world, tokens, nq in ((8, [37000] * 8, 128), (4, [74000] * 4, 256), (2, [150000] * 2, 512),
                              (5, [900, 40000, 10, 70000, 3000], 7), (3, [5, 5, 5], 1)):
        for rank in range(world):
            ranges = mdist.fetch_schedule(rank, tokens, nq, 32, 128, 2)
            order = [r for first, last in ranges for r in range(first, last)]
            assert order == [(rank + k) % world for k in range(1, world)], (world, rank, ranges)
            assert all(0 <= first < last <= world for first, last in ranges)
    assert mdist.fetch_schedule(0, [74000] * 4, 256, 32, 128, 2) == [(1, 4)]
    assert mdist.fetch_schedule(1, [74000] * 4, 256, 32, 128, 2) == [(2, 4), (0, 1)]
    eight = mdist.fetch_schedule(0, [37000] * 8, 128, 32, 128, 2)
    assert 2 <= len(eight) <= 4 and eight[0][1] - eight[0][0] <= 2, eight
