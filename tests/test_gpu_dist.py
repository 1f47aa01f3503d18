"""The multi-GPU drivers on real devices (NCCL, one process per GPU): sharded
contrastive training and query-sharded rerank against the same computation on a
single GPU.  Skipped when fewer than two GPUs are visible."""

from __future__ import annotations

import os
import socket
import sys
from datetime import timedelta
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    import maxsim_b200 as maxsim
    from maxsim_b200 import dist as mdist, workloads as W

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=timedelta(seconds=120))
    try:
        n = 96
        full = W.c5_device(dev, Nq=n, Nb=n, lo=16, hi=200)
        q0, q1 = mdist.shard_range(n, rank, world)
        d0, d1 = mdist.shard_range(n, rank, world)
        part = W.c5_device(dev, Nq=n, Nb=n, lo=16, hi=200, q_begin=q0, q_end=q1, d_begin=d0, d_end=d1)
        off = full["document_offsets"]
        assert torch.equal(part["queries"], full["queries"][q0:q1])
        assert torch.equal(part["documents"], full["documents"][int(off[d0]):int(off[d1])])
        q = part["queries"].clone().requires_grad_(True)
        d = part["documents"].clone().requires_grad_(True)
        lens = full["doc_lengths_all"][d0:d1].to(dev)
        g = torch.randn(n, n, generator=torch.Generator().manual_seed(3)).to(dev)
        # both ways of getting grad_documents to its owner
        q_rs = part["queries"].clone().requires_grad_(True)
        d_rs = part["documents"].clone().requires_grad_(True)
        s_rs = mdist.score_contrastive_sharded(q_rs, d_rs, lens, exchange="reduce_scatter")
        (s_rs * g[q0:q1]).sum().backward()
        s = mdist.score_contrastive_sharded(q, d, lens, exchange="owner")
        (s * g[q0:q1]).sum().backward()
        assert torch.equal(s, s_rs) and torch.equal(q.grad, q_rs.grad)
        torch.testing.assert_close(d.grad.float(), d_rs.grad.float(), rtol=2e-2, atol=2e-2)
        # the same thing on this GPU alone
        qf = full["queries"].clone().requires_grad_(True)
        df = full["documents"].clone().requires_grad_(True)
        sf = maxsim.score_contrastive_train(qf, df, off)
        (sf * g).sum().backward()
        torch.testing.assert_close(s, sf[q0:q1], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(q.grad.float(), qf.grad[q0:q1].float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(d.grad.float(), df.grad[int(off[d0]):int(off[d1])].float(),
                                   rtol=2e-2, atol=2e-2)
        # the owner exchange over peer-mapped buffers, two steps (the buffers alternate)
        from maxsim_b200 import _ops
        from maxsim_b200.peer import PeerExchange
        lens_all = full["doc_lengths_all"].cpu()
        sizes = []
        for r in range(world):
            a0, a1 = mdist.shard_range(n, r, world)
            sizes.append((int(lens_all[a0:a1].sum()), a1 - a0, a1 - a0))
        px = PeerExchange(max_doc_tokens=max(t for t, _, _ in sizes), max_docs=max(c for _, c, _ in sizes),
                          max_queries=max(c for _, _, c in sizes), lq=q.shape[1], dim=q.shape[2],
                          dtype=q.dtype)
        for it in range(3):
            q_p = part["queries"].clone().requires_grad_(True)
            d_p = part["documents"].clone().requires_grad_(True)
            s_p = mdist.score_contrastive_sharded(q_p, d_p, lens, shard_sizes=sizes, peer=px)
            (s_p * g[q0:q1]).sum().backward()
            assert torch.equal(s_p, s), f"peer transport, step {it}: scores differ"
            assert torch.equal(q_p.grad, q.grad)
            torch.testing.assert_close(d_p.grad.float(), d.grad.float(), rtol=2e-2, atol=2e-2)
        assert _ops.device_status() == 0
        # the same step replayed from CUDA graphs (one per buffer slot), on changing inputs
        stepper = maxsim.GraphedShardedContrastiveStep(px, sizes)
        target = mdist.contrastive_targets(q1 - q0, device=dev, docs_per_rank=[c for _, c, _ in sizes])
        for it in range(4):
            q_in = (part["queries"].float() * (1.0 + 0.25 * it)).to(part["queries"].dtype)
            d_in = part["documents"].roll(it, 0).contiguous()
            loss_g, gq, gd = stepper.step(q_in, d_in, lens)
            q_e = q_in.clone().requires_grad_(True)
            d_e = d_in.clone().requires_grad_(True)
            s_e = mdist.score_contrastive_sharded(q_e, d_e, lens, shard_sizes=sizes, peer=px)
            loss_e = torch.nn.functional.cross_entropy(s_e, target, reduction="sum") / n
            loss_e.backward()
            torch.testing.assert_close(loss_g, loss_e.detach(), rtol=1e-5, atol=1e-6)
            assert torch.equal(gq, q_e.grad), f"graphed step {it}: grad_queries differ"
            torch.testing.assert_close(gd.float(), d_e.grad.float(), rtol=2e-2, atol=1e-6)
        assert _ops.device_status() == 0
        # rerank shard
        wl = W.c3_device_shard(rank * 3, rank * 3 + 3, dev, C=40)
        local = mdist.score_candidates_padded_sharded(wl["queries"], wl["documents"],
                                                      wl["query_lengths"], wl["doc_lengths"])
        gathered = mdist.score_candidates_padded_sharded(wl["queries"], wl["documents"],
                                                         wl["query_lengths"], wl["doc_lengths"],
                                                         gather=True)
        assert gathered.shape == (3 * world, 40)
        assert torch.equal(gathered[rank * 3:(rank + 1) * 3], local)
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_drivers_match_single_gpu(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
