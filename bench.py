"""Benchmark of the MaxSim hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload: the large padded rerank configuration (fp16, Nq=256 queries
of Lq=32, C=1000 candidates each, lognormal document lengths padded to 300,
dim 128) -- the configuration the pairs/s metric is quoted on.  A step is one
pass of the padded forward over one such shard.  With N GPUs every rank holds
its own shard of 256 queries (queries are independent, there is no data-path
collective), so the headline scaling is weak: the value is all ranks' pairs
divided by the slowest rank's time.

Printed JSON (one line, rank 0):
  value      pairs/s with inputs resident in HBM, through the C-ABI operator,
             over a burst of K launches right after warm-up
  e2e        pairs/s through the public API from pinned HOST tensors, with the
             host->device copy of that step's inputs and the device->host read
             of its scores inside the timed region
  roofline   algorithmic bytes per launch / measured launch duration, against
             the measured HBM copy bandwidth; `sustained` inside it is the same
             kernel over at least half a second of back-to-back launches
  strong_scaling  the SAME 256-query problem split over the N GPUs (256/N
             queries per rank), next to the weak-scaling headline
  cpu_baseline  the reference's PyTorch CPU formulation (einsum + max) timed on
             all host cores on a bounded sample of the same workload
  train_step contrastive train-step times (forward + cross-entropy + backward)
             for the small and the large bf16 contrastive configurations; with
             N > 1 the large one sharded over the ranks, with the single-GPU
             step of the same run as base and a parity check of its results
  summary    (last key) the figures of the other configurations in short form
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "scored_pairs_per_s"
UNIT = "pairs/s"
WORKLOAD = "c3_padded_rerank_fp16"
C3 = dict(Nq=256, Lq=32, C=1000, Ld=300, dim=128)

# DRAM bytes per algorithmic byte for the streaming forward kernel, from the
# ncu capture summarised in profiles/ (dram__bytes_read.sum + write.sum over the
# algorithmic bytes of the captured launch).  None until a capture exists.
NCU_TRAFFIC_RATIO = 1.0073  # (764.93 MB read + 5.53 MB written) / 764.87 MB, from the ncu capture of this kernel summarised under profiles/


def c3_config(world: int, nq_per_gpu: int):
    """The `config` object of the JSON line; both arms print the same one."""
    from maxsim_b200 import workloads as W

    Lq, C, Ld, dim = (C3[k] for k in ("Lq", "C", "Ld", "dim"))
    _, dlen = W.c3_shard_lengths(0, nq_per_gpu, Lq=Lq, C=C, Ld=Ld)
    return {"workload": WORKLOAD, "per_gpu": dict(Nq=nq_per_gpu, Lq=Lq, C=C, Ld=Ld, dim=dim),
            "pairs_per_gpu": nq_per_gpu * C, "valid_doc_tokens_per_gpu": int(dlen.sum()),
            "parallelism": f"query-sharded x{world}, no collective",
            "l2": "inputs (19.7 GB padded, 12.3 GB valid) are larger than L2"}


def use_all_host_cores() -> int:
    """The CPU legs run on every core of the box, whatever a launcher put in
    OMP_NUM_THREADS (torch.distributed.run sets it to 1)."""
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                        source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------
# clocks sampling
# ---------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons of one GPU while the
    benchmark runs.  Uses NVML from a thread of this process: two light queries
    per sample.  (An `nvidia-smi -lms` subprocess polling many fields was seen
    to stall kernels of the timed loop for 10-20 ms at a time.)"""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, device_index: int, interval_s: float = 0.05):
        self.interval = interval_s
        self.samples = []
        self._stop = None
        self._thread = None
        self._handle = None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(ident.encode())
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(ident)
            self._nvml = pynvml
        except Exception:
            self._handle = None

    def _loop(self):
        nv, h = self._nvml, self._handle
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((mhz, int(reasons)))
            except Exception:
                pass
            self._stop.wait(self.interval)

    def start(self):
        if self._handle is None:
            return
        import threading
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def mark(self):
        """Index of the next sample: brackets a region of interest."""
        return len(self.samples)

    def stop(self, begin: int = 0, end=None):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        return self.summary(begin, end)

    def summary(self, begin: int = 0, end=None):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self._thread is None:
            return out
        rows = self.samples[begin:end] or self.samples
        if not rows:
            return out
        try:
            out["sm_max_mhz"] = self._nvml.nvmlDeviceGetMaxClockInfo(self._handle, self._nvml.NVML_CLOCK_SM)
        except Exception:
            out["sm_max_mhz"] = max(r[0] for r in rows)
        out["sm_mhz"] = statistics.median(r[0] for r in rows)
        out["samples"] = len(rows)
        seen = 0
        for _, r in rows:
            seen |= r
        out["reasons"] = [name for bit, name in self.REASONS.items() if seen & bit]
        return out


# ---------------------------------------------------------------------------
# CPU baseline (the reference's PyTorch formulation, restated in oracle/)
# ---------------------------------------------------------------------------

def cpu_padded_baseline(target_seconds: float = 12.0, sample_queries: int = 4, seed: int = 2):
    """Times einsum+max on the host for a bounded sample of the rerank workload
    (whole queries with all their C candidates, repeated until about
    `target_seconds` of CPU work).  Returns (pairs_per_s, cores, sample)."""
    from maxsim_b200 import workloads as W
    from oracle import torch_cpu_path as cpu  # baseline leg only

    threads = use_all_host_cores()
    wl = W.c3_large_rerank_fp16(seed=seed, Nq=sample_queries,
                                **{k: C3[k] for k in ("Lq", "C", "Ld", "dim")})
    q, d = W.to_torch(wl.queries, "fp16"), W.to_torch(wl.documents, "fp16")
    ql, dl = torch.from_numpy(wl.query_lengths).long(), torch.from_numpy(wl.doc_lengths).long()
    cpu.padded_scores(q[:1], d[:1], ql[:1], dl[:1], chunk=1)  # warm-up
    t0 = time.perf_counter()
    cpu.padded_scores(q, d, ql, dl, chunk=1)
    once = time.perf_counter() - t0
    reps = int(max(1, min(400, target_seconds / max(once, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        cpu.padded_scores(q, d, ql, dl, chunk=1)
    dt = time.perf_counter() - t0
    pairs = sample_queries * C3["C"] * reps
    return pairs / dt, threads, (f"{sample_queries} queries x {C3['C']} candidates of {WORKLOAD}, "
                                 f"{reps} passes, {dt:.1f} s")


def run_reference_arm(args):
    """The reference's own CPU path (PyTorch einsum + max) on the host cores.
    The reference is a Python package whose CPU implementation is its pure
    PyTorch formulation; it is restated in oracle/torch_cpu_path.py."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from maxsim_b200 import workloads as W
    from oracle import torch_cpu_path as cpu

    cores = use_all_host_cores()
    nq = 4
    wl = W.c3_large_rerank_fp16(seed=2, Nq=nq, **{k: C3[k] for k in ("Lq", "C", "Ld", "dim")})
    q, d = W.to_torch(wl.queries, "fp16"), W.to_torch(wl.documents, "fp16")
    ql, dl = torch.from_numpy(wl.query_lengths).long(), torch.from_numpy(wl.doc_lengths).long()
    for _ in range(max(1, min(args.warmup, 3))):
        cpu.padded_scores(q, d, ql, dl, chunk=1)
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu.padded_scores(q, d, ql, dl, chunk=1)
    dt = time.perf_counter() - t0
    pairs = nq * C3["C"]
    value = steps * pairs / dt
    sample = f"{nq} queries x {C3['C']} candidates per step of {WORKLOAD}"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": c3_config(max(1, args.gpus), 16 if args.small else C3["Nq"]),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores,
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------

def _event_ms(fn, iters: int):
    """Per-iteration device times of fn() in ms, CUDA events on the current stream."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(iters)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def contrastive_train_step(maxsim, q, d, off, target):
    q.grad = None
    d.grad = None
    s = maxsim.score_contrastive_train(q, d, off)
    loss = torch.nn.functional.cross_entropy(s, target)
    loss.backward()
    return loss


def bench_train_steps(dev, peaks, full: bool):
    """Contrastive train-step times: the 64x64 configuration always, the
    1024x1024 configuration with ties when `full`."""
    import maxsim_b200 as maxsim
    from maxsim_b200 import workloads as W

    out = {}
    wl = W.c2_contrastive_train_bf16()
    q = W.to_torch(wl.queries, "bf16", dev).requires_grad_(True)
    d = W.to_torch(wl.documents, "bf16", dev).requires_grad_(True)
    off = torch.from_numpy(wl.document_offsets).to(dev)
    target = torch.arange(q.shape[0], device=dev)
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)

    def step2():
        flush.zero_()
        contrastive_train_step(maxsim, q, d, off, target)

    def only_flush():
        flush.zero_()

    for _ in range(5):
        step2()
    t_all = statistics.median(_event_ms(step2, 30))
    t_flush = statistics.median(_event_ms(only_flush, 30))
    def step2_fused():
        flush.zero_()
        q.grad = None
        d.grad = None
        maxsim.contrastive_loss(q, d, off).backward()

    for _ in range(5):
        step2_fused()
    t_fused = statistics.median(_event_ms(step2_fused, 30)) - t_flush
    # the same step captured once in a CUDA graph and replayed (launch overhead removed)
    t_graph = None
    try:
        def graph_body():
            loss = maxsim.contrastive_loss(q, d, off)
            return torch.autograd.grad(loss, (q, d))

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                graph_body()
        torch.cuda.current_stream().wait_stream(side)
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            graph_body()

        def step2_graph():
            flush.zero_()
            cg.replay()

        for _ in range(5):
            step2_graph()
        t_graph = statistics.median(_event_ms(step2_graph, 30)) - t_flush
    except Exception as exc:  # report, do not fail the benchmark
        t_graph = f"unavailable: {type(exc).__name__}"
    lens = np.diff(wl.document_offsets).astype(np.int64)
    flops = 2 * 128 * q.shape[0] * 32 * int(lens.sum()) + 4 * 128 * q.shape[0] * lens.shape[0] * 32
    out["c2_contrastive_train_bf16"] = {
        "ms_per_step": t_all - t_flush, "pairs_per_s": q.shape[0] * lens.shape[0] / ((t_all - t_flush) * 1e-3),
        "tensor_frac": flops / ((t_all - t_flush) * 1e-3) / (peaks["bf16_tflops"] * 1e12),
        "ms_per_step_fused_loss": t_fused,
        "ms_per_step_cuda_graph": t_graph,
        "note": "Nq=Nb=64; L2 flushed between steps (flush time subtracted); launch-latency bound; "
                "fused_loss = contrastive_loss() instead of score_contrastive_train + torch cross_entropy; "
                "cuda_graph = that step (loss + both gradients) captured once and replayed",
    }
    # config 1: padded rerank forward + argmax, fp32 (512 pairs; launch-latency bound)
    wl1 = W.c1_padded_rerank_fp32()
    q1, d1 = W.to_torch(wl1.queries, "fp32", dev), W.to_torch(wl1.documents, "fp32", dev)
    ql1 = torch.from_numpy(wl1.query_lengths).to(dev)
    dl1 = torch.from_numpy(wl1.doc_lengths).to(dev)

    def step1():
        flush.zero_()
        maxsim.score_candidates_padded_with_argmax(q1, d1, ql1, dl1)

    for _ in range(5):
        step1()
    t1 = statistics.median(_event_ms(step1, 30)) - t_flush
    bytes1 = (int(wl1.doc_lengths.sum()) + 16 * 32) * 128 * 4 + 512 * 4 + 512 * 32 * 4
    out["c1_padded_rerank_fp32"] = {
        "ms": t1, "pairs_per_s": 512 / (t1 * 1e-3),
        "hbm_frac": bytes1 / (t1 * 1e-3) / (peaks["hbm_gbs"] * 1e9),
        "note": "Nq=16, C=32, forward with fp32 argmax; L2 flushed (flush time subtracted); launch-latency bound"}

    if full:
        # config 4: packed ragged pair grid, fp16, forward + backward
        wl4 = W.c4_packed_grid_fp16()
        q4 = W.to_torch(wl4.queries, "fp16", dev).requires_grad_(True)
        d4 = W.to_torch(wl4.documents, "fp16", dev).requires_grad_(True)
        qo4 = torch.from_numpy(wl4.query_offsets).to(dev)
        do4 = torch.from_numpy(wl4.document_offsets).to(dev)
        pq4 = torch.from_numpy(wl4.pair_query_ids).to(dev)
        pd4 = torch.from_numpy(wl4.pair_document_ids).to(dev)
        g4 = torch.from_numpy(wl4.dscore).to(dev)

        def step4():
            q4.grad = None
            d4.grad = None
            s4 = maxsim.score_pairs_packed_train(q4, qo4, d4, do4, pq4, pd4, max_q_len=32)
            s4.backward(g4)

        def fwd4():
            maxsim._ops.ops.maxsim_packed_forward_with_argmax(q4.detach(), qo4, d4.detach(), do4,
                                                              pq4, pd4, 32)

        maxsim._ops.set_pair_grouping(False)
        for _ in range(3):
            step4()
        t4_list = statistics.median(_event_ms(step4, 10))
        t4f_list = statistics.median(_event_ms(fwd4, 10))
        maxsim._ops.set_pair_grouping(True)
        for _ in range(3):
            step4()
        t_group = statistics.median(_event_ms(lambda: maxsim._ops.group_pairs(pd4, do4.shape[0] - 1), 10))
        t4 = statistics.median(_event_ms(step4, 10))
        t4f = statistics.median(_event_ms(fwd4, 10))
        dl = np.diff(wl4.document_offsets).astype(np.int64)
        qlens = np.diff(wl4.query_offsets).astype(np.int64)
        pair_doc_bytes = int(dl[wl4.pair_document_ids].sum()) * 96 * 2   # documents are streamed per pair
        fwd_bytes = pair_doc_bytes + int(qlens[wl4.pair_query_ids].sum()) * 96 * 2 + 65536 * (4 + 32 * 4)
        bwd_bytes = (q4.numel() + d4.numel()) * 4 * 2 + 65536 * (4 + 32 * 4)      # zero fill + accumulate
        out["c4_packed_grid_fp16"] = {
            "ms_per_step": t4, "forward_ms": t4f, "pairs_per_s": 65536 / (t4 * 1e-3),
            "forward_hbm_frac": fwd_bytes / (t4f * 1e-3) / (peaks["hbm_gbs"] * 1e9),
            "step_hbm_frac": (fwd_bytes + bwd_bytes) / (t4 * 1e-3) / (peaks["hbm_gbs"] * 1e9),
            "forward_ms_list_order": t4f_list, "ms_per_step_list_order": t4_list,
            "group_pairs_ms": t_group,
            "forward_unique_doc_hbm_frac": ((int(dl[np.unique(wl4.pair_document_ids)].sum())
                                             + int(qlens.sum())) * 96 * 2 + 65536 * (4 + 32 * 4))
            / (t4f * 1e-3) / (peaks["hbm_gbs"] * 1e9),
            "note": "65536 pairs with duplicates, dim 96; pairs are visited in document order (the "
                    "grouping is built once per pair-id tensor by three small kernels, group_pairs_ms, "
                    "and remembered), so repeats of a document hit in L2, and the backward runs on "
                    "owner warps over the by-query and by-document groups (no zero fill, no atomics); "
                    "forward_hbm_frac counts the bytes streamed through the SMs (1.6 GB, every pair's "
                    "document), forward_unique_doc_hbm_frac the unique bytes (0.54 GB); *_list_order = "
                    "the same calls in list order with atomic routing; step = forward+argmax and "
                    "backward through the public API"}
        del q4, d4, wl4

        data = W.c5_device(dev)
        q5 = data["queries"].requires_grad_(True)
        d5 = data["documents"].requires_grad_(True)
        off5 = data["document_offsets"]
        t5 = torch.arange(q5.shape[0], device=dev)
        for _ in range(3):
            contrastive_train_step(maxsim, q5, d5, off5, t5)
        ms = statistics.median(_event_ms(lambda: contrastive_train_step(maxsim, q5, d5, off5, t5), 10))
        with torch.no_grad():
            fwd = statistics.median(_event_ms(
                lambda: maxsim._ops.ops.maxsim_contrastive_forward_with_argmax(q5.detach(), d5.detach(), off5), 10))
        T = int(d5.shape[0])
        flops = 2 * 128 * 1024 * 32 * T + 4 * 128 * 1024 * 1024 * 32
        out["c5_contrastive_train_bf16"] = {
            "ms_per_step": ms, "forward_ms": fwd, "pairs_per_s": 1024 * 1024 / (ms * 1e-3),
            "tensor_frac": flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12),
            "forward_tensor_frac": (2 * 128 * 1024 * 32 * T) / (fwd * 1e-3) / (peaks["bf16_tflops"] * 1e12),
            "note": "Nq=Nb=1024, 5% duplicated tokens; step = forward+argmax, cross-entropy, backward",
        }
        del q5, d5, data

        # hard-negative training on the padded layout: 128 queries x 64 candidates, bf16
        wlp = W.c3_large_rerank_fp16(seed=21, Nq=128, C=64, Ld=300)
        qp = W.to_torch(wlp.queries, "bf16", dev).requires_grad_(True)
        dp = W.to_torch(wlp.documents, "bf16", dev).requires_grad_(True)
        qlp = torch.from_numpy(wlp.query_lengths).to(dev)
        dlp = torch.from_numpy(wlp.doc_lengths).to(dev)
        tp = torch.zeros(128, dtype=torch.int64, device=dev)

        def step_p():
            qp.grad = None
            dp.grad = None
            sp = maxsim.score_candidates_padded_train(qp, dp, qlp, dlp)
            torch.nn.functional.cross_entropy(sp, tp).backward()

        for _ in range(3):
            step_p()
        tpd = statistics.median(_event_ms(step_p, 10))
        valid = int(wlp.doc_lengths.sum()) * 128 * 2
        out["padded_hard_negative_train_bf16"] = {
            "ms_per_step": tpd, "pairs_per_s": 128 * 64 / (tpd * 1e-3),
            "step_hbm_frac": (valid + dp.numel() * 2 + 128 * 64 * 32 * 8) / (tpd * 1e-3)
            / (peaks["hbm_gbs"] * 1e9),
            "note": "B=128, C=64, Ld_max=300; step = forward+argmax, cross-entropy, backward through "
                    "the public API; gradients are written once by the kernels in bf16; step_hbm_frac "
                    "counts the valid document tokens read, 2 B per gradient element written and the "
                    "argmax written and read"}
        del qp, dp, wlp

        # either side of the operators: packing an encoder output, ranking a rerank result
        enc = torch.randn(1024, 512, 128, device=dev, dtype=torch.bfloat16)
        ln = torch.randint(64, 513, (1024,), device=dev, dtype=torch.int32)
        total = int(ln.sum())
        for _ in range(3):
            maxsim.pack_padded(enc, ln, total_tokens=total)
        t_pack = statistics.median(_event_ms(lambda: maxsim.pack_padded(enc, ln, total_tokens=total), 20))
        mask = torch.arange(512, device=dev)[None, :] < ln[:, None]
        t_pack_torch = statistics.median(_event_ms(lambda: enc.reshape(-1, 128)[mask.reshape(-1)], 10))
        sc = torch.randn(256, 1000, device=dev)
        for _ in range(3):
            maxsim.rerank_topk(sc, 100)
        t_topk = statistics.median(_event_ms(lambda: maxsim.rerank_topk(sc, 100), 20))
        t_topk_torch = statistics.median(_event_ms(lambda: torch.topk(sc, 100, dim=1), 20))
        t_sort = statistics.median(_event_ms(lambda: maxsim.rerank_order(sc), 20))
        t_sort_torch = statistics.median(_event_ms(lambda: sc.argsort(dim=1, descending=True), 20))
        out["layout_steps"] = {
            "pack_1024x512x128_bf16_ms": t_pack,
            "pack_hbm_frac": 2 * total * 256 / (t_pack * 1e-3) / (peaks["hbm_gbs"] * 1e9),
            "pack_torch_mask_gather_ms": t_pack_torch,
            "topk100_256x1000_ms": t_topk, "topk100_torch_ms": t_topk_torch,
            "rank_256x1000_ms": t_sort, "rank_torch_argsort_ms": t_sort_torch,
            "note": "pack = offsets scan + segment copy (no host synchronisation); ranking = one CTA per row; "
                    "torch figures are the formulations the reference's callers use, same device"}
    return out


# The reference's own benchmark matrix (scripts/bench_matrix.py:711-724 of the
# reference: shapes; :237-265: method -- one CUDA-event pair per iteration with
# a synchronise after it, median of 30 after 10 warm-ups, the Python wrapper
# and, for the training rows, two input clones inside the timed call).  The
# published figures are the reference's maxsim_step_ms on an H200
# (bench_results/v2/h200.json), i.e. other hardware.
REFERENCE_MATRIX = [
    ("Contrastive", "contrastive", dict(Nq=32, Nb=32, Lq=32, Ld=80, dim=128), {"fp16": 0.261, "bf16": 0.272}),
    ("LongDocs", "contrastive", dict(Nq=32, Nb=32, Lq=32, Ld=512, dim=128), {"fp16": 0.270}),
    ("BigBatch", "contrastive", dict(Nq=64, Nb=64, Lq=32, Ld=128, dim=128), {"fp16": 0.320, "bf16": 0.321}),
    ("Rerank", "padded", dict(B=32, C=50, Lq=32, Ld=180, dim=128), {"fp16": 0.327, "bf16": 0.338}),
    ("HeavyRerank", "padded", dict(B=32, C=100, Lq=32, Ld=256, dim=128), {"fp16": 0.335, "bf16": 0.374}),
    ("PackedRerank", "packed", dict(B=32, C=50, Lq=32, Ld=180, dim=128), {"fp16": 5.527}),
    ("PackedHeavyRerank", "packed", dict(B=32, C=100, Lq=32, Ld=256, dim=128), {"fp16": 14.640}),
]


def bench_reference_matrix(dev):
    import maxsim_b200 as maxsim

    def timed(fn, iters=30, warm=10):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        out = []
        for _ in range(iters):
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return statistics.median(out)

    rows = []
    for name, kind, shp, published in REFERENCE_MATRIX:
        for dname, ref_ms in published.items():
            dtype = torch.float16 if dname == "fp16" else torch.bfloat16
            gen = torch.Generator().manual_seed(1234)
            if kind == "contrastive":
                q = torch.randn(shp["Nq"], shp["Lq"], shp["dim"], generator=gen).to(dev, dtype)
                docs = torch.randn(shp["Nb"] * shp["Ld"], shp["dim"], generator=gen).to(dev, dtype)
                cu = torch.arange(0, (shp["Nb"] + 1) * shp["Ld"], shp["Ld"], dtype=torch.int32, device=dev)

                def step():
                    q_r = q.detach().clone().requires_grad_(True)
                    d_r = docs.detach().clone().requires_grad_(True)
                    maxsim.score_contrastive_train(q_r, d_r, cu).sum().backward()
            else:
                B, C, Lq, Ld, dim = (shp[k] for k in ("B", "C", "Lq", "Ld", "dim"))
                q = torch.randn(B, Lq, dim, generator=gen).to(dev, dtype)
                d = torch.randn(B, C, Ld, dim, generator=gen).to(dev, dtype)
                qlen = torch.full((B,), Lq, dtype=torch.int32, device=dev)
                dlen = torch.full((B, C), Ld, dtype=torch.int32, device=dev)
                if kind == "padded":
                    def step():
                        return maxsim.score_candidates_padded(q, d, qlen, dlen)
                else:
                    qf = q.reshape(B * Lq, dim).contiguous()
                    df = d.reshape(B * C * Ld, dim).contiguous()
                    qoff = torch.arange(0, (B + 1) * Lq, Lq, dtype=torch.int32, device=dev)
                    doff = torch.arange(0, (B * C + 1) * Ld, Ld, dtype=torch.int32, device=dev)
                    qids = torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(C)
                    dids = torch.arange(B * C, dtype=torch.int32, device=dev)

                    def step():
                        return maxsim.score_pairs_packed(qf, qoff, df, doff, qids, dids, max_q_len=Lq)
            ms = timed(step)
            row = {"name": name, "dtype": dname, "shape": shp, "ms": round(ms, 4),
                   "reference_h200_ms": ref_ms, "ratio": round(ref_ms / ms, 2)}
            if kind == "contrastive":
                # the same training step (in-batch cross-entropy instead of a plain sum)
                # replayed from a CUDA graph, input copies into the static buffers included
                try:
                    stepper = maxsim.GraphedContrastiveStep(shp["Nq"], shp["Lq"], shp["Nb"], shp["dim"],
                                                            shp["Nb"] * shp["Ld"] + 64, dtype=dtype, device=dev)
                    row["graphed_step_ms"] = round(timed(lambda: stepper.step(q, docs, cu)), 4)
                    del stepper
                except Exception as exc:  # report, do not fail the benchmark
                    row["graphed_step_ms"] = f"unavailable: {type(exc).__name__}"
            rows.append(row)
    return {"rows": rows,
            "note": "the reference's benchmark matrix with its timing method (per-iteration CUDA events "
                    "and synchronise, median of 30, Python wrapper and input clones included); "
                    "reference_h200_ms are the reference's published H200 figures (other hardware), "
                    "ratio = reference_h200_ms / ms; graphed_step_ms = GraphedContrastiveStep.step "
                    "(loss + both gradients replayed from a CUDA graph) on the same batch"}


def bench_sharded_train_step(dev, dist, rank, world, peaks, small=False):
    """Contrastive training step of the 1024 x 1024 ties configuration with
    queries and documents sharded over the ranks (strong scaling).  Forward:
    all-gather of the document shards, this rank's queries scored against all
    documents, cross-entropy on diagonal targets.  Backward: grad_queries where
    the queries are; for grad_documents each owner receives the argmax / score
    gradient records of its documents and the all-gathered queries and computes
    the gradient of its own shard (`exchange="owner"`, the default), or every
    rank routes a partial gradient and the sums are reduce-scattered.

    The same run times the whole problem on one GPU (every rank does, the
    slowest counts) as the base of the speed-up, and checks the sharded results:
    scores and grad_queries against the single-GPU step's rows, grad_documents
    against its shard, and the identity sum(grad_q * q) = sum(grad_d * d) =
    sum(dscore * scores) over all ranks."""
    import maxsim_b200 as maxsim
    from maxsim_b200 import dist as mdist
    from maxsim_b200 import workloads as W

    n = 256 if small else 1024
    full = W.c5_device(dev, Nq=n, Nb=n)
    qf = full["queries"].requires_grad_(True)
    df = full["documents"].requires_grad_(True)
    off_f = full["document_offsets"]
    tf = torch.arange(n, device=dev)

    def reduce_max(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # --- the whole problem on one GPU (base of the speed-up, source of the parity check)
    for _ in range(3):
        contrastive_train_step(maxsim, qf, df, off_f, tf)
    torch.cuda.synchronize()
    dist.barrier()
    ms_single = reduce_max(statistics.median(
        _event_ms(lambda: contrastive_train_step(maxsim, qf, df, off_f, tf), 10)))
    qf.grad = None
    df.grad = None
    s_full = maxsim.score_contrastive_train(qf, df, off_f)
    torch.nn.functional.cross_entropy(s_full, tf).backward()

    q0, q1 = mdist.shard_range(n, rank, world)
    d0, d1 = mdist.shard_range(n, rank, world)
    offs_host = off_f.cpu()
    t0, t1 = int(offs_host[d0]), int(offs_host[d1])
    q = qf.detach()[q0:q1].clone().requires_grad_(True)
    d = df.detach()[t0:t1].clone().requires_grad_(True)
    lens_host = full["doc_lengths_all"].cpu()
    lens = lens_host[d0:d1].to(dev)
    docs_per_rank = [mdist.shard_range(n, r, world)[1] - mdist.shard_range(n, r, world)[0]
                     for r in range(world)]
    target = mdist.contrastive_targets(q1 - q0, device=dev, docs_per_rank=docs_per_rank)
    shard_sizes = []
    for r in range(world):
        a0, a1 = mdist.shard_range(n, r, world)
        shard_sizes.append((int(lens_host[a0:a1].sum()), a1 - a0, a1 - a0))

    # the record exchange of the backward pass on a group with NCCL's default CTA count
    records_group = dist.new_group(
        backend="nccl",
        pg_options=dist.ProcessGroupNCCL.Options(is_high_priority_stream=True))

    # exchange buffers in peer-mapped memory (all ranks on one node); if the mapping cannot be
    # set up here the collective transport alone is measured and the reason is reported
    peer, peer_error = None, None
    try:
        from maxsim_b200.peer import PeerExchange
        peer = PeerExchange(max_doc_tokens=max(s[0] for s in shard_sizes),
                            max_docs=max(s[1] for s in shard_sizes),
                            max_queries=max(s[2] for s in shard_sizes),
                            lq=q.shape[1], dim=q.shape[2], dtype=q.dtype,
                            wait_polls=1 << 21)  # a barrier gives up after about two seconds
    except Exception as exc:  # noqa: BLE001 -- reported in the record
        peer_error = f"{type(exc).__name__}: {exc}"[:300]
    have = torch.tensor([1 if peer is not None else 0], device=dev)
    dist.all_reduce(have, op=dist.ReduceOp.MIN)
    if not bool(have.item()):
        peer = None

    def one_step(exchange, sizes, keep=False, transport=None):
        q.grad = None
        d.grad = None
        s = mdist.score_contrastive_sharded(q, d, lens, exchange=exchange, shard_sizes=sizes,
                                            records_group=records_group, peer=transport)
        if keep:
            s.retain_grad()
        # every rank averages over its own queries; the global mean is over all n
        loss = torch.nn.functional.cross_entropy(s, target, reduction="sum") / n
        loss.backward()
        return s, loss

    # --- parity of the sharded step
    def check(exchange, sizes, transport=None):
        s, loss = one_step(exchange, sizes, keep=True, transport=transport)
        g = s.grad
        sums = torch.stack([(g.double() * s.detach().double()).sum(),
                            (q.grad.double() * q.detach().double()).sum(),
                            (d.grad.double() * d.detach().double()).sum(),
                            (g.double() * s.detach().double()).abs().sum(),
                            loss.detach().double()])
        dist.all_reduce(sums)
        gs, gq, gd, scale, loss_all = (float(x) for x in sums.tolist())
        ref_loss = float(torch.nn.functional.cross_entropy(s_full.detach(), tf))
        dq_err = float((q.grad.float() - qf.grad[q0:q1].float()).abs().max())
        dd_err = float((d.grad.float() - df.grad[t0:t1].float()).abs().max())
        dd_ref = float(df.grad[t0:t1].float().abs().max())
        rec = {"scores_equal_single_gpu": bool(torch.equal(s.detach(), s_full.detach()[q0:q1])),
               "loss": loss_all, "loss_single_gpu": ref_loss,
               "sum_dscore_scores": gs, "sum_gradq_q": gq, "sum_gradd_d": gd,
               "grad_q_max_abs_diff_vs_single_gpu": dq_err,
               "grad_d_max_abs_diff_vs_single_gpu": dd_err, "grad_d_max_abs": dd_ref}
        ok = (rec["scores_equal_single_gpu"] and abs(loss_all - ref_loss) <= 1e-4 * max(1.0, abs(ref_loss))
              and abs(gq - gs) <= 1e-2 * scale and abs(gd - gs) <= 1e-2 * scale
              and dq_err <= 1e-2 * max(1e-6, float(qf.grad.float().abs().max()))
              and dd_err <= 2e-2 * max(1e-6, dd_ref))
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        rec["ok_all_ranks"] = bool(flag.item())
        return rec, s.detach()

    par_owner, s_owner = check("owner", shard_sizes)
    par_rs, s_rs = check("reduce_scatter", None)
    same = torch.tensor([1 if torch.equal(s_owner, s_rs) else 0], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    parity_ok = par_owner["ok_all_ranks"] and par_rs["ok_all_ranks"] and bool(same.item())
    par_peer = None
    if peer is not None:
        par_peer, s_peer = check("owner", shard_sizes, peer)
        same_p = torch.tensor([1 if torch.equal(s_owner, s_peer) else 0], device=dev)
        dist.all_reduce(same_p, op=dist.ReduceOp.MIN)
        status = torch.tensor([_ops_status()], device=dev)
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
        par_peer["device_status_all_ranks"] = int(status.item())
        parity_ok = (parity_ok and par_peer["ok_all_ranks"] and bool(same_p.item())
                     and int(status.item()) == 0)

    def timed(exchange, sizes=None, transport=None):
        for _ in range(3):
            one_step(exchange, sizes, transport=transport)
        torch.cuda.synchronize()
        dist.barrier()
        iters = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            one_step(exchange, sizes, transport=transport)
        e1.record()
        torch.cuda.synchronize()
        return reduce_max(e0.elapsed_time(e1) / iters)

    ms_rs = timed("reduce_scatter")
    ms_owner = timed("owner")
    ms_nccl = timed("owner", shard_sizes)
    ms_peer = timed("owner", shard_sizes, peer) if peer is not None else None

    # the same step over the peer transport, captured in CUDA graphs and replayed
    ms_graph, graph_error, par_graph = None, None, None
    if peer is not None:
        stepper = None
        try:
            stepper = maxsim.GraphedShardedContrastiveStep(peer, shard_sizes)
        except Exception as exc:  # noqa: BLE001 -- reported in the record
            graph_error = f"{type(exc).__name__}: {exc}"[:300]
        have = torch.tensor([1 if stepper is not None else 0], device=dev)
        dist.all_reduce(have, op=dist.ReduceOp.MIN)
        if bool(have.item()):
            qd, dd_ = q.detach(), d.detach()
            loss_g, gq, gd = stepper.step(qd, dd_, lens)
            loss_all = loss_g.detach().double().clone()
            dist.all_reduce(loss_all)
            ref_loss = float(torch.nn.functional.cross_entropy(s_full.detach(), tf))
            dq_err = float((gq.float() - qf.grad[q0:q1].float()).abs().max())
            dd_err = float((gd.float() - df.grad[t0:t1].float()).abs().max())
            status = torch.tensor([_ops_status()], device=dev)
            dist.all_reduce(status, op=dist.ReduceOp.MAX)
            ok = (abs(float(loss_all) - ref_loss) <= 1e-4 * max(1.0, abs(ref_loss))
                  and dq_err <= 1e-2 * max(1e-6, float(qf.grad.float().abs().max()))
                  and dd_err <= 2e-2 * max(1e-6, float(df.grad[t0:t1].float().abs().max()))
                  and int(status.item()) == 0)
            flag = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            par_graph = {"loss": float(loss_all), "loss_single_gpu": ref_loss,
                         "grad_q_max_abs_diff_vs_single_gpu": dq_err,
                         "grad_d_max_abs_diff_vs_single_gpu": dd_err,
                         "device_status_all_ranks": int(status.item()),
                         "ok_all_ranks": bool(flag.item())}
            parity_ok = parity_ok and par_graph["ok_all_ranks"]
            if par_graph["ok_all_ranks"]:
                for _ in range(4):
                    stepper.step(qd, dd_, lens)
                torch.cuda.synchronize()
                dist.barrier()
                iters = 10
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    stepper.step(qd, dd_, lens)
                e1.record()
                torch.cuda.synchronize()
                ms_graph = reduce_max(e0.elapsed_time(e1) / iters)
        elif graph_error is None:
            graph_error = "capture failed on another rank"
    ms = ms_graph if ms_graph is not None else ms_peer if ms_peer is not None else ms_nccl
    T = int(full["doc_lengths_all"].sum().item())
    flops = 2 * 128 * n * 32 * T + 4 * 128 * n * n * 32
    return {"c5_contrastive_train_bf16_sharded": {
        "ms_per_step": ms, "pairs_per_s": n * n / (ms * 1e-3),
        "single_gpu_ms_same_run": ms_single, "speedup": ms_single / ms,
        "efficiency": ms_single / ms / world,
        "tensor_frac_all_gpus": flops / (ms * 1e-3) / (world * peaks["bf16_tflops"] * 1e12),
        "parity_ok": parity_ok,
        "transport": ("peer, step replayed from CUDA graphs" if ms_graph is not None
                      else "peer" if ms_peer is not None else "nccl"),
        "peer_transport_unavailable": peer_error,
        "graph_capture_unavailable": graph_error,
        "ms_per_step_peer_eager": ms_peer,
        "efficiency_peer_eager": (ms_single / ms_peer / world) if ms_peer is not None else None,
        "parity": {"owner": par_owner, "reduce_scatter": par_rs, "owner_peer_transport": par_peer,
                   "owner_peer_transport_graphed": par_graph,
                   "owner_and_reduce_scatter_scores_equal": bool(same.item())},
        "ms_per_step_nccl": ms_nccl, "efficiency_nccl": ms_single / ms_nccl / world,
        "ms_per_step_sizes_exchanged_in_step": ms_owner,
        "ms_per_step_reduce_scatter": ms_rs,
        "efficiency_reduce_scatter": ms_single / ms_rs / world,
        "note": f"global Nq=Nb={n} over {world} ranks (strong scaling); ms_per_step: owner exchange "
                "with every rank's shard sizes passed in (known to the data pipeline), so the host "
                "never waits for the device, over the transport named in 'transport' -- 'peer': "
                "shards fetched from peer-mapped buffers by the copy engines, argmax records stored "
                "into the owners' memory by the regrouping kernel, one barrier kernel per pass; "
                "'peer, step replayed from CUDA graphs': the same, the whole step (input copies into "
                "static buffers, exchange, forward, loss, both gradients) captured once per buffer "
                "slot and replayed (GraphedShardedContrastiveStep), ms_per_step_peer_eager being the "
                "eager form; "
                "'nccl' (always measured, ms_per_step_nccl): per-owner broadcasts and an all-to-all; "
                "ms_per_step_sizes_exchanged_in_step (nccl): the sizes "
                "all-gathered and read back inside the step; ms_per_step_reduce_scatter: fp32 "
                "partial grad_documents reduce-scattered; single_gpu_ms_same_run: the whole problem "
                "on one GPU in this run (every rank times it, the slowest counts); all times max "
                "over ranks; rank 0's parity record is shown, parity_ok is the AND over ranks"}}


def _ops_status() -> int:
    from maxsim_b200 import _ops
    return _ops.device_status()


def bench_strong_scaling(dev, dist, rank, world, steps, weak_kernel_ms):
    """The 256-query rerank problem split over the ranks: rank r scores queries
    [r * 256 / N, (r + 1) * 256 / N) of the same global workload."""
    from maxsim_b200 import _ops
    from maxsim_b200 import workloads as W

    Nq, Lq, C, Ld, dim = (C3[k] for k in ("Nq", "Lq", "C", "Ld", "dim"))
    nq = Nq // world
    data = W.c3_device_shard(rank * nq, (rank + 1) * nq, dev, Lq=Lq, C=C, Ld=Ld, dim=dim)
    q_flat = data["queries"].view(nq * Lq, dim)
    d_flat = data["documents"].view(nq * C * Ld, dim)
    qlen, dlen = data["query_lengths"], data["doc_lengths"].view(-1).contiguous()

    def step():
        return _ops.ops.maxsim_padded_forward(q_flat, qlen, d_flat, dlen, Lq, Ld, C)

    for _ in range(5):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    del data, q_flat, d_flat
    torch.cuda.empty_cache()
    return {"workload": WORKLOAD, "pairs": Nq * C, "queries_per_gpu": nq, "ms_per_step": ms,
            "pairs_per_s": Nq * C / (ms * 1e-3), "single_gpu_ms_same_run": weak_kernel_ms,
            "speedup": weak_kernel_ms / ms, "efficiency": weak_kernel_ms / ms / world,
            "note": "one 256-query problem over all ranks, no collective; single_gpu_ms_same_run is "
                    "this run's launch time for 256 queries on one GPU (the weak-scaling shard, same "
                    "size and distributions); max over ranks"}


def run_contrastive_profile(args):
    """A few train steps of the contrastive-with-ties configuration, nothing
    else: the command a profiler wraps."""
    import maxsim_b200 as maxsim
    from maxsim_b200 import workloads as W

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n = 512 if args.small else 1024
    # --short-docs: 32-256 tokens per document, the range served by the kernel
    # whose tiles start at document starts; --lq / --dim: another query length or
    # dim (the general tcgen05 kernel instead of the Lq = 32, dim = 128 one)
    lo, hi = (32, 256) if args.short_docs else (64, 512)
    data = W.c5_device(dev, Nq=n, Nb=n, lo=lo, hi=hi, Lq=args.lq, dim=args.dim)
    q = data["queries"].requires_grad_(True)
    d = data["documents"].requires_grad_(True)
    off = data["document_offsets"]
    target = torch.arange(n, device=dev)
    for _ in range(max(1, args.warmup)):
        contrastive_train_step(maxsim, q, d, off, target)
    ms = _event_ms(lambda: contrastive_train_step(maxsim, q, d, off, target), max(1, args.steps))
    print(json.dumps({"profile_run": True, "workload": "c5_contrastive_ties_bf16", "Nq": n, "Nb": n,
                      "Lq": args.lq, "dim": args.dim, "doc_tokens": int(d.shape[0]),
                      "ms_per_step": statistics.median(ms)}), flush=True)


def run_packed_profile(args):
    """A few train steps (forward+argmax, backward) of the packed pair grid,
    nothing else: the command a profiler wraps."""
    import maxsim_b200 as maxsim
    from maxsim_b200 import workloads as W

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    maxsim._ops.set_pair_grouping(not args.list_order)
    wl = W.c4_packed_grid_fp16()
    q = W.to_torch(wl.queries, "fp16", dev).requires_grad_(True)
    d = W.to_torch(wl.documents, "fp16", dev).requires_grad_(True)
    qo = torch.from_numpy(wl.query_offsets).to(dev)
    do = torch.from_numpy(wl.document_offsets).to(dev)
    pq = torch.from_numpy(wl.pair_query_ids).to(dev)
    pd = torch.from_numpy(wl.pair_document_ids).to(dev)
    g = torch.from_numpy(wl.dscore).to(dev)

    def step():
        q.grad = None
        d.grad = None
        maxsim.score_pairs_packed_train(q, qo, d, do, pq, pd, max_q_len=32).backward(g)

    for _ in range(max(1, args.warmup)):
        step()
    ms = _event_ms(step, max(1, args.steps))
    print(json.dumps({"profile_run": True, "workload": "c4_packed_grid_fp16",
                      "pairs": int(pq.shape[0]), "order": "list" if args.list_order else "grouped",
                      "ms_per_step": statistics.median(ms)}), flush=True)


def run_gpu_arm(args):
    import maxsim_b200 as maxsim
    from maxsim_b200 import _ops
    from maxsim_b200 import workloads as W

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        # Collectives run beside persistent compute kernels that leave them a few SMs: keep
        # NCCL's kernels within those, on a high-priority stream
        from maxsim_b200 import dist as mdist
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        opts.config.max_ctas = mdist.COLLECTIVE_SMS
        opts.config.cga_cluster_size = 1  # single CTAs fit the scattered free SMs; clusters do not
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    peaks = _peaks()

    Nq, Lq, C, Ld, dim = (C3[k] for k in ("Nq", "Lq", "C", "Ld", "dim"))
    if args.small:
        Nq = 16
    q_begin = rank * Nq
    data = W.c3_device_shard(q_begin, q_begin + Nq, dev, Lq=Lq, C=C, Ld=Ld, dim=dim)
    queries, documents = data["queries"], data["documents"]
    qlen, dlen = data["query_lengths"], data["doc_lengths"]
    q_flat = queries.view(Nq * Lq, dim)
    d_flat = documents.view(Nq * C * Ld, dim)
    dlen_flat = dlen.view(-1).contiguous()
    pairs = Nq * C
    valid_doc_tokens = int(dlen.sum().item())
    valid_q_tokens = int(qlen.sum().item())
    algo_bytes = (valid_doc_tokens + valid_q_tokens) * dim * 2 + 4 * pairs

    sampler = ClockSampler(local_rank)
    sampler.start()
    load_begin = 0

    def step():
        return _ops.ops.maxsim_padded_forward(q_flat, qlen, d_flat, dlen_flat, Lq, Ld, C)

    # --- device-resident throughput -----------------------------------------
    load_begin = sampler.mark()
    t_warm = time.time()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    # The device comes to this point from seconds of host-side input generation.
    # Keep the kernel running for at least 60 ms before the timed steps so that
    # the clock ramp from the idle state (seen as one 10 ms launch among 2 ms
    # ones) does not land inside them; this is still far shorter than the
    # ~0.5 s after which the power cap lowers the clocks.
    while time.time() - t_warm < 0.06:
        step()
        torch.cuda.synchronize()
    if dist:
        dist.barrier()
    launches0 = _ops.launch_count()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    torch.cuda.synchronize()
    for i in range(args.steps):
        marks[i].record()
        scores = step()
    marks[args.steps].record()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    launches = _ops.launch_count() - launches0
    elapsed_ms = marks[0].elapsed_time(marks[args.steps])
    # per-launch durations for the roofline: the same launches, same stream
    launch_ms = [marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps)]
    kernel_ms = statistics.mean(launch_ms)

    if args.kernel_only:
        sampler.stop(load_begin)
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": WORKLOAD, "pairs": pairs,
                              "algorithmic_bytes": algo_bytes, "kernel_ms": kernel_ms,
                              "ms_per_step": elapsed_ms / args.steps}), flush=True)
        if dist:
            dist.destroy_process_group()
        return

    # --- the same kernel over at least half a second of back-to-back launches
    # (the power cap lowers the clocks after a few hundred milliseconds)
    burst_end = sampler.mark()
    n_sus = max(50, int(0.7 / max(kernel_ms * 1e-3, 1e-5)))
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(n_sus):
        step()
    s1.record()
    torch.cuda.synchronize()
    sustained_ms = s0.elapsed_time(s1) / n_sus
    sustained_end = sampler.mark()
    sustained_clocks = sampler.summary(burst_end, sustained_end)

    # --- end to end from host memory through the public API -----------------
    e2e_steps = max(1, min(args.steps, 3))
    # Host staging buffers: pinned when the box has the room for every rank's
    # 19.7 GB, pageable otherwise (recorded in the output).
    host_kind = "pinned"
    try:
        import psutil
        need = documents.numel() * 2 * max(1, world) * 1.25
        if psutil.virtual_memory().available < need:
            host_kind = "pageable"
    except Exception:
        pass

    def host_like(t):
        if host_kind == "pinned":
            try:
                return torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            except RuntimeError:
                pass
        return torch.empty(t.shape, dtype=t.dtype)

    hq = host_like(queries).copy_(queries)
    hd = host_like(documents)
    if not hd.is_pinned():
        host_kind = "pageable"
    hd.copy_(documents)
    hql = qlen.cpu()
    hdl = dlen.cpu()
    h_scores = host_like(torch.empty((Nq, C), dtype=torch.float32))

    valid_rows = host_kind == "pinned"

    def e2e_step():
        # the public call for a batch in host memory: queries and lengths are
        # copied, the documents' valid rows are read from the pinned buffer by a
        # kernel (padding never crosses PCIe), scores are copied back
        maxsim.score_candidates_padded_from_host(hq, hd, hql, hdl, device=dev,
                                                 staging=documents, out=h_scores)

    e2e_step()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    doc_bytes = (valid_doc_tokens * dim * 2) if valid_rows else hd.numel() * 2
    h2d = hq.numel() * 2 + doc_bytes + hql.numel() * 4 + hdl.numel() * 4
    d2h = h_scores.numel() * 4
    hq_bytes_padded = hq.numel() * 2 + hd.numel() * 2 + hql.numel() * 4 + hdl.numel() * 4
    del hd

    clocks = sampler.stop(load_begin)
    clocks["note"] = ("NVML samples every 50 ms from the start of warm-up through the timed burst, "
                      "the sustained window and the end-to-end steps")
    status = _ops.device_status()

    # --- max over ranks ------------------------------------------------------
    times = torch.tensor([elapsed_ms, e2e_ms, kernel_ms, sustained_ms], dtype=torch.float64, device=dev)
    if dist:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, kernel_ms, sustained_ms = (float(x) for x in times.tolist())

    train = None
    cpu_base = None
    ref_matrix = None
    strong = None
    del documents, d_flat, data
    torch.cuda.empty_cache()
    if world == 1:
        strong = {"workload": WORKLOAD, "pairs": pairs, "queries_per_gpu": Nq,
                  "ms_per_step": elapsed_ms / args.steps,
                  "pairs_per_s": pairs * args.steps / (elapsed_ms * 1e-3),
                  "single_gpu_ms_same_run": elapsed_ms / args.steps, "speedup": 1.0, "efficiency": 1.0,
                  "note": "one GPU: the strong-scaling problem is the headline shard"}
        train = bench_train_steps(dev, peaks, full=not args.small)
        ref_matrix = bench_reference_matrix(dev)
        v, cores, sample = cpu_padded_baseline(target_seconds=2.0 if args.small else 12.0)
        cpu_base = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    else:
        if not args.small:
            strong = bench_strong_scaling(dev, dist, rank, world, args.steps, elapsed_ms / args.steps)
        train = bench_sharded_train_step(dev, dist, rank, world, peaks, small=args.small)

    if rank == 0:
        value = world * pairs * args.steps / (elapsed_ms * 1e-3)
        achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
        sustained = algo_bytes / (sustained_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": c3_config(world, Nq),
            "timed_window": f"burst: {args.steps} launches right after a 60 ms warm-up, before the "
                            "power cap lowers the clocks; roofline.sustained is the same kernel over "
                            f"{n_sus} back-to-back launches",
            "e2e": {"value": world * pairs * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "host_memory": host_kind,
                    "padded_bytes_per_step": hq_bytes_padded,
                    "note": "score_candidates_padded_from_host: only the valid document rows of the "
                            "padded host batch cross PCIe (read by a kernel from pinned memory); "
                            "h2d_bytes_per_step counts the bytes that crossed, padded_bytes_per_step "
                            "what a whole-tensor copy would move"},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_source": peaks["source"],
                         "peak_note": "peak = the driver-measured copy bandwidth (read + write bytes of "
                                      "a device copy); a read-only stream can exceed it, so the "
                                      "fraction of the 8 TB/s data-sheet figure is given too",
                         "frac_of_datasheet_8tbs": achieved / 8000.0,
                         "kernel_ms": kernel_ms,
                         "kernel_ms_min_median_max": [min(launch_ms), statistics.median(launch_ms),
                                                      max(launch_ms)],
                         "kernel_ms_each": [round(x, 3) for x in launch_ms[:64]],
                         "algorithmic_bytes": algo_bytes,
                         "traffic": (None if NCU_TRAFFIC_RATIO is None
                                     else NCU_TRAFFIC_RATIO * algo_bytes),
                         "sustained": {"launches": n_sus, "seconds": n_sus * sustained_ms * 1e-3,
                                       "kernel_ms": sustained_ms, "achieved": sustained,
                                       "frac": sustained / peaks["hbm_gbs"],
                                       "frac_of_datasheet_8tbs": sustained / 8000.0,
                                       "clocks": sustained_clocks}},
            "clocks": clocks,
            "device_status": status,
        }
        if strong is not None:
            line["strong_scaling"] = strong
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        if ref_matrix is not None:
            line["reference_matrix"] = ref_matrix
        if train is not None:
            line["train_step"] = train
        # last key: the other configurations in short form
        summary = {"c3_rerank_hbm_frac_burst": round(achieved / peaks["hbm_gbs"], 3),
                   "c3_rerank_hbm_frac_sustained": round(sustained / peaks["hbm_gbs"], 3)}
        if strong is not None:
            summary["c3_strong_scaling_efficiency"] = round(strong["efficiency"], 3)
            summary["c3_strong_scaling_ms"] = round(strong["ms_per_step"], 4)
        if train is not None:
            for name, rec in train.items():
                if not isinstance(rec, dict):
                    continue
                short = {}
                for key in ("ms_per_step", "forward_ms", "tensor_frac", "forward_tensor_frac",
                            "forward_unique_doc_hbm_frac", "step_hbm_frac", "single_gpu_ms_same_run",
                            "efficiency", "transport", "ms_per_step_peer_eager", "efficiency_peer_eager",
                            "ms_per_step_nccl", "efficiency_nccl",
                            "efficiency_reduce_scatter", "ms_per_step_reduce_scatter",
                            "parity_ok", "ms"):
                    if key in rec:
                        v = rec[key]
                        short[key] = round(v, 4) if isinstance(v, float) else v
                if short:
                    summary[name] = short
        line["summary"] = summary
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def run_sharded_timeline(args):
    """Launched under torchrun on N GPUs: a few sharded contrastive train steps
    of the ties configuration under the torch profiler; rank 0 prints the
    device timeline of the last step (start and duration of every kernel and
    copy, microseconds) and every rank how long its barriers waited.  Not a
    bench value: the profiler slows the host side."""
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile

    from maxsim_b200 import dist as mdist
    from maxsim_b200 import workloads as W

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--timeline-sharded needs torchrun with at least two ranks")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
    opts.config.max_ctas = mdist.COLLECTIVE_SMS
    opts.config.cga_cluster_size = 1
    dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    n = 256 if args.small else 1024
    full = W.c5_device(dev, Nq=n, Nb=n)
    off = full["document_offsets"].cpu()
    lens_host = full["doc_lengths_all"].cpu()
    q0, q1 = mdist.shard_range(n, rank, world)
    q = full["queries"][q0:q1].clone().requires_grad_(True)
    d = full["documents"][int(off[q0]):int(off[q1])].clone().requires_grad_(True)
    lens = lens_host[q0:q1].to(dev)
    sizes = []
    for r in range(world):
        a0, a1 = mdist.shard_range(n, r, world)
        sizes.append((int(lens_host[a0:a1].sum()), a1 - a0, a1 - a0))
    target = mdist.contrastive_targets(q1 - q0, device=dev, docs_per_rank=[s[1] for s in sizes])
    peer = None
    if args.transport == "peer":
        from maxsim_b200.peer import PeerExchange
        peer = PeerExchange(max_doc_tokens=max(s[0] for s in sizes), max_docs=max(s[1] for s in sizes),
                            max_queries=max(s[2] for s in sizes), lq=q.shape[1], dim=q.shape[2],
                            dtype=q.dtype, wait_polls=1 << 21)
    records_group = dist.new_group(
        backend="nccl", pg_options=dist.ProcessGroupNCCL.Options(is_high_priority_stream=True))

    def step():
        q.grad = None
        d.grad = None
        s = mdist.score_contrastive_sharded(q, d, lens, shard_sizes=sizes, records_group=records_group,
                                            peer=peer)
        (torch.nn.functional.cross_entropy(s, target, reduction="sum") / n).backward()

    for _ in range(5):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
                     and not e.name.startswith("nccl:")), key=lambda e: e.time_range.start)
    per_step = len(events) // 3
    last = events[-per_step:]
    waits = [e.time_range.end - e.time_range.start for e in last if "peer_barrier" in e.name]
    for r in range(world):
        if r == rank:
            if rank == 0:
                base = last[0].time_range.start
                print(f"# {world} GPUs, transport {args.transport}, global Nq = Nb = {n}; rank 0, last of 3 "
                      "profiled steps; start us, duration us, kernel or copy", flush=True)
                for e in last:
                    print(f"{e.time_range.start - base:9.1f} {e.time_range.end - e.time_range.start:8.1f}  "
                          f"{e.name[:72]}", flush=True)
                print(f"# span {last[-1].time_range.end - base:.1f} us", flush=True)
            print(f"# rank {rank}: barrier kernels waited " + " ".join(f"{w:.0f}" for w in waits) + " us",
                  flush=True)
        dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="maxsim_b200", choices=["maxsim_b200", "reference"])
    ap.add_argument("--small", action="store_true",
                    help="16 queries per GPU instead of 256 (for profiler captures; not a bench value)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="run only the device-resident loop (for profiler captures)")
    ap.add_argument("--profile-contrastive", action="store_true",
                    help="run only contrastive forward+backward steps of the ties configuration "
                         "(Nq=Nb=1024, or 512 with --small); for profiler captures")
    ap.add_argument("--short-docs", action="store_true",
                    help="with --profile-contrastive: documents of 32-256 tokens instead of 64-512")
    ap.add_argument("--lq", type=int, default=32, help="with --profile-contrastive: query length")
    ap.add_argument("--dim", type=int, default=128, help="with --profile-contrastive: embedding dim")
    ap.add_argument("--profile-packed", action="store_true",
                    help="run only train steps of the packed pair grid (65536 pairs); for profiler captures")
    ap.add_argument("--list-order", action="store_true",
                    help="with --profile-packed: visit pairs in list order, atomic backward")
    ap.add_argument("--timeline-sharded", action="store_true",
                    help="under torchrun: print the device timeline of one sharded contrastive train "
                         "step (torch profiler; Nq=Nb=1024, or 256 with --small)")
    ap.add_argument("--transport", default="peer", choices=["peer", "nccl"],
                    help="with --timeline-sharded: how the shards and records travel")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.timeline_sharded:
        run_sharded_timeline(args)
    elif args.profile_contrastive:
        run_contrastive_profile(args)
    elif args.profile_packed:
        run_packed_profile(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
