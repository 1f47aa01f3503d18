"""Shared helpers for the tests: oracle access, tolerances, comparisons.

Tolerances (stated by the benchmark definition this repository is built to):
argmax bit-exact except where the oracle's two best similarities differ by
less than 1e-6 (fp32) or 1e-3 (fp16/bf16); scores and gradients within 1e-5
relative (fp32) or 2e-2 relative / 1e-2 absolute (fp16/bf16).
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import maxsim_oracle as oracle  # noqa: E402

GOLDEN = ROOT / "tests" / "golden" / "reference_outputs.npz"

TORCH_DTYPE = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
NAME_OF = {v: k for k, v in TORCH_DTYPE.items()}

SCORE_TOL = {
    "fp32": dict(rtol=1e-5, atol=1e-5),
    "fp16": dict(rtol=2e-2, atol=1e-2),
    "bf16": dict(rtol=2e-2, atol=1e-2),
}
GAP_TOL = {"fp32": 1e-6, "fp16": 1e-3, "bf16": 1e-3}


def f32(t: torch.Tensor) -> np.ndarray:
    """Device tensor -> float32 numpy on the host."""
    return t.detach().float().cpu().numpy()


def i64(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy().astype(np.int64)


def assert_scores(got, want, dtype: str, what="scores"):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    tol = SCORE_TOL[dtype]
    # non-finite entries must match exactly (same sign of infinity, NaN where NaN)
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin), f"{what}: finite pattern differs"
    assert np.array_equal(got[~fin], want[~fin], equal_nan=True), f"{what}: non-finite values differ"
    err = np.abs(got[fin] - want[fin])
    bound = tol["atol"] + tol["rtol"] * np.abs(want[fin])
    bad = err > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} outside tolerance; "
                           f"max err {err.max():.3e}")


def assert_argmax(got, want, gaps, dtype: str, valid=None, what="argmax"):
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    ok = oracle.argmax_mismatch_allowed(got, want, gaps, GAP_TOL[dtype])
    if valid is not None:
        ok = ok | ~valid
    assert ok.all(), (f"{what}: {(~ok).sum()} of {ok.size} entries differ where the oracle's "
                      f"top-2 gap is >= {GAP_TOL[dtype]}")
    return int((got != want).sum())


def assert_grads(got, want, dtype: str, what="grad"):
    """Gradients against the oracle at the stated tolerance (2e-2 relative /
    1e-2 absolute for fp16 / bf16, 1e-5 / 1e-5 for fp32), element by element."""
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape
    tol = SCORE_TOL[dtype]
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin), f"{what}: finite pattern differs"
    err = np.abs(got[fin] - want[fin])
    bound = tol["atol"] + tol["rtol"] * np.abs(want[fin])
    if dtype == "fp32":
        # sums of hundreds of fp32 products in a different order than the oracle's float64:
        # the absolute term follows the magnitude of the sums
        bound = bound + 1e-6 * (float(np.abs(want[fin]).max()) if fin.any() else 0.0)
    bad = err > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance; max err {err.max():.3e}"

# ---------------------------------------------------------------------------
# fp32 einsum checker on the GPU (tests only): the reference's formulation,
# sim = einsum, mask, max over document tokens, sum over query tokens, written
# with torch ops in fp32 and chunked so that the similarity tensor fits.  It
# checks EVERY pair of the full-size configurations, where the CPU oracle would
# take hours.  Ties go to the first index (min over the positions of the
# maximum), as the oracle does.
# ---------------------------------------------------------------------------

def _fold_similarities(sim: torch.Tensor, valid: torch.Tensor):
    """sim [..., L] fp32, valid [..., L] bool (broadcastable) -> (max, first
    index of the max, gap between the two best) over the last axis."""
    sim = sim.masked_fill(~valid, float("-inf"))
    top = torch.topk(sim, k=min(2, sim.shape[-1]), dim=-1).values
    best = top[..., 0]
    gap = (best - top[..., 1]) if top.shape[-1] > 1 else torch.full_like(best, float("inf"))
    gap = torch.where(torch.isfinite(top[..., -1]), gap, torch.full_like(gap, float("inf")))
    pos = torch.arange(sim.shape[-1], device=sim.device)
    first = torch.where(sim == best[..., None], pos, sim.shape[-1]).amin(dim=-1)
    return best, first.to(torch.int32), gap


def gpu_einsum_padded(q, d, qlen, dlen, chunk=2):
    """q [B, Lq, D], d [B, C, Ld, D] on the GPU -> (scores [B, C] fp32,
    argmax [B, C, Lq] int32 with 0 past the query length, gaps [B, C, Lq])."""
    B, C, Ld, _ = d.shape
    Lq = q.shape[1]
    scores = torch.empty((B, C), dtype=torch.float32, device=q.device)
    argmax = torch.empty((B, C, Lq), dtype=torch.int32, device=q.device)
    gaps = torch.empty((B, C, Lq), dtype=torch.float32, device=q.device)
    jpos = torch.arange(Ld, device=q.device)
    ipos = torch.arange(Lq, device=q.device)
    for b0 in range(0, B, chunk):
        b1 = min(B, b0 + chunk)
        sim = torch.einsum("bid,bcjd->bcij", q[b0:b1].float(), d[b0:b1].float())
        valid = (jpos[None, None, None, :] < dlen[b0:b1, :, None, None])
        best, first, gap = _fold_similarities(sim, valid)
        qok = ipos[None, None, :] < qlen[b0:b1, None, None]
        scores[b0:b1] = torch.where(qok, best, torch.zeros_like(best)).sum(dim=-1)
        argmax[b0:b1] = torch.where(qok, first, torch.zeros_like(first))
        gaps[b0:b1] = torch.where(qok, gap, torch.full_like(gap, float("inf")))
    return scores, argmax, gaps


def gpu_einsum_contrastive(q, d, offsets, q_chunk=32):
    """q [Nq, Lq, D], packed d [T, D], offsets [Nb + 1] on the GPU -> (scores
    [Nq, Nb] fp32, argmax [Nq, Nb, Lq] int32, gaps [Nq, Nb, Lq])."""
    Nq, Lq, D = q.shape
    off = offsets.to(torch.int64)
    lens = off[1:] - off[:-1]
    Nb, Lmax = lens.numel(), int(lens.max())
    jpos = torch.arange(Lmax, device=q.device)
    valid = jpos[None, :] < lens[:, None]                              # [Nb, Lmax]
    rows = (off[:-1, None] + jpos[None, :]).clamp(max=d.shape[0] - 1)  # [Nb, Lmax]
    dp = d.float()[rows]                                               # [Nb, Lmax, D]
    scores = torch.empty((Nq, Nb), dtype=torch.float32, device=q.device)
    argmax = torch.empty((Nq, Nb, Lq), dtype=torch.int32, device=q.device)
    gaps = torch.empty((Nq, Nb, Lq), dtype=torch.float32, device=q.device)
    for q0 in range(0, Nq, q_chunk):
        q1 = min(Nq, q0 + q_chunk)
        sim = torch.einsum("qid,njd->qnij", q[q0:q1].float(), dp)
        best, first, gap = _fold_similarities(sim, valid[None, :, None, :])
        scores[q0:q1] = best.sum(dim=-1)
        argmax[q0:q1] = first
        gaps[q0:q1] = gap
    return scores, argmax, gaps


def assert_all_pairs(scores, argmax, want_scores, want_argmax, gaps, dtype: str):
    """Device-side comparison of every pair: scores within the tolerance of
    `dtype`, argmax equal wherever the checker's two best differ by at least
    the stated gap.  Returns the number of (exempt) argmax differences."""
    tol = SCORE_TOL[dtype]
    err = (scores - want_scores).abs()
    bound = tol["atol"] + tol["rtol"] * want_scores.abs()
    assert bool((err <= bound).all()), f"scores: max err {float(err.max()):.3e}"
    differ = argmax != want_argmax
    bad = differ & (gaps >= GAP_TOL[dtype])
    assert not bool(bad.any()), f"argmax: {int(bad.sum())} entries differ outside the tie exemption"
    return int(differ.sum()), float(err.max())
