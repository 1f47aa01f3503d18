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
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape
    tol = SCORE_TOL[dtype]
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin), f"{what}: finite pattern differs"
    scale = max(1.0, float(np.abs(want[fin]).max())) if fin.any() else 1.0
    err = np.abs(got[fin] - want[fin])
    # gradients are sums of up to hundreds of routed rows: the absolute term
    # scales with the largest magnitude so fp32 add-order noise is tolerated
    bound = tol["atol"] * scale + tol["rtol"] * np.abs(want[fin])
    bad = err > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance; max err {err.max():.3e}"
