"""Host-side checks that need no GPU: validation (exception types and message
fragments pinned by the reference's tests/test_invalid_inputs.py and
tests/test_ragged.py:64-106), the C-ABI library's exported symbols, and the
loud failure when a tensor is not on a CUDA device."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _build, _ops

ROOT = Path(__file__).resolve().parent.parent


def _padded(B=2, C=3, Lq=16, Ld=32, dim=64, dtype=torch.float16):
    q = torch.randn(B, Lq, dim).to(dtype)
    d = torch.randn(B, C, Ld, dim).to(dtype)
    return q, d, torch.full((B,), Lq, dtype=torch.int32), torch.full((B, C), Ld, dtype=torch.int32)


PADDED_ENTRIES = [maxsim.score_candidates_padded, maxsim.score_candidates_padded_with_argmax,
                  maxsim.score_candidates_padded_train]
PACKED_ENTRIES = [maxsim.score_pairs_packed, maxsim.score_pairs_packed_with_argmax,
                  maxsim.score_pairs_packed_train]
CONTRASTIVE_ENTRIES = [maxsim.score_contrastive, maxsim.score_contrastive_with_argmax,
                       maxsim.score_contrastive_train]


@pytest.mark.parametrize("entry", PADDED_ENTRIES)
def test_padded_validation(entry):
    q, d, qlen, dlen = _padded()
    with pytest.raises(ValueError, match="dim|D"):
        entry(q, torch.randn(2, 3, 32, 32).half(), qlen, dlen)
    with pytest.raises(TypeError, match="same dtype"):
        entry(q, d.to(torch.bfloat16), qlen, dlen)
    with pytest.raises(TypeError, match="float|dtype"):
        entry(torch.randint(0, 5, (2, 16, 64), dtype=torch.int32), d.to(torch.int32), qlen, dlen)
    with pytest.raises(ValueError, match="doc_lengths"):
        entry(q, d, qlen, dlen[:, :2])
    with pytest.raises(ValueError, match="3-D"):
        entry(q[0], d, qlen, dlen)
    with pytest.raises(ValueError, match="4-D"):
        entry(q, d[0], qlen, dlen)
    with pytest.raises(TypeError, match="int32 or int64"):
        entry(q, d, qlen.float(), dlen)
    for bad, msg in (("q0", "query_lengths"), ("q+", "query_lengths"),
                     ("d0", "doc_lengths"), ("d+", "doc_lengths")):
        ql, dl = qlen.clone(), dlen.clone()
        if bad == "q0":
            ql[0] = 0
        elif bad == "q+":
            ql[0] = q.shape[1] + 1
        elif bad == "d0":
            dl[0, 0] = 0
        else:
            dl[0, 0] = d.shape[2] + 1
        with pytest.raises(ValueError, match=msg):
            entry(q, d, ql, dl)


def _packed():
    q = torch.randn(13, 64).half()
    d = torch.randn(20, 64).half()
    return (q, torch.tensor([0, 5, 13], dtype=torch.int32), d,
            torch.tensor([0, 20], dtype=torch.int32),
            torch.tensor([1], dtype=torch.int32), torch.tensor([0], dtype=torch.int32))


@pytest.mark.parametrize("entry", PACKED_ENTRIES)
def test_packed_validation(entry):
    q, qoff, d, doff, pq, pd = _packed()
    with pytest.raises(ValueError, match="dim|match"):
        entry(q, qoff, torch.randn(20, 32).half(), doff, pq, pd)
    with pytest.raises(TypeError, match="dtype"):
        entry(q, qoff, d.float(), doff, pq, pd)
    with pytest.raises(RuntimeError, match=r"\[0\] must equal 0"):
        entry(q, torch.tensor([1, 5, 13], dtype=torch.int32), d, doff, pq, pd)
    with pytest.raises(RuntimeError, match="must equal total token count"):
        entry(q, torch.tensor([0, 5, 12], dtype=torch.int32), d, doff, pq, pd)
    with pytest.raises(RuntimeError, match="empty segment in query_offsets at index 1"):
        entry(q, torch.tensor([0, 5, 5, 13], dtype=torch.int32), d, doff, pq, pd)
    with pytest.raises(RuntimeError, match=r"pair_query_ids\[0\] = 5 out of range \[0, 2\)"):
        entry(q, qoff, d, doff, torch.tensor([5], dtype=torch.int32), pd)
    with pytest.raises(RuntimeError, match="out of range"):
        entry(q, qoff, d, doff, pq, torch.tensor([-1], dtype=torch.int32))
    with pytest.raises(ValueError, match="max_q_len"):
        entry(q, qoff, d, doff, pq, pd, max_q_len=5)
    with pytest.raises(ValueError, match="max_q_len must be > 0"):
        entry(q, qoff, d, doff, pq, pd, max_q_len=0)
    with pytest.raises(ValueError, match="same shape"):
        entry(q, qoff, d, doff, pq, torch.tensor([0, 0], dtype=torch.int32))
    with pytest.raises(RuntimeError, match="length >= 2"):
        entry(q, torch.tensor([0], dtype=torch.int32), d, doff, pq, pd)


def test_packed_score_only_wording():
    q, qoff, d, doff, pq, pd = _packed()
    with pytest.raises(TypeError, match="same dtype"):
        maxsim.score_pairs_packed(q, qoff, d.float(), doff, pq, pd)
    with pytest.raises(ValueError, match="dim"):
        maxsim.score_pairs_packed(q, qoff, torch.randn(20, 16).half(), doff, pq, pd)


@pytest.mark.parametrize("entry", CONTRASTIVE_ENTRIES)
def test_contrastive_validation(entry):
    q = torch.randn(2, 16, 64).half()
    d = torch.randn(128, 64).half()
    off = torch.arange(0, 160, 32, dtype=torch.int32)
    with pytest.raises(ValueError, match="Nq, Lq"):
        entry(torch.randn(2, 16, 64, 4).half(), d, off)
    with pytest.raises(ValueError, match="packed"):
        entry(q, torch.randn(64, 64, 4).half(), off)
    with pytest.raises(ValueError, match="must match"):
        entry(q, torch.randn(128, 65).half(), off)
    with pytest.raises(TypeError, match="share dtype"):
        entry(q, d.to(torch.bfloat16), off)
    with pytest.raises(ValueError, match="must equal 0"):
        entry(q, d, off + 1)
    with pytest.raises(ValueError, match="strictly increasing"):
        entry(q, d, torch.tensor([0, 32, 16, 96, 128], dtype=torch.int32))
    with pytest.raises(ValueError, match="strictly"):
        entry(q, d, torch.tensor([0, 0, 128], dtype=torch.int32))
    with pytest.raises(ValueError, match="total"):
        entry(q, d, torch.tensor([0, 25, 50, 75, 100], dtype=torch.int32))
    with pytest.raises(ValueError, match="Lq"):
        entry(q[:, :0], d, off)
    with pytest.raises(ValueError, match="dim"):
        entry(q[:, :, :0], d[:, :0], off)
    with pytest.raises(ValueError, match="length >= 2"):
        entry(q, d, off[:1])
    with pytest.raises(TypeError, match="int32 or int64"):
        entry(q, d, off.float())


def test_no_cpu_fallback():
    q, d, qlen, dlen = _padded()
    with pytest.raises(RuntimeError, match="CUDA"):
        maxsim.score_candidates_padded(q, d, qlen, dlen)
    with pytest.raises(RuntimeError, match="CUDA"):
        maxsim.score_contrastive(torch.randn(2, 16, 64).half(), torch.randn(64, 64).half(),
                                 torch.tensor([0, 32, 64], dtype=torch.int32))


def test_prefix_mask_helper():
    m = torch.tensor([[True, True, False], [True, False, False]])
    assert maxsim.lengths_from_prefix_mask(m).tolist() == [2, 1]
    with pytest.raises(ValueError, match="prefix"):
        maxsim.lengths_from_prefix_mask(torch.tensor([[True, False, True]]))


def _declared_symbols():
    text = (ROOT / "include" / "maxsim_b200.h").read_text()
    return re.findall(r"MAXSIM_API\s+[\w\s\*]+?\b(maxsim_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 14 and "maxsim_contrastive_forward_with_argmax" in names
    _build.build()
    lib = ctypes.CDLL(str(_build.LIB_PATH))
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/maxsim_b200.h but not exported"
    assert set(names) == set(_ops.EXPORTED_SYMBOLS), "ctypes table and header disagree"
    lib.maxsim_b200_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.maxsim_b200_version()


def test_ops_namespace_matches_reference_operator_names():
    expected = {
        "maxsim_forward", "maxsim_padded_forward", "maxsim_padded_forward_with_argmax",
        "maxsim_padded_backward", "maxsim_packed_forward_with_argmax", "maxsim_packed_backward",
        "maxsim_contrastive_forward", "maxsim_contrastive_forward_with_argmax",
        "maxsim_contrastive_backward",
    }
    assert expected == set(vars(_ops.ops))


def test_reference_python_layer_runs_on_this_ops_namespace():
    """The reference's own maxsim/__init__.py imports and dispatches into this
    package's operator namespace when it is installed as maxsim._ops, the one
    seam through which the reference reaches its compiled kernels.  Needs a
    checkout of the reference next to this repository (or in
    $MAXSIM_REFERENCE_DIR); skipped without one."""
    import importlib
    import sys
    import types

    import os
    ref = Path(os.environ.get("MAXSIM_REFERENCE_DIR",
                              Path(__file__).resolve().parents[2] / "reference")) / "torch-ext"
    if not (ref / "maxsim" / "__init__.py").exists():
        pytest.skip("reference checkout not present")
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "maxsim" or k.startswith("maxsim.")}
    shim = types.ModuleType("maxsim._ops")
    shim.ops = _ops.ops
    sys.modules["maxsim._ops"] = shim
    sys.path.insert(0, str(ref))
    try:
        ref_maxsim = importlib.import_module("maxsim")
        for name in ("score_pairs_packed", "score_candidates_padded_train", "score_contrastive_with_argmax"):
            assert hasattr(ref_maxsim, name)
        q, d, qlen, dlen = _padded()
        with pytest.raises(RuntimeError, match="CUDA"):  # reached our operator, which has no CPU path
            ref_maxsim.score_candidates_padded(q, d, qlen, dlen)
    finally:
        sys.path.remove(str(ref))
        for k in [k for k in sys.modules if k == "maxsim" or k.startswith("maxsim.")]:
            del sys.modules[k]
        sys.modules.update(saved)
