"""Regenerates the golden fixtures in this directory.

Runs the REFERENCE's own pure-PyTorch implementation
(``torch-ext/maxsim/reference.py`` in the reference checkout, loaded by file
path so that its package ``__init__`` -- which needs compiled ops -- is not
imported) on seeded inputs from ``maxsim_b200.workloads`` and stores its
outputs.  The reference checkout only exists on the development machine; the
fixtures travel, this script documents how they were made.

    python tests/golden/make_golden.py /path/to/reference-checkout
"""

from __future__ import annotations

import hashlib
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from maxsim_b200 import workloads as W  # noqa: E402


def load_reference(root: Path):
    path = root / "torch-ext" / "maxsim" / "reference.py"
    spec = importlib.util.spec_from_file_location("maxsim_reference_impl", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def t(x, dtype):
    return W.to_torch(x, dtype)


def i32(x):
    return torch.from_numpy(np.ascontiguousarray(x).astype(np.int32))


def padded_case(ref, wl: W.PaddedWorkload, seed_g: int):
    q, d = t(wl.queries, wl.dtype), t(wl.documents, wl.dtype)
    ql, dl = i32(wl.query_lengths), i32(wl.doc_lengths)
    s, a = ref.score_candidates_padded_with_argmax_reference(q, d, ql, dl)
    s2 = ref.score_candidates_padded_reference(q, d, ql, dl)
    assert torch.equal(s, s2)
    g = torch.from_numpy(np.random.default_rng(seed_g).standard_normal(s.shape, dtype=np.float32))
    dq, dd = ref.score_candidates_padded_backward_reference(g, q, d, ql, dl, a)
    return dict(scores=s.numpy(), argmax=a.numpy(), dscore=g.numpy(), dq=dq.numpy(), dd=dd.numpy())


def contrastive_case(ref, wl: W.ContrastiveWorkload, seed_g: int, with_backward=True):
    q, d = t(wl.queries, wl.dtype), t(wl.documents, wl.dtype)
    off = i32(wl.document_offsets)
    s, a = ref.score_contrastive_with_argmax_reference(q, d, off)
    out = dict(scores=s.numpy(), argmax=a.numpy())
    if with_backward:
        g = torch.from_numpy(np.random.default_rng(seed_g).standard_normal(s.shape, dtype=np.float32))
        dq, dd = ref.score_contrastive_backward_reference(g, q, d, off, a)
        out.update(dscore=g.numpy(), dq=dq.numpy(), dd=dd.numpy())
    return out


def packed_case(ref, wl: W.PackedWorkload):
    q, d = t(wl.queries, wl.dtype), t(wl.documents, wl.dtype)
    qo, do = i32(wl.query_offsets), i32(wl.document_offsets)
    pq, pd = i32(wl.pair_query_ids), i32(wl.pair_document_ids)
    mql = int(np.diff(wl.query_offsets).max())
    s, a = ref.score_pairs_packed_with_argmax_reference(q, qo, d, do, pq, pd, mql)
    s2 = ref.score_pairs_packed_reference(q, qo, d, do, pq, pd)
    assert torch.equal(s, s2)
    g = torch.from_numpy(wl.dscore)
    dq, dd = ref.score_pairs_packed_backward_reference(g, q, qo, d, do, pq, pd, a)
    return dict(scores=s.numpy(), argmax=a.numpy(), dq=dq.numpy(), dd=dd.numpy())


def main(root: Path):
    ref = load_reference(root)
    out = {}

    # --- small cases, one per layout and dtype, with backward -----------------
    for dtype in ("fp32", "fp16", "bf16"):
        wl = W.c1_padded_rerank_fp32(seed=10, Nq=3, Lq=12, C=4, Ld=40, dim=32, lo=1)
        wl.dtype = dtype
        wl.query_lengths = np.array([12, 7, 1], dtype=np.int32)
        for k, v in padded_case(ref, wl, 100).items():
            out[f"padded_small_{dtype}/{k}"] = v
        wl = W.c2_contrastive_train_bf16(seed=11, Nq=5, Nb=6, Lq=16, dim=64, lo=1, hi=70, dtype=dtype)
        for k, v in contrastive_case(ref, wl, 101).items():
            out[f"contrastive_small_{dtype}/{k}"] = v
        wl = W.c4_packed_grid_fp16(seed=12, n_queries=7, n_docs=9, n_pairs=40, dim=96)
        wl.dtype = dtype
        for k, v in packed_case(ref, wl).items():
            out[f"packed_small_{dtype}/{k}"] = v

    # --- ties: contrastive with duplicated tokens, scaled down -----------------
    wl = W.c5_contrastive_ties_bf16(seed=13, Nq=6, Nb=8, Lq=32, dim=128, lo=20, hi=90, dup_frac=0.2)
    for k, v in contrastive_case(ref, wl, 102).items():
        out[f"contrastive_ties_bf16/{k}"] = v

    # --- configuration 1 at full size (fp32 padded rerank) --------------------
    wl = W.c1_padded_rerank_fp32()
    q, d = t(wl.queries, "fp32"), t(wl.documents, "fp32")
    s, a = ref.score_candidates_padded_with_argmax_reference(
        q, d, i32(wl.query_lengths), i32(wl.doc_lengths))
    out["c1/scores"] = s.numpy()
    out["c1/argmax"] = a.numpy().astype(np.int16)
    out["c1/input_digest"] = np.frombuffer(
        digest(wl.queries, wl.documents, wl.doc_lengths).encode(), dtype=np.uint8)

    # --- configuration 2 at full size (bf16 contrastive), forward only --------
    wl = W.c2_contrastive_train_bf16()
    res = contrastive_case(ref, wl, 0, with_backward=False)
    out["c2/scores"] = res["scores"]
    out["c2/argmax"] = res["argmax"].astype(np.int16)
    out["c2/input_digest"] = np.frombuffer(
        digest(wl.queries, wl.documents, wl.document_offsets).encode(), dtype=np.uint8)

    np.savez_compressed(HERE / "reference_outputs.npz", **out)
    total = sum(v.nbytes for v in out.values())
    print(f"wrote {len(out)} arrays, {total/1e6:.2f} MB raw ->",
          (HERE / "reference_outputs.npz").stat().st_size / 1e6, "MB")


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else HERE.parents[2] / "reference")
