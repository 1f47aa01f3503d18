"""CPU checks of the packing / ranking oracle against the formulations the
reference's callers use (plain torch on the host), and of the host-side
argument checks of ``maxsim_b200.layout``."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from oracle import maxsim_oracle as oracle


def _mask_gather(padded: torch.Tensor, lengths: torch.Tensor):
    # torch-ext/maxsim/__init__.py:594-606 of the reference, on the host
    N, L = padded.shape[:2]
    mask = torch.arange(L)[None, :] < lengths[:, None]
    packed = padded.reshape((N * L,) + tuple(padded.shape[2:]))[mask.reshape(-1)]
    offsets = torch.zeros(N + 1, dtype=torch.int32)
    offsets[1:] = lengths.cumsum(0)
    return packed, offsets


@pytest.mark.parametrize("N,L,D", [(1, 1, 1), (7, 13, 5), (64, 300, 16)])
def test_oracle_pack_matches_mask_gather(N, L, D):
    g = torch.Generator().manual_seed(N * 1000 + L)
    padded = torch.randn(N, L, D, generator=g)
    lengths = torch.randint(1, L + 1, (N,), generator=g)
    want_p, want_o = _mask_gather(padded, lengths)
    got_p, got_o = oracle.pack_padded(padded.numpy(), lengths.numpy())
    np.testing.assert_array_equal(got_p, want_p.numpy())
    np.testing.assert_array_equal(got_o, want_o.numpy())
    back = oracle.unpack_packed(got_p, got_o, L)
    mask = (torch.arange(L)[None, :] < lengths[:, None]).numpy()
    np.testing.assert_array_equal(back, padded.numpy() * mask[:, :, None])


def test_oracle_rank_matches_stable_sort():
    g = torch.Generator().manual_seed(3)
    scores = torch.randn(9, 50, generator=g).round(decimals=1)  # many ties
    scores[2, 7] = float("inf")
    scores[3, 5] = float("-inf")
    want = torch.sort(scores, dim=1, descending=True, stable=True)
    vals, idx = oracle.rank_rows(scores.numpy(), 50)
    np.testing.assert_array_equal(idx, want.indices.numpy())
    np.testing.assert_array_equal(vals, want.values.numpy())
    vals, idx = oracle.rank_rows(scores.numpy(), 10)
    np.testing.assert_array_equal(idx, want.indices.numpy()[:, :10])


def test_oracle_rank_puts_nan_first():
    scores = np.array([[0.5, np.nan, 2.0, np.nan, -1.0]], dtype=np.float32)
    _, idx = oracle.rank_rows(scores, 5)
    assert idx.tolist() == [[1, 3, 2, 0, 4]]
    want = torch.sort(torch.from_numpy(scores), dim=1, descending=True, stable=True).indices
    assert idx.tolist() == want.tolist()


def test_layout_argument_checks_run_without_a_gpu():
    x = torch.zeros(4, 8, 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        maxsim.pack_padded(x, torch.tensor([1, 2, 3, 4]))
    with pytest.raises(ValueError, match="at least 2-D"):
        maxsim.pack_padded(torch.zeros(4), torch.tensor([1, 2, 3, 4]))
    with pytest.raises(ValueError, match="2-D"):
        maxsim.rerank_topk(torch.zeros(4), 1)
    with pytest.raises(ValueError, match="k must be"):
        maxsim.rerank_topk(torch.zeros(4, 3), 5)
