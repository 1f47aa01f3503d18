"""Layout validation with the tensors on the GPU: the device-side statistics
kernel behind it, int32 and int64 index tensors, the error messages the
reference pins (tests/test_invalid_inputs.py, tests/test_ragged.py:64-106), and
the rule that a tensor is inspected again once it has been written to."""

from __future__ import annotations

import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops, _validate

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
def test_layout_stats_kernel(idt):
    off = torch.tensor([0, 3, 10, 11, 40], dtype=idt, device=DEV)
    ids = torch.tensor([5, 2, 9, 2], dtype=idt, device=DEV)
    rows = _ops.layout_stats([(off, None), (None, ids), (off, ids)])
    assert rows[0][:4] == [0, 40, 1, 29]
    assert rows[1][4:6] == [2, 9]
    assert rows[2][:6] == [0, 40, 1, 29, 2, 9]
    big = torch.arange(0, 3 * 100001, 3, dtype=idt, device=DEV)
    assert _ops.layout_stats([(big, None)])[0][:4] == [0, 300000, 3, 3]
    if idt == torch.int64:  # values past int32 survive
        wide = torch.tensor([0, 2 ** 33], dtype=idt, device=DEV)
        assert _ops.layout_stats([(wide, None)])[0][:4] == [0, 2 ** 33, 2 ** 33, 2 ** 33]


@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
def test_packed_errors_on_device(idt):
    q = torch.randn(13, 64, device=DEV, dtype=torch.float16)
    d = torch.randn(20, 64, device=DEV, dtype=torch.float16)
    qoff = torch.tensor([0, 5, 13], dtype=idt, device=DEV)
    doff = torch.tensor([0, 20], dtype=idt, device=DEV)
    pq = torch.tensor([1], dtype=idt, device=DEV)
    pd = torch.tensor([0], dtype=idt, device=DEV)
    assert maxsim.score_pairs_packed(q, qoff, d, doff, pq, pd).shape == (1,)
    with pytest.raises(RuntimeError, match=r"query_offsets\[0\] must equal 0, got 1"):
        maxsim.score_pairs_packed(q, torch.tensor([1, 5, 13], dtype=idt, device=DEV), d, doff, pq, pd)
    with pytest.raises(RuntimeError, match=r"\(12\) must equal total token count \(13\)"):
        maxsim.score_pairs_packed(q, torch.tensor([0, 5, 12], dtype=idt, device=DEV), d, doff, pq, pd)
    with pytest.raises(RuntimeError, match="empty segment in query_offsets at index 1"):
        maxsim.score_pairs_packed(q, torch.tensor([0, 5, 5, 13], dtype=idt, device=DEV), d, doff, pq, pd)
    with pytest.raises(RuntimeError, match=r"pair_query_ids\[0\] = 5 out of range \[0, 2\)"):
        maxsim.score_pairs_packed(q, qoff, d, doff, torch.tensor([5], dtype=idt, device=DEV), pd)
    with pytest.raises(RuntimeError, match=r"pair_document_ids\[0\] = -1 out of range"):
        maxsim.score_pairs_packed(q, qoff, d, doff, pq, torch.tensor([-1], dtype=idt, device=DEV))
    with pytest.raises(ValueError, match="max_q_len"):
        maxsim.score_pairs_packed_train(q, qoff, d, doff, pq, pd, max_q_len=5)


def test_padded_and_contrastive_errors_on_device():
    q = torch.randn(2, 16, 64, device=DEV, dtype=torch.float16)
    d = torch.randn(2, 3, 32, 64, device=DEV, dtype=torch.float16)
    qlen = torch.full((2,), 16, dtype=torch.int32, device=DEV)
    dlen = torch.full((2, 3), 32, dtype=torch.int32, device=DEV)
    for which, bad, msg in (("q", 0, "query_lengths"), ("q", 17, "query_lengths"),
                            ("d", 0, "doc_lengths"), ("d", 33, "doc_lengths")):
        ql, dl = qlen.clone(), dlen.clone()
        if which == "q":
            ql[0] = bad
        else:
            dl[0, 0] = bad
        with pytest.raises(ValueError, match=msg):
            maxsim.score_candidates_padded(q, d, ql, dl)
    docs = torch.randn(128, 64, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError, match="must equal 0"):
        maxsim.score_contrastive(q, docs, torch.tensor([1, 33, 65, 97, 128], dtype=torch.int32, device=DEV))
    with pytest.raises(ValueError, match=r"document_offsets\[2\] \(16\) <= document_offsets\[1\] \(32\)"):
        maxsim.score_contrastive(q, docs, torch.tensor([0, 32, 16, 96, 128], dtype=torch.int32, device=DEV))
    with pytest.raises(ValueError, match="total doc tokens"):
        maxsim.score_contrastive(q, docs, torch.tensor([0, 25, 50, 75, 100], dtype=torch.int32, device=DEV))
    with pytest.raises(RuntimeError, match="device"):
        maxsim.score_candidates_padded(q.cpu(), d, qlen, dlen)


def test_a_tensor_is_inspected_again_after_it_is_written():
    q = torch.randn(2, 16, 64, device=DEV, dtype=torch.float16)
    docs = torch.randn(128, 64, device=DEV, dtype=torch.float16)
    off = torch.tensor([0, 32, 64, 96, 128], dtype=torch.int32, device=DEV)
    a = maxsim.score_contrastive(q, docs, off)
    assert _validate._cache_get(off) is not None       # remembered while untouched
    assert torch.equal(a, maxsim.score_contrastive(q, docs, off))
    off[2] = 20                                        # in-place write bumps the version
    assert _validate._cache_get(off) is None
    with pytest.raises(ValueError, match="strictly increasing"):
        maxsim.score_contrastive(q, docs, off)
    fresh = torch.tensor([0, 32, 64, 96, 127], dtype=torch.int32, device=DEV)  # a new object is never trusted
    with pytest.raises(ValueError, match="total doc tokens"):
        maxsim.score_contrastive(q, docs, fresh)


def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_clean():
    """The kernels' waits are bounded: one that runs out sets a status bit the
    host can read.  The probe kernel waits on a barrier nothing arrives at (no
    copy or MMA is in flight, so giving up leaves nothing behind); the status
    word has to show the time-out once, and the operators have to work after."""
    import maxsim_b200 as maxsim
    from maxsim_b200 import _ops
    assert _ops.device_status() == 0
    assert _ops.wait_probe(polls=32) is True
    assert _ops.device_status() == 2          # the bounded-wait bit of the tensor-core kernels
    assert _ops.device_status() == 0          # reading clears it
    g = torch.Generator().manual_seed(0)
    q = torch.randn(16, 32, 128, generator=g).to("cuda", torch.bfloat16)
    d = torch.randn(400, 128, generator=g).to("cuda", torch.bfloat16)
    off = torch.tensor([0, 100, 250, 400], dtype=torch.int32, device="cuda")
    s, a = maxsim.score_contrastive_with_argmax(q, d, off)
    assert torch.isfinite(s).all() and _ops.device_status() == 0
