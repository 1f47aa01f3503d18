"""Gradients written by the kernels in the inputs' 16-bit type: they must be
the fp32 operators' gradients rounded once (what autograd's cast produces),
and shapes outside the covered range must fall back to the fp32 operators."""

from __future__ import annotations

import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _defaults():
    _ops.set_native_gradients(True)
    yield
    _ops.set_native_gradients(True)
    assert _ops.device_status() == 0


def _padded(B, C, Lq, Ld, dim, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Lq, dim, generator=g).to(DEV, dtype)
    d = torch.randn(B, C, Ld, dim, generator=g).to(DEV, dtype)
    # duplicated document tokens make several query tokens win the same row
    d[:, :, 1::7] = d[:, :, 0:1]
    ql = torch.randint(1, Lq + 1, (B,), generator=g, dtype=torch.int32).to(DEV)
    dl = torch.randint(1, Ld + 1, (B, C), generator=g, dtype=torch.int32).to(DEV)
    w = torch.randn(B, C, generator=g).to(DEV)
    return q, d, ql, dl, w


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,C,Lq,Ld,dim", [(3, 5, 32, 120, 128), (2, 2, 9, 33, 64), (1, 4, 16, 1024, 96),
                                           (4, 7, 32, 300, 128), (1, 1, 1, 1, 8)])
def test_padded_native_gradients_are_the_fp32_gradients_rounded_once(B, C, Lq, Ld, dim, dtype):
    q, d, ql, dl, w = _padded(B, C, Lq, Ld, dim, dtype, seed=B * 100 + Ld)
    _, a = maxsim.score_candidates_padded_with_argmax(q, d, ql, dl)
    args = (w.reshape(-1), q.reshape(B * Lq, dim), d.reshape(B * C * Ld, dim), ql, dl.reshape(-1),
            a.reshape(B * C, Lq), Lq, Ld, C)
    native = _ops.padded_backward_native(*args)
    assert native is not None
    dq32, dd32 = _ops.ops.maxsim_padded_backward(*args)
    assert native[0].dtype == dtype and native[1].dtype == dtype
    assert torch.equal(native[0], dq32.to(dtype))
    assert torch.equal(native[1], dd32.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Nq,Lq,d_lens,dim", [(4, 32, [50, 50, 50, 50], 128), (6, 32, [1, 65, 64, 130, 300], 128),
                                              (3, 20, [33, 5], 96), (9, 32, [2500, 40], 128),
                                              (1024, 32, [70, 9], 128)])
def test_contrastive_native_gradients_are_the_fp32_gradients_rounded_once(Nq, Lq, d_lens, dim, dtype):
    g = torch.Generator().manual_seed(Nq + len(d_lens))
    q = torch.randn(Nq, Lq, dim, generator=g).to(DEV, dtype)
    d = torch.randn(sum(d_lens), dim, generator=g).to(DEV, dtype)
    off = torch.zeros(len(d_lens) + 1, dtype=torch.int32)
    off[1:] = torch.tensor(d_lens, dtype=torch.int32).cumsum(0)
    off = off.to(DEV)
    w = torch.randn(Nq, len(d_lens), generator=g).to(DEV)
    _, a = maxsim.score_contrastive_with_argmax(q, d, off)
    native = _ops.contrastive_backward_native(w, q, d, off, a)
    assert native is not None
    dq32, dd32 = _ops.ops.maxsim_contrastive_backward(w, q, d, off, a)
    assert torch.equal(native[0], dq32.to(dtype))
    # grad_documents: the order in which a token's routed rows are summed is set
    # by shared-memory atomics and differs from launch to launch, so the fp32
    # sums agree to rounding and the 16-bit values to one unit in the last place
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    torch.testing.assert_close(native[1].float(), dd32.to(dtype).float(), rtol=2 * ulp, atol=1e-4)


def test_shapes_outside_the_range_fall_back_to_the_fp32_operators():
    q, d, ql, dl, w = _padded(2, 3, 40, 50, 128, torch.float16, 1)          # Lq_max > 32
    _, a = maxsim.score_candidates_padded_with_argmax(q, d, ql, dl)
    assert _ops.padded_backward_native(w.reshape(-1), q.reshape(80, 128), d.reshape(300, 128), ql,
                                       dl.reshape(-1), a.reshape(6, 40), 40, 50, 3) is None
    q32 = torch.randn(2, 16, 64, device=DEV)                                   # fp32 inputs
    assert _ops.contrastive_backward_native(torch.zeros(2, 1, device=DEV), q32,
                                            torch.randn(5, 64, device=DEV),
                                            torch.tensor([0, 5], dtype=torch.int32, device=DEV),
                                            torch.zeros(2, 1, 16, dtype=torch.int32, device=DEV)) is None
    # more (query, token) entries per document than one pass holds
    qb = torch.randn(1100, 32, 128, device=DEV).half()
    db = torch.randn(40, 128, device=DEV).half()
    off = torch.tensor([0, 40], dtype=torch.int32, device=DEV)
    _, ab = maxsim.score_contrastive_with_argmax(qb, db, off)
    assert _ops.contrastive_backward_native(torch.ones(1100, 1, device=DEV), qb, db, off, ab) is None
    # ... and autograd still delivers leaf-dtype gradients through the fp32 path
    qb.requires_grad_(True)
    db.requires_grad_(True)
    maxsim.score_contrastive_train(qb, db, off).sum().backward()
    assert qb.grad.dtype == torch.float16 and db.grad.dtype == torch.float16


@pytest.mark.parametrize("api", ["padded", "contrastive", "loss"])
def test_autograd_results_do_not_depend_on_the_switch(api):
    torch.manual_seed(3)
    grads = []
    for native in (True, False):
        _ops.set_native_gradients(native)
        if api == "padded":
            q, d, ql, dl, w = _padded(3, 4, 32, 90, 128, torch.bfloat16, 7)
            q.requires_grad_(True); d.requires_grad_(True)
            (maxsim.score_candidates_padded_train(q, d, ql, dl) * w).sum().backward()
        else:
            g = torch.Generator().manual_seed(5)
            q = torch.randn(8, 32, 128, generator=g).to(DEV, torch.bfloat16).requires_grad_(True)
            d = torch.randn(400, 128, generator=g).to(DEV, torch.bfloat16).requires_grad_(True)
            off = torch.tensor([0, 100, 130, 260, 400], dtype=torch.int32, device=DEV)
            if api == "contrastive":
                w = torch.randn(8, 4, generator=g).to(DEV)
                (maxsim.score_contrastive_train(q, d, off) * w).sum().backward()
            else:
                maxsim.contrastive_loss(q, d, off, torch.arange(8, device=DEV) % 4, temperature=0.3).backward()
        grads.append((q.grad.clone(), d.grad.clone()))
    assert torch.equal(grads[0][0], grads[1][0])
    if api == "padded":
        assert torch.equal(grads[0][1], grads[1][1])
    else:  # summation order of grad_documents varies between launches (see above)
        torch.testing.assert_close(grads[0][1].float(), grads[1][1].float(), rtol=2.0 ** -6, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n_pairs,n_docs,n_queries,dim", [(4096, 300, 80, 96), (3000, 7, 40, 128),
                                                         (2048, 2000, 3, 64), (20000, 11, 11, 32)])
def test_packed_native_gradients_match_the_fp32_operator(n_pairs, n_docs, n_queries, dim, dtype):
    """Grouped pair lists: both gradients in the leaf dtype, every row summed in
    fp32 and stored once.  grad_queries is the fp32 operator's result rounded
    once (same kernel, same order); grad_documents sums in pair-list order
    instead of the operator's read-modify-write order, so it may differ in the
    last place; few documents with many pairs (7 or 11 documents for thousands
    of pairs) exercise the batches of 512 terms, and both launches of the same
    call must give the same bits."""
    from maxsim_b200 import workloads as W
    from _util import assert_grads, f32, oracle
    name = "fp16" if dtype == torch.float16 else "bf16"
    wl = W.c4_packed_grid_fp16(seed=n_pairs % 97, n_queries=n_queries, n_docs=n_docs,
                               n_pairs=n_pairs, dim=dim)
    q = W.to_torch(wl.queries, name, DEV)
    d = W.to_torch(wl.documents, name, DEV)
    qo = torch.from_numpy(wl.query_offsets).to(DEV)
    do = torch.from_numpy(wl.document_offsets).to(DEV)
    pq = torch.from_numpy(wl.pair_query_ids).to(DEV)
    pd = torch.from_numpy(wl.pair_document_ids).to(DEV)
    w = torch.from_numpy(wl.dscore).to(DEV)
    _, a = maxsim.score_pairs_packed_with_argmax(q, qo, d, do, pq, pd, max_q_len=32)
    native = _ops.packed_backward_native(w, q, qo, d, do, pq, pd, a, 32)
    assert native is not None and native[0].dtype == dtype and native[1].dtype == dtype
    again = _ops.packed_backward_native(w, q, qo, d, do, pq, pd, a, 32)
    assert torch.equal(native[0], again[0]) and torch.equal(native[1], again[1])
    dq32, dd32 = _ops.ops.maxsim_packed_backward(w, q, qo, d, do, pq, pd, a, 32)
    assert torch.equal(native[0], dq32.to(dtype))
    wq, wd = oracle.pairs_packed_backward(wl.dscore, f32(q), wl.query_offsets, f32(d), wl.document_offsets,
                                          wl.pair_query_ids, wl.pair_document_ids, a.cpu().numpy())
    assert_grads(f32(native[1]), wd, name)
    assert_grads(f32(native[0]), wq, name)
    # through autograd: the leaves receive the native tensors
    qr, dr = q.clone().requires_grad_(True), d.clone().requires_grad_(True)
    maxsim.score_pairs_packed_train(qr, qo, dr, do, pq, pd, max_q_len=32).backward(w)
    assert torch.equal(qr.grad, native[0]) and torch.equal(dr.grad, native[1])
    # short lists are not grouped: the fp32 operator serves them
    assert _ops.packed_backward_native(w[:100], q, qo, d, do, pq[:100].contiguous(), pd[:100].contiguous(),
                                       a[:100].contiguous(), 32) is None
