"""GPU parity of the packing / unpacking / ranking kernels (through the C ABI)
against the CPU oracle, plus the size-independent properties: pack then unpack
is the identity on valid rows, a ranking is a sorted permutation."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import maxsim_b200 as maxsim
from maxsim_b200 import _ops
from oracle import maxsim_oracle as oracle

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _case(N, L, shape_tail, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    if dtype in (torch.int8, torch.uint8):
        padded = torch.randint(0, 100, (N, L) + shape_tail, generator=g).to(dtype)
    else:
        padded = torch.randn((N, L) + shape_tail, generator=g).to(dtype)
    lengths = torch.randint(1, L + 1, (N,), generator=g, dtype=torch.int32)
    return padded, lengths


@pytest.mark.parametrize("N,L,tail,dtype", [
    (1, 1, (128,), torch.float16),
    (33, 77, (128,), torch.bfloat16),
    (64, 300, (96,), torch.float16),
    (17, 40, (128,), torch.float32),
    (9, 21, (3,), torch.float16),      # 6-byte rows: byte path
    (9, 21, (5,), torch.float32),      # 20-byte rows: 4-byte path
    (5, 16, (7,), torch.uint8),
    (12, 33, (2, 8), torch.float16),   # rows with two trailing dims
])
@pytest.mark.parametrize("where", ["host", "device", "device_total"])
def test_pack_and_unpack_match_the_oracle(N, L, tail, dtype, where):
    padded, lengths = _case(N, L, tail, dtype, seed=N * 131 + L)
    as_np = padded.view(torch.int16).numpy() if dtype == torch.bfloat16 else padded.numpy()
    want_p, want_o = oracle.pack_padded(as_np, lengths.numpy())
    x = padded.to(DEV)
    if where == "host":
        got_p, got_o = maxsim.pack_padded(x, lengths)
    elif where == "device":
        got_p, got_o = maxsim.pack_padded(x, lengths.to(DEV))
    else:
        got_p, got_o = maxsim.pack_padded(x, lengths.to(DEV).long(), total_tokens=int(lengths.sum()))
    assert got_o.dtype == torch.int32 and got_p.dtype == dtype
    np.testing.assert_array_equal(got_o.cpu().numpy(), want_o)
    got_np = got_p.cpu().view(torch.int16).numpy() if dtype == torch.bfloat16 else got_p.cpu().numpy()
    np.testing.assert_array_equal(got_np, want_p)

    back = maxsim.unpack_packed(got_p, got_o, L)
    want_b = oracle.unpack_packed(want_p, want_o, L)
    back_np = back.cpu().view(torch.int16).numpy() if dtype == torch.bfloat16 else back.cpu().numpy()
    np.testing.assert_array_equal(back_np, want_b)
    # a shorter target truncates, a longer one pads with zeros
    for L2 in (max(1, L // 2), L + 3):
        b2 = maxsim.unpack_packed(got_p, got_o, L2)
        w2 = oracle.unpack_packed(want_p, want_o, L2)
        b2_np = b2.cpu().view(torch.int16).numpy() if dtype == torch.bfloat16 else b2.cpu().numpy()
        np.testing.assert_array_equal(b2_np, w2)


def test_pack_of_unaligned_views():
    base = torch.randn(10 * 12 * 8 + 1, device=DEV)
    padded = base[1:].view(10, 12, 8)          # 4-byte aligned only
    lengths = torch.arange(1, 11, dtype=torch.int32)
    got_p, got_o = maxsim.pack_padded(padded, lengths)
    want_p, want_o = oracle.pack_padded(padded.cpu().numpy(), lengths.numpy())
    np.testing.assert_array_equal(got_p.cpu().numpy(), want_p)
    np.testing.assert_array_equal(got_o.cpu().numpy(), want_o)


def test_pack_rejects_bad_lengths_and_totals():
    x = torch.zeros(4, 8, 16, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError, match="lengths must be in"):
        maxsim.pack_padded(x, torch.tensor([1, 0, 3, 4]))
    with pytest.raises(ValueError, match="lengths must be in"):
        maxsim.pack_padded(x, torch.tensor([1, 9, 3, 4]))
    with pytest.raises(ValueError, match="shape"):
        maxsim.pack_padded(x, torch.tensor([1, 2, 3]))
    with pytest.raises(TypeError):
        maxsim.pack_padded(x, torch.tensor([1.0, 2.0, 3.0, 4.0]))
    with pytest.raises(ValueError, match="total_tokens"):
        maxsim.pack_padded(x, torch.tensor([1, 2, 3, 4]), total_tokens=11)


def test_too_small_total_drops_rows_instead_of_overrunning():
    x = torch.randn(4, 8, 16, device=DEV)
    lengths = torch.tensor([8, 8, 8, 8], device=DEV, dtype=torch.int32)
    guard = torch.full((64, 16), 7.0, device=DEV)
    offsets, _ = _ops.offsets_from_lengths(lengths, 8)
    # hand the kernel a packed buffer of 20 rows inside a larger guarded allocation
    rc_buf = guard[:20]
    lib = _ops.load_library()
    rc = lib.maxsim_b200_pack_rows(x.data_ptr(), offsets.data_ptr(), rc_buf.data_ptr(), 4, 8, 64, 20,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(guard[:20], x.reshape(32, 16)[:20])
    assert bool((guard[20:] == 7.0).all())


def test_empty_inputs():
    x = torch.zeros(0, 8, 16, device=DEV, dtype=torch.float16)
    p, o = maxsim.pack_padded(x, torch.zeros(0, dtype=torch.int32))
    assert p.shape == (0, 16) and o.tolist() == [0]
    p, o = maxsim.pack_padded(x, torch.zeros(0, dtype=torch.int32, device=DEV))
    assert p.shape == (0, 16) and o.tolist() == [0]
    v, i = maxsim.rerank_topk(torch.zeros(0, 5, device=DEV), 2)
    assert v.shape == (0, 2) and i.shape == (0, 2)
    v, i = maxsim.rerank_topk(torch.zeros(3, 5, device=DEV), 0)
    assert v.shape == (3, 0) and i.dtype == torch.int64


def test_pack_is_differentiable_and_feeds_the_contrastive_operator():
    torch.manual_seed(5)
    Nq, Nb, Lq, L, D = 8, 12, 32, 50, 128
    q = torch.nn.functional.normalize(torch.randn(Nq, Lq, D, device=DEV), dim=-1).to(torch.bfloat16)
    enc = torch.nn.functional.normalize(torch.randn(Nb, L, D, device=DEV), dim=-1).to(torch.bfloat16)
    lengths = torch.randint(5, L + 1, (Nb,), dtype=torch.int32)

    # with the kernels
    e1 = enc.clone().requires_grad_(True)
    docs, off = maxsim.pack_padded(e1, lengths)
    loss1 = maxsim.contrastive_loss(q, docs, off, temperature=0.5)
    loss1.backward()

    # with the reference's caller formulation (slices + cat), same operator
    e2 = enc.clone().requires_grad_(True)
    docs2 = torch.cat([e2[i, :int(lengths[i])] for i in range(Nb)], dim=0)
    loss2 = maxsim.contrastive_loss(q, docs2, off, temperature=0.5)
    loss2.backward()

    assert torch.equal(docs, docs2)
    torch.testing.assert_close(loss1, loss2, rtol=0, atol=0)
    # grad_documents sums a token's routed query rows in the order shared-memory atomics
    # set, which varies between launches: equal up to the last place of bf16
    torch.testing.assert_close(e1.grad.float(), e2.grad.float(), rtol=2.0 ** -6, atol=1e-4)
    mask = (torch.arange(L)[None, :] < lengths[:, None]).to(DEV)
    assert bool((e1.grad[~mask] == 0).all())
    assert float(e1.grad.float().abs().sum()) > 0


def test_unpack_gradient_is_pack():
    packed = torch.randn(30, 16, device=DEV, requires_grad=True)
    off = torch.tensor([0, 10, 18, 30], dtype=torch.int32, device=DEV)
    out = maxsim.unpack_packed(packed, off, 12)
    w = torch.randn_like(out)
    (out * w).sum().backward()
    want, _ = oracle.pack_padded(w.cpu().numpy(), np.array([10, 8, 12]))
    np.testing.assert_array_equal(packed.grad.cpu().numpy(), want)


@pytest.mark.parametrize("B,C,k", [(1, 1, 1), (3, 2, 2), (16, 50, 10), (32, 100, 100),
                                   (8, 1000, 100), (4, 1000, 1000), (2, 1025, 7),
                                   (2, 4096, 4096), (1, 16384, 64)])
def test_topk_matches_the_oracle(B, C, k):
    g = torch.Generator().manual_seed(B * 7 + C)
    scores = torch.randn(B, C, generator=g)
    if C >= 50:
        scores = scores.round(decimals=2)       # many exact ties
        scores[0, 3] = float("inf")
        scores[0, 9] = float("-inf")
        scores[B - 1, 11] = float("nan")
        scores[B - 1, 5] = -0.0
        scores[B - 1, 6] = 0.0
    want_v, want_i = oracle.rank_rows(scores.numpy(), k)
    got_v, got_i = maxsim.rerank_topk(scores.to(DEV), k)
    np.testing.assert_array_equal(got_i.cpu().numpy(), want_i)
    np.testing.assert_array_equal(got_v.cpu().numpy(), want_v)


def test_topk_limit_is_reported():
    with pytest.raises(RuntimeError, match="at most 16384"):
        maxsim.rerank_topk(torch.zeros(1, 16385, device=DEV), 1)


def test_ranking_of_a_full_rerank_is_a_sorted_permutation():
    torch.manual_seed(0)
    scores = (torch.randn(256, 1000, device=DEV) * 4).round(decimals=1)
    order = maxsim.rerank_order(scores)
    assert order.shape == (256, 1000) and order.dtype == torch.int64
    ranked = torch.gather(scores, 1, order)
    assert bool((ranked[:, :-1] >= ranked[:, 1:]).all())
    assert torch.equal(order.sort(dim=1).values,
                       torch.arange(1000, device=DEV).expand(256, 1000))
    tie = ranked[:, :-1] == ranked[:, 1:]
    assert bool((order[:, :-1][tie] < order[:, 1:][tie]).all())
    want = torch.sort(scores, dim=1, descending=True, stable=True).indices
    assert torch.equal(order, want)


def test_full_size_pack_round_trip():
    # config-5-like encoder output: 1024 documents padded to 512 tokens, bf16
    torch.manual_seed(1)
    enc = torch.randn(1024, 512, 128, device=DEV, dtype=torch.bfloat16)
    lengths = torch.randint(64, 513, (1024,), device=DEV, dtype=torch.int32)
    docs, off = maxsim.pack_padded(enc, lengths)
    assert docs.shape[0] == int(lengths.sum())
    back = maxsim.unpack_packed(docs, off, 512)
    mask = torch.arange(512, device=DEV)[None, :] < lengths[:, None]
    assert torch.equal(back[mask], enc[mask])
    assert bool((back[~mask] == 0).all())
    assert torch.equal(docs, enc[mask])


def test_copy_valid_rows_from_pinned_host_and_from_device():
    torch.manual_seed(2)
    N, L, D = 37, 50, 128
    src = torch.randn(N, L, D).to(torch.float16)
    lengths = torch.randint(1, L + 1, (N,), dtype=torch.int32)
    mask = (torch.arange(L)[None, :] < lengths[:, None])
    for source in (src.pin_memory(), src.to(DEV)):
        dst = torch.full((N, L, D), 7.0, dtype=torch.float16, device=DEV)
        _ops.copy_valid_rows(source, lengths.to(DEV), dst)
        got = dst.cpu()
        assert torch.equal(got[mask], src[mask])
        assert bool((got[~mask] == 7.0).all())          # padding rows untouched
    with pytest.raises(RuntimeError, match="pinned"):
        _ops.copy_valid_rows(src, lengths.to(DEV), torch.empty_like(src, device=DEV))


@pytest.mark.parametrize("pinned", [True, False])
def test_rerank_from_host_equals_the_device_path(pinned):
    from maxsim_b200 import workloads as W
    wl = W.c3_large_rerank_fp16(seed=12, Nq=6, C=40, Ld=300)
    q = W.to_torch(wl.queries, "fp16")
    d = W.to_torch(wl.documents, "fp16")
    # padding rows hold values that would change the scores if they were read
    pad = torch.arange(300)[None, None, :] >= torch.from_numpy(wl.doc_lengths)[:, :, None]
    d[pad] = 1.0e4
    ql, dl = torch.from_numpy(wl.query_lengths), torch.from_numpy(wl.doc_lengths)
    want = maxsim.score_candidates_padded(q.to(DEV), d.to(DEV), ql.to(DEV), dl.to(DEV)).cpu()
    if pinned:
        q, d = q.pin_memory(), d.pin_memory()
    got = maxsim.score_candidates_padded_from_host(q, d, ql, dl, device=DEV)
    assert got.device.type == "cpu" and got.dtype == torch.float32
    assert torch.equal(got, want)
    out = torch.empty(6, 40, dtype=torch.float32).pin_memory()
    staging = torch.full(d.shape, float("nan"), dtype=torch.float16, device=DEV)
    ret = maxsim.score_candidates_padded_from_host(q, d, ql, dl, device=DEV, staging=staging, out=out)
    torch.cuda.synchronize()
    assert ret is out and torch.equal(out, want)
    ws, _ = oracle.score_candidates_padded(q.float().numpy(), d.float().numpy(),
                                           wl.query_lengths, wl.doc_lengths)
    np.testing.assert_allclose(got.numpy(), ws, rtol=2e-2, atol=1e-2)


def test_rerank_from_host_rejects_device_tensors_and_bad_staging():
    q = torch.zeros(2, 32, 128, dtype=torch.float16)
    d = torch.zeros(2, 3, 40, 128, dtype=torch.float16)
    ql, dl = torch.tensor([32, 32]), torch.full((2, 3), 40)
    with pytest.raises(RuntimeError, match="CPU tensor"):
        maxsim.score_candidates_padded_from_host(q.to(DEV), d, ql, dl, device=DEV)
    with pytest.raises(ValueError, match="staging"):
        maxsim.score_candidates_padded_from_host(q, d, ql, dl, device=DEV,
                                                 staging=torch.empty(1, device=DEV))
    with pytest.raises(ValueError, match="doc_lengths"):
        maxsim.score_candidates_padded_from_host(q, d, ql, dl * 0, device=DEV)
