// Contrastive forward on tcgen05 / TMEM with tiles that start at document
// starts.
//
// fwd_tc05_kernel cuts the packed token stream into 128-token tiles that ignore
// document boundaries, which keeps every MMA column useful but makes the
// epilogue cut its folds wherever a document ends: the chunk that holds a
// boundary is walked column by column, twice, and the rest of that tile is
// folded in pieces.  For documents of a hundred tokens or more that boundary
// work is about a third of the epilogue's instructions, and the epilogue sets
// the pace of the kernel.
//
// Here every document is tiled on its own: tile t of a document covers its
// tokens [128 t, 128 t + 128).  Full tiles never mix documents and take the
// whole-tile fold; only the last tile of a document is partial, and its MMAs
// are issued with N rounded up to 16 columns, so the tensor pipe spends at
// most 15 columns per document on padding, and TMA fetches it as boxes of 32
// rows (rows past the document's end belong to the next document or are
// zero-filled past the end of the tensor; their columns are never read from
// TMEM).  Roles, barriers, register hand-over and bounded waits are those of
// fwd_tc05_kernel.
#pragma once

#include "fwd_tc05.cuh"

namespace maxsim {
namespace tc05 {

// The first e (< 32) columns of a chunk belong to the document.  Groups of
// eight columns past e are skipped with a warp-uniform branch.
template <bool ARGMAX>
__device__ __forceinline__ void fold_prefix(const float (&v)[32], int e, int base_ix, float& run,
                                            int& idx) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (g * 8 < e) {
#pragma unroll
      for (int j = g * 8; j < g * 8 + 8; ++j) {
        if (ARGMAX) {
          if (j < e && v[j] > run) { run = v[j]; idx = base_ix + j; }
        } else {
          if (j < e) run = fmaxf(run, v[j]);
        }
      }
    }
  }
}

// n (< 64) columns held in x (columns 0-31) and y (32-63).
template <bool ARGMAX>
__device__ __forceinline__ void fold_tail(const float (&x)[32], const float (&y)[32], int n,
                                          int base_ix, float& run, int& idx) {
  if (n >= 32) {
    fold32<ARGMAX>(x, base_ix, run, idx);
    fold_prefix<ARGMAX>(y, n - 32, base_ix + 32, run, idx);
  } else {
    fold_prefix<ARGMAX>(x, n, base_ix, run, idx);
  }
}

constexpr int kBox32Bytes = 32 * 128;  // 32 rows x 64 elements of 2 bytes

template <bool ARGMAX>
__global__ void __launch_bounds__(Cfg<2, 128>::kThreads, 1)
fwd_tc05_doc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_d,
                    const __grid_constant__ CUtensorMap tm_d32, const Params P) {
  using C = Cfg<2, 128>;
  constexpr int kMSub = C::kMSub, kBN = C::kBN, kBStages = C::kBStages, kEpiWarps = C::kEpiWarps;
  constexpr int kTmemCols = C::kTmemCols;
  constexpr size_t kSmemA = C::kSmemA, kSmemB = C::kSmemB;
  static_assert(C::kThreads == 384, "register hand-over is sized for 12 warps");
  extern __shared__ unsigned char tc05_smem_raw[];
  const uint32_t raw_base = smem_u32(tc05_smem_raw);
  const uint32_t base = (raw_base + 1023u) & ~1023u;
  const uint32_t smA = base;
  const uint32_t smB = base + (uint32_t)kSmemA;
  const uint32_t bars = smB + (uint32_t)kSmemB;
  const uint32_t b_full = bars;
  const uint32_t b_empty = bars + 8 * kBStages;
  const uint32_t a_full = bars + 16 * kBStages;
  const uint32_t a_empty = a_full + 8;
  const uint32_t t_full = a_empty + 8;
  const uint32_t t_empty = t_full + 8 * kAccStages;
  const uint32_t tmem_slot = t_empty + 8 * kAccStages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kBStages; ++i) { mbar_init(b_full + 8 * i, 1); mbar_init(b_empty + 8 * i, 1); }
    mbar_init(a_full, 1);
    mbar_init(a_empty, 1);
    for (int i = 0; i < kAccStages; ++i) {
      mbar_init(t_full + 8 * i, 1);
      mbar_init(t_empty + 8 * i, kEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(tmem_slot), "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  const int32_t* __restrict__ doff = P.doc_offsets;

  if (warp < C::kProducerWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    if (warp == 0) {
      // ===================== TMA producer ==================================
      if (lane == 0) {
        uint32_t bs = 0, bph = 0, iter = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < P.n_items; item += gridDim.x, ++iter) {
          const int dc = item / P.n_qgroups, qg = item - dc * P.n_qgroups;
          const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
          if (!wait_bounded(a_empty, (iter & 1u) ^ 1u)) { ok = false; break; }
          mbar_expect_tx(a_full, (uint32_t)kSmemA);
#pragma unroll
          for (int sub = 0; sub < kMSub; ++sub)
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_2d(smA + sub * C::kATileBytes + h * kABoxBytes, &tm_q, h * 64,
                          (qg * kMSub + sub) * kBM, a_full);
          int dbeg = __ldg(doff + d_lo);
          int dend_next = __ldg(doff + d_lo + 1);
          for (int d = d_lo; ok && d < d_hi; ++d) {
            const int dend = dend_next;
            if (d + 1 < d_hi) dend_next = __ldg(doff + d + 2);  // in flight while this document's tiles are issued
            for (int t0 = dbeg; t0 < dend; t0 += kBN) {
              if (!wait_bounded(b_empty + 8 * bs, bph ^ 1u)) { ok = false; break; }
              const int rows = dend - t0;
              if (rows >= kBN) {
                mbar_expect_tx(b_full + 8 * bs, (uint32_t)C::kBTileBytes);
#pragma unroll
                for (int h = 0; h < 2; ++h)
                  tma_load_2d(smB + bs * C::kBTileBytes + h * C::kBBoxBytes, &tm_d, h * 64, t0,
                              b_full + 8 * bs);
              } else {
                // last tile of the document: 32-row boxes, as many as it has tokens.  A box
                // of 32 rows is four whole swizzle atoms, so it lands exactly where the same
                // rows of a 128-row box would.
                const int nbox = (rows + 31) >> 5;
                mbar_expect_tx(b_full + 8 * bs, (uint32_t)(nbox * 2 * kBox32Bytes));
                for (int b = 0; b < nbox; ++b)
#pragma unroll
                  for (int h = 0; h < 2; ++h)
                    tma_load_2d(smB + bs * C::kBTileBytes + h * C::kBBoxBytes + b * kBox32Bytes,
                                &tm_d32, h * 64, t0 + b * 32, b_full + 8 * bs);
              }
              if (++bs == kBStages) { bs = 0; bph ^= 1u; }
            }
            dbeg = dend;
          }
        }
      }
    } else if (warp == 1) {
      // ===================== MMA issuer ====================================
      if (lane == 0) {
        uint32_t bs = 0, bph = 0, acc = 0, aph = 0, iter = 0;
        const uint32_t idesc0 = P.idesc & ~(0x3Fu << 17);  // everything but the N field
        bool ok = true;
        for (int item = blockIdx.x; ok && item < P.n_items; item += gridDim.x, ++iter) {
          const int dc = item / P.n_qgroups;
          const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
          if (!wait_bounded(a_full, iter & 1u)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          int dbeg = __ldg(doff + d_lo);
          int dend_next = __ldg(doff + d_lo + 1);
          for (int d = d_lo; ok && d < d_hi; ++d) {
            const int dend = dend_next;
            if (d + 1 < d_hi) dend_next = __ldg(doff + d + 2);
            for (int t0 = dbeg; t0 < dend; t0 += kBN) {
              if (!wait_bounded(t_empty + 8 * acc, aph ^ 1u)) { ok = false; break; }
              if (!wait_bounded(b_full + 8 * bs, bph)) { ok = false; break; }
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              // the last tile of a document: only as many columns as it has tokens, in steps of 16
              const int n16 = min(kBN, (dend - t0 + 15) & ~15);
              const uint32_t idesc = idesc0 | ((uint32_t)(n16 >> 3) << 17);
#pragma unroll
              for (int sub = 0; sub < kMSub; ++sub) {
                const uint32_t d_tmem = tmem_base + acc * (kMSub * kBN) + sub * kBN;
#pragma unroll
                for (int k = 0; k < kDim / 16; ++k) {
                  const uint64_t ad =
                      umma_desc(smA + sub * C::kATileBytes + (k >> 2) * kABoxBytes + (k & 3) * 32);
                  const uint64_t bd =
                      umma_desc(smB + bs * C::kBTileBytes + (k >> 2) * C::kBBoxBytes + (k & 3) * 32);
                  umma_f16(d_tmem, ad, bd, idesc, k > 0 ? 1u : 0u);
                }
              }
              umma_commit(b_empty + 8 * bs);
              umma_commit(t_full + 8 * acc);
              if (++bs == kBStages) { bs = 0; bph ^= 1u; }
              if (++acc == kAccStages) { acc = 0; aph ^= 1u; }
            }
            dbeg = dend;
          }
          umma_commit(a_empty);
        }
      }
    }
  } else {
    // ===================== epilogue ========================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
    const int ew = warp - C::kProducerWarps;
    const int sub = ew >> 2;
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t acc = 0, aph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < P.n_items; item += gridDim.x) {  // goes on after a wait
      // ran out: the pairs this warp does not get to are given NaN scores
      const int dc = item / P.n_qgroups, qg = item - dc * P.n_qgroups;
      const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
      const int q = (qg * kMSub + sub) * kQPerSub + quad;  // this warp's query
      const bool q_ok = q < P.Nq;
      int dbeg = __ldg(doff + d_lo);
      int dend_next = __ldg(doff + d_lo + 1);
      for (int d = d_lo; d < d_hi; ++d) {
        const int dend = dend_next;
        if (d + 1 < d_hi) dend_next = __ldg(doff + d + 2);
        const int Ld = dend - dbeg;
        float run = neg_inf();
        int idx = 0;
        for (int t0 = 0; ok && t0 < Ld; t0 += kBN) {
          if (!__all_sync(0xffffffffu, wait_bounded(t_full + 8 * acc, aph))) { ok = false; break; }  // leave together
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t taddr0 =
              tmem_base + ((uint32_t)(quad * 32) << 16) + acc * (kMSub * kBN) + sub * kBN;
          const int n_valid = min(Ld - t0, kBN);
          // the tile goes to registers and the TMEM stage is handed back before any arithmetic
          uint32_t raw[2][64];
          tmem_ld64_issue(taddr0, raw[0]);
          if (n_valid > 64) tmem_ld64_issue(taddr0 + 64, raw[1]);
          tmem_ld_wait64(raw[0]);
          tmem_ld_wait64(raw[1]);
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(t_empty + 8 * acc);
          if (++acc == kAccStages) { acc = 0; aph ^= 1u; }

          float va[32], vb[32], vc[32], vd[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            va[j] = __uint_as_float(raw[0][j]);
            vb[j] = __uint_as_float(raw[0][32 + j]);
            vc[j] = __uint_as_float(raw[1][j]);
            vd[j] = __uint_as_float(raw[1][32 + j]);
          }
          if (n_valid == kBN) {
            fold128_sel<ARGMAX>(va, vb, vc, vd, t0, run, idx);
          } else if (n_valid >= 64) {
            fold64_sel<ARGMAX>(va, vb, t0, run, idx);
            fold_tail<ARGMAX>(vc, vd, n_valid - 64, t0 + 64, run, idx);
          } else {
            fold_tail<ARGMAX>(va, vb, n_valid, t0, run, idx);
          }
        }
        // document complete for this warp's query: sum the 32 row maxima, store
        float sum = run;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (q_ok) {
          const int64_t pair = (int64_t)q * P.out_ld + P.out_col0 + d;
          if (ARGMAX) P.argmax[pair * kLq + lane] = ok ? idx : 0;
          if (lane == 0) P.scores[pair] = ok ? sum : __int_as_float(0x7fc00000);
        }
        dbeg = dend;
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

}  // namespace tc05

// Returns 0 on success, 1 if the launch could not be prepared (caller falls
// back to another kernel), or a CUDA error code < 0.
template <bool ARGMAX>
int launch_tc05_doc(const PairTable& t, float* scores, int32_t* argmax, int dtype, int sms,
                    cudaStream_t st) {
  using C = tc05::Cfg<2, 128>;
  const int64_t Nq = t.n_pairs / t.C;
  CUtensorMap tm_q, tm_d, tm_d32;
  const bool bf16 = dtype == 2;
  if (!encode_rows128(&tm_q, t.queries, Nq * tc05::kLq, tc05::kBM, bf16)) return 1;
  if (!encode_rows128(&tm_d, t.documents, t.d_rows, C::kBN, bf16)) return 1;
  if (!encode_rows128(&tm_d32, t.documents, t.d_rows, 32, bf16)) return 1;
  tc05::Params P;
  if (!tc05_fill_params(t, scores, argmax, dtype, sms, C::kQPerCta, C::kBN, &P)) return 1;

  auto kern = tc05::fwd_tc05_doc_kernel<ARGMAX>;
  static std::atomic<unsigned char> configured[64];
  if (int rc = tc05_configure(kern, C::kSmemBytes, configured)) return rc;
  const int grid = (int)(P.n_items < sms ? P.n_items : sms);
  kern<<<grid, C::kThreads, C::kSmemBytes, st>>>(tm_q, tm_d, tm_d32, P);
  return 0;
}

}  // namespace maxsim
