// Contrastive forward on the 5th-generation tensor cores (tcgen05 + TMEM),
// specialised for the late-interaction shape Lq = 32, dim = 128 (other query
// lengths and dims take the general kernel in fwd_tc05_any.cuh, which measures
// 5-10 % slower on this shape).
//
// All-pairs scoring of rectangular queries [Nq, 32, 128] against packed
// documents [T_d, 128] is a dense contraction with only 256 flop per
// similarity value, so the kernel is organised around keeping the tensor pipe
// fed and consuming its output at the rate it is produced:
//
//   * one CTA per SM, M = 256: two accumulators of 128 TMEM lanes, each lane a
//     (query, query-token) row -- 4 queries x 32 tokens per accumulator;
//   * the packed document stream is cut into tiles of 128 tokens that ignore
//     document boundaries, so no MMA column is spent on padding;
//   * warp 0 stages tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle)
//     into a 4-deep shared-memory ring; warp 1 issues tcgen05.mma (K = 128 as
//     8 steps of 16) for both accumulators against each staged tile and
//     commits to mbarriers; accumulators are double-buffered in TMEM (512
//     columns) so the tensor pipe runs ahead of the epilogue;
//   * eight epilogue warps read their row's 128 similarities of a tile into
//     registers with tcgen05.ld and hand the TMEM stage back at once, then fold
//     them into a running maximum and first-index argmax held in registers,
//     cutting at document boundaries; when a document ends the 32 row maxima of
//     a query are summed with a warp shuffle tree.  No similarity value is ever
//     written to shared or global memory.
//   * the epilogue, not the tensor pipe, sets the pace (with the epilogue
//     disabled the TMA/MMA pipeline alone runs at 0.92 of the measured bf16
//     peak), so its arithmetic is arranged for few instructions and much
//     independent work: 3-input max trees, a whole tile folded per step, and
//     an argmax search that first picks the 32-column chunk holding the
//     maximum with selects and then finds the index inside it on the FMA pipe;
//   * the two producer warps sit in a warpgroup of their own (warps 0-3) that
//     hands most of its registers to the epilogue warps (setmaxnreg: 40 and
//     232 per thread), so a whole tile and the fold's temporaries stay in
//     registers without spills.
//
// Every wait is bounded; a wait that runs out records a status bit and the
// CTA drains to the common exit, where TMEM is released.
#pragma once

#include <cuda.h>

#include <atomic>

#include "common.cuh"
#include "fwd_mma.cuh"

namespace maxsim {
namespace tc05 {

constexpr int kBM = 128;   // rows per accumulator (TMEM lanes)
constexpr int kLq = 32;
constexpr int kQPerSub = kBM / kLq;  // 4 queries per accumulator
constexpr int kDim = 128;
constexpr int kAccStages = 2;
constexpr int kABoxBytes = kBM * 128;  // one 128-row x 64-element box of the query block: 16 KB
constexpr uint32_t kWaitLimit = 1u << 22;

// The kernel's configuration: MSUB = 2 accumulators of 128 rows per CTA (M = 256)
// and document tiles of BN = 128 tokens; TMEM holds MSUB * BN * 2 = 512 columns;
// eight epilogue warps, each folding 128 columns per tile.
template <int MSUB, int BN>
struct Cfg {
  static_assert(MSUB == 2 && BN == 128, "one configuration");
  static constexpr int kMSub = MSUB;
  static constexpr int kBN = BN;
  static constexpr int kQPerCta = kQPerSub * MSUB;
  static constexpr int kEpiWarps = 4 * MSUB;
  static constexpr int kProducerWarps = 4;  // TMA, MMA, two idle: a whole warpgroup, so that its
                                            // registers can be handed to the epilogue warps
  static constexpr int kThreads = 32 * (kProducerWarps + kEpiWarps);
  static constexpr int kTmemCols = MSUB * BN * kAccStages;
  static constexpr int kBBoxBytes = BN * 128;          // one BN-row x 64-element box
  static constexpr int kBTileBytes = 2 * kBBoxBytes;
  static constexpr int kATileBytes = 2 * kABoxBytes;   // 32 KB per accumulator
  static constexpr int kBStages = 4;
  static constexpr int kMinBlocks = 1;
  static constexpr size_t kSmemA = (size_t)MSUB * kATileBytes;
  static constexpr size_t kSmemB = (size_t)kBStages * kBTileBytes;
  static constexpr size_t kSmemBytes = kSmemA + kSmemB + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
};

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  atomicOr(&g_device_status, 2);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of
// 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= (uint64_t)1 << 16;                        // leading-dim offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));  // NaN operands are ignored
  return d;
}

// Maximum of 32 values with 3-input max instructions (16 instead of 31).
__device__ __forceinline__ float max32(const float (&v)[32]) {
  float t[11];
#pragma unroll
  for (int i = 0; i < 10; ++i) t[i] = max3(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
  t[10] = fmaxf(v[30], v[31]);
  const float a = max3(t[0], t[1], t[2]), b = max3(t[3], t[4], t[5]), c = max3(t[6], t[7], t[8]);
  return max3(max3(a, b, c), t[9], t[10]);
}

// First index j in [0, 32) with v[j] == m, for a finite m that is the maximum
// of v.  The search runs on the FMA pipe instead of compare/select pairs:
// key_j = (v[j] - m) * 2^126 + c_j with c_j = 2^23 + (31 - j).  Where
// v[j] == m the key is exactly c_j (larger for smaller j); elsewhere it is
// hugely negative.  The maximum key therefore carries 31 - j* in its low
// mantissa bits.  Returns -1 when no key is valid (m infinite or NaN), in which
// case the caller falls back to a compare loop.
__device__ __forceinline__ int first_index_of_max(const float (&v)[32], float m) {
  const float kScale = 8.507059173023462e37f;  // 2^126
  float key[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) key[j] = fmaf(v[j] - m, kScale, 8388608.0f + (float)(31 - j));
  const float k = max32(key);
  if (!(k >= 8388608.0f)) return -1;
  return 31 - (__float_as_int(k) & 31);
}

// 64-column TMEM load (two of them bring a whole 128-token tile to registers).
// tcgen05.ld is asynchronous: its destination registers may only be read after
// tcgen05.wait::ld.  The wait takes the registers as in/out operands so that
// the compiler cannot schedule a use of them ahead of it.
__device__ __forceinline__ void tmem_ld64_issue(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
        "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]),
        "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]),
        "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]),
        "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]),
        "=r"(r[62]), "=r"(r[63])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait64(uint32_t (&r)[64]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                 "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                 "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]),
                 "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                 "+r"(r[30]), "+r"(r[31]), "+r"(r[32]), "+r"(r[33]), "+r"(r[34]), "+r"(r[35]),
                 "+r"(r[36]), "+r"(r[37]), "+r"(r[38]), "+r"(r[39]), "+r"(r[40]), "+r"(r[41]),
                 "+r"(r[42]), "+r"(r[43]), "+r"(r[44]), "+r"(r[45]), "+r"(r[46]), "+r"(r[47]),
                 "+r"(r[48]), "+r"(r[49]), "+r"(r[50]), "+r"(r[51]), "+r"(r[52]), "+r"(r[53]),
                 "+r"(r[54]), "+r"(r[55]), "+r"(r[56]), "+r"(r[57]), "+r"(r[58]), "+r"(r[59]),
                 "+r"(r[60]), "+r"(r[61]), "+r"(r[62]), "+r"(r[63])
               :
               : "memory");
}

// Folds of 64 and 128 similarities of one document.  Once the maximum m of the
// columns is known, the first 32-column chunk whose own maximum equals m holds
// the first index; its 32 values are picked per lane with select instructions
// (one per column for 64 columns, three for 128) and only they go through the
// FMA-pipe key search: about 1.9 instructions per similarity.
template <bool ARGMAX>
__device__ __forceinline__ void fold64_sel(const float (&a)[32], const float (&b)[32], int base_ix,
                                           float& run, int& idx) {
  const float ma = max32(a);
  const float m = fmaxf(ma, max32(b));
  if (ARGMAX) {
    if (__any_sync(0xffffffffu, m > run)) {
      const bool in_a = ma == m;
      float w[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) w[j] = in_a ? a[j] : b[j];
      int first = first_index_of_max(w, m);
      if (m > run) {
        if (first < 0) {  // infinite maximum: compare loop
          first = 31;
#pragma unroll
          for (int j = 30; j >= 0; --j) first = (w[j] == m) ? j : first;
        }
        run = m;
        idx = base_ix + (in_a ? 0 : 32) + first;
      }
    }
  } else {
    run = fmaxf(run, m);
  }
}

template <bool ARGMAX>
__device__ __forceinline__ void fold128_sel(const float (&a)[32], const float (&b)[32],
                                            const float (&c)[32], const float (&d)[32],
                                            int base_ix, float& run, int& idx) {
  const float ma = max32(a), mb = max32(b), mc = max32(c), md = max32(d);
  const float mab = fmaxf(ma, mb);
  const float m = fmaxf(mab, fmaxf(mc, md));
  if (ARGMAX) {
    if (__any_sync(0xffffffffu, m > run)) {
      const bool lower = mab == m;                      // the first maximum lies in a or b
      const bool even = lower ? (ma == m) : (mc == m);  // ... in the first chunk of that half
      float w[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = lower ? a[j] : c[j];
        const float y = lower ? b[j] : d[j];
        w[j] = even ? x : y;
      }
      int first = first_index_of_max(w, m);
      if (m > run) {
        if (first < 0) {  // infinite maximum: compare loop
          first = 31;
#pragma unroll
          for (int j = 30; j >= 0; --j) first = (w[j] == m) ? j : first;
        }
        run = m;
        idx = base_ix + (lower ? 0 : 64) + (even ? 0 : 32) + first;
      }
    }
  } else {
    run = fmaxf(run, m);
  }
}

// Folds 32 similarities of one document into the row's running maximum and
// first-index argmax.  `base_ix` is the document-local index of column 0.
template <bool ARGMAX>
__device__ __forceinline__ void fold32(const float (&w)[32], int base_ix, float& run, int& idx) {
  const float m = max32(w);
  if (ARGMAX) {
    if (__any_sync(0xffffffffu, m > run)) {
      int first = first_index_of_max(w, m);
      if (m > run) {
        if (first < 0) {  // infinite maximum: compare loop
          first = 31;
#pragma unroll
          for (int j = 30; j >= 0; --j) first = (w[j] == m) ? j : first;
        }
        run = m;
        idx = base_ix + first;
      }
    }
  } else {
    run = fmaxf(run, m);
  }
}

struct Params {
  const int32_t* doc_offsets;
  float* scores;
  int32_t* argmax;
  int32_t Nq, Nb;
  int32_t n_qgroups;      // ceil(Nq / queries per CTA)
  int32_t docs_per_item;
  int32_t n_items;        // document runs x query groups, query group fastest
  int32_t out_ld;         // the pair (q, d) is output slot q * out_ld + out_col0 + d
  int32_t out_col0;
  uint32_t idesc;
};

// The producer warpgroup gives most of its registers to the epilogue warps
// (setmaxnreg), which then hold a whole tile plus the fold's temporaries
// without spilling.
template <bool ARGMAX, int MSUB, int BN>
__global__ void __launch_bounds__(Cfg<MSUB, BN>::kThreads, Cfg<MSUB, BN>::kMinBlocks)
fwd_tc05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_d,
                const Params P) {
  using C = Cfg<MSUB, BN>;
  constexpr int kMSub = C::kMSub, kBN = C::kBN, kBStages = C::kBStages, kEpiWarps = C::kEpiWarps;
  constexpr int kTmemCols = C::kTmemCols, kQPerCta = C::kQPerCta;
  constexpr size_t kSmemA = C::kSmemA, kSmemB = C::kSmemB;
  (void)kQPerCta;
  // Register hand-over: the CTA owns 384 x 168 registers from launch; the producer warpgroup
  // drops to 40 per thread, which frees exactly the 2 x 128 x 64 registers the two epilogue
  // warpgroups need to grow to 232.  setmaxnreg.inc waits, without limit, until that many
  // registers are free: the three numbers have to balance.
  static_assert(C::kThreads == 384 && 128 * (168 - 40) == 256 * (232 - 168),
                "register hand-over does not balance");
  extern __shared__ unsigned char tc05_smem_raw[];
  const uint32_t raw = smem_u32(tc05_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t smA = base;
  const uint32_t smB = base + (uint32_t)kSmemA;
  const uint32_t bars = smB + (uint32_t)kSmemB;
  // barrier slots (8 bytes each)
  const uint32_t b_full = bars;                        // [kBStages]
  const uint32_t b_empty = bars + 8 * kBStages;        // [kBStages]
  const uint32_t a_full = bars + 16 * kBStages;
  const uint32_t a_empty = a_full + 8;
  const uint32_t t_full = a_empty + 8;                 // [kAccStages]
  const uint32_t t_empty = t_full + 8 * kAccStages;    // [kAccStages]
  const uint32_t tmem_slot = t_empty + 8 * kAccStages; // 4 bytes

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
  // Items are dealt round-robin with the query group varying fastest, so the
  // CTAs running at any moment work on the same run of documents and share its
  // tiles through L2.  (Giving each CTA a contiguous range of items to spare
  // query-block reloads measured slower.)

  if (warp < C::kProducerWarps) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
  if (warp == 0) {
    // ===================== TMA producer ====================================
    if (lane == 0) {
      uint32_t bs = 0, bph = 0, iter = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < P.n_items; item += gridDim.x, ++iter) {
        const int dc = item / P.n_qgroups, qg = item - dc * P.n_qgroups;
        const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
        const int s0 = __ldg(doff + d_lo), s1 = __ldg(doff + d_hi);
        const int ntiles = (s1 - s0 + kBN - 1) / kBN;
        if (!wait_bounded(a_empty, (iter & 1u) ^ 1u)) { ok = false; break; }
        mbar_expect_tx(a_full, (uint32_t)kSmemA);
#pragma unroll
        for (int sub = 0; sub < kMSub; ++sub)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_2d(smA + sub * C::kATileBytes + h * kABoxBytes, &tm_q, h * 64,
                        (qg * kMSub + sub) * kBM, a_full);
        for (int tile = 0; tile < ntiles; ++tile) {
          if (!wait_bounded(b_empty + 8 * bs, bph ^ 1u)) { ok = false; break; }
          mbar_expect_tx(b_full + 8 * bs, (uint32_t)C::kBTileBytes);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_2d(smB + bs * C::kBTileBytes + h * C::kBBoxBytes, &tm_d, h * 64,
                        s0 + tile * kBN, b_full + 8 * bs);
          if (++bs == kBStages) { bs = 0; bph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer ======================================
    if (lane == 0) {
      uint32_t bs = 0, bph = 0, acc = 0, aph = 0, iter = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < P.n_items; item += gridDim.x, ++iter) {
        const int dc = item / P.n_qgroups;
        const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
        const int s0 = __ldg(doff + d_lo), s1 = __ldg(doff + d_hi);
        const int ntiles = (s1 - s0 + kBN - 1) / kBN;
        if (!wait_bounded(a_full, iter & 1u)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int tile = 0; tile < ntiles; ++tile) {
          if (!wait_bounded(t_empty + 8 * acc, aph ^ 1u)) { ok = false; break; }
          if (!wait_bounded(b_full + 8 * bs, bph)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int sub = 0; sub < kMSub; ++sub) {
            const uint32_t d_tmem = tmem_base + acc * (kMSub * kBN) + sub * kBN;
#pragma unroll
            for (int k = 0; k < kDim / 16; ++k) {
              const uint64_t ad =
                  umma_desc(smA + sub * C::kATileBytes + (k >> 2) * kABoxBytes + (k & 3) * 32);
              const uint64_t bd =
                  umma_desc(smB + bs * C::kBTileBytes + (k >> 2) * C::kBBoxBytes + (k & 3) * 32);
              umma_f16(d_tmem, ad, bd, P.idesc, k > 0 ? 1u : 0u);
            }
          }
          umma_commit(b_empty + 8 * bs);  // slot reusable once these MMAs retire
          umma_commit(t_full + 8 * acc);  // accumulators ready for the epilogue
          if (++bs == kBStages) { bs = 0; bph ^= 1u; }
          if (++acc == kAccStages) { acc = 0; aph ^= 1u; }
        }
        umma_commit(a_empty);  // query block reusable once this item's MMAs retire
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
    for (int item = blockIdx.x; item < P.n_items; item += gridDim.x) {
      const int dc = item / P.n_qgroups, qg = item - dc * P.n_qgroups;
      const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
      const int s0 = __ldg(doff + d_lo), s1 = __ldg(doff + d_hi);
      const int ntiles = ok ? (s1 - s0 + kBN - 1) / kBN : 0;
      const int q = (qg * kMSub + sub) * kQPerSub + quad;  // this warp's query
      const bool q_ok = q < P.Nq;

      int d = d_lo;
      int dstart = s0;
      int dend = __ldg(doff + d_lo + 1);
      float run = neg_inf();
      int idx = 0;

      for (int tile = 0; tile < ntiles; ++tile) {
        if (!__all_sync(0xffffffffu, wait_bounded(t_full + 8 * acc, aph))) { ok = false; break; }  // leave together
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr0 =
            tmem_base + ((uint32_t)(quad * 32) << 16) + acc * (kMSub * kBN) + sub * kBN;
        const int tok_tile = s0 + tile * kBN;
        int n_valid = min(s1 - tok_tile, kBN);  // columns of this tile that hold tokens of the item
        if (d >= d_hi) n_valid = 0;

        // document d complete for this warp's query: sum the 32 row maxima, store
        auto finish_document = [&]() {
          float sum = run;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
          if (q_ok) {
            const int64_t pair = (int64_t)q * P.out_ld + P.out_col0 + d;
            if (ARGMAX) P.argmax[pair * kLq + lane] = idx;
            if (lane == 0) P.scores[pair] = sum;
          }
          run = neg_inf();
          idx = 0;
          ++d;
          dstart = dend;
          if (d < d_hi) dend = __ldg(doff + d + 1);
        };
        // 32 columns starting at token tok0, cut at document boundaries
        auto fold_chunk = [&](const float (&v)[32], int tok0) {
          int col = 0;
          while (col < 32 && d < d_hi) {
            const int seg_end = min(32, dend - tok0);
            const int base_ix = tok0 - dstart;
            // Columns of this chunk that belong to document d: [col, seg_end).
            if (col == 0 && seg_end == 32) {
              fold32<ARGMAX>(v, base_ix, run, idx);
            } else {
              // boundary chunk: per-column predicated update; groups of eight
              // columns that lie outside the document are skipped (warp-uniform)
#pragma unroll
              for (int g8 = 0; g8 < 32; g8 += 8) {
                if (g8 + 8 > col && g8 < seg_end) {
#pragma unroll
                  for (int j = g8; j < g8 + 8; ++j) {
                    if (j >= col && j < seg_end) {
                      if (ARGMAX) {
                        if (v[j] > run) { run = v[j]; idx = base_ix + j; }
                      } else {
                        run = fmaxf(run, v[j]);
                      }
                    }
                  }
                }
              }
            }
            col = max(col, seg_end);
            if (tok0 + col >= dend) finish_document();
          }
        };

        // The whole tile goes to registers at once and the TMEM stage is handed
        // back before any arithmetic, so the tensor pipe never waits on the fold.
        uint32_t raw[2][64];
        if (n_valid > 0) {
          tmem_ld64_issue(taddr0, raw[0]);
          if (n_valid > 64) tmem_ld64_issue(taddr0 + 64, raw[1]);
          tmem_ld_wait64(raw[0]);
          tmem_ld_wait64(raw[1]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(t_empty + 8 * acc);
        if (++acc == kAccStages) { acc = 0; aph ^= 1u; }
        if (n_valid > 0) {
          float va[32], vb[32], vc[32], vd[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            va[j] = __uint_as_float(raw[0][j]);
            vb[j] = __uint_as_float(raw[0][32 + j]);
            vc[j] = __uint_as_float(raw[1][j]);
            vd[j] = __uint_as_float(raw[1][32 + j]);
          }
          if (d < d_hi && tok_tile + 128 <= dend) {
            fold128_sel<ARGMAX>(va, vb, vc, vd, tok_tile - dstart, run, idx);
            if (tok_tile + 128 == dend) finish_document();
          } else {
            if (d < d_hi && tok_tile + 64 <= dend) {
              fold64_sel<ARGMAX>(va, vb, tok_tile - dstart, run, idx);
              if (tok_tile + 64 == dend) finish_document();
            } else {
              fold_chunk(va, tok_tile);
              if (32 < n_valid) fold_chunk(vb, tok_tile + 32);
            }
            if (64 < n_valid) {
              if (d < d_hi && tok_tile + 128 <= dend) {
                fold64_sel<ARGMAX>(vc, vd, tok_tile + 64 - dstart, run, idx);
                if (tok_tile + 128 == dend) finish_document();
              } else {
                fold_chunk(vc, tok_tile + 64);
                if (96 < n_valid) fold_chunk(vd, tok_tile + 96);
              }
            }
          }
        }
      }
      // Documents of the item that no tile finished: documents without tokens at its end, or,
      // after a wait that ran out, everything this warp did not get to (NaN scores then).
      if (q_ok) {
        for (; d < d_hi; ++d) {
          const int64_t pair = (int64_t)q * P.out_ld + P.out_col0 + d;
          if (ARGMAX) P.argmax[pair * kLq + lane] = 0;
          if (lane == 0) P.scores[pair] = ok ? neg_inf() : __int_as_float(0x7fc00000);
        }
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

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                      const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                      const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TensorMapEncodeFn tensor_map_encoder() {
  // function-local static: initialised once, thread-safe since C++11
  static const TensorMapEncodeFn fn = []() -> TensorMapEncodeFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return reinterpret_cast<TensorMapEncodeFn>(p);
    return nullptr;
  }();
  return fn;
}

// rows x 128 row-major matrix of 16-bit elements, boxes of 128 rows x 64 elements
inline bool encode_rows128(CUtensorMap* map, const void* base, int64_t rows, int box_rows, bool bf16) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc || rows <= 0) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)tc05::kDim, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)tc05::kDim * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

inline bool tc05_eligible(const PairTable& t, int dtype) {
  if (dtype != 1 && dtype != 2) return false;  // fp16 / bf16
  if (t.dim != tc05::kDim || t.q_slots != tc05::kLq) return false;
  if ((reinterpret_cast<uintptr_t>(t.queries) & 15u) || (reinterpret_cast<uintptr_t>(t.documents) & 15u))
    return false;
  const int64_t Nb = t.C, Nq = t.n_pairs / (Nb > 0 ? Nb : 1);
  if (Nq < 8 || Nb < 1) return false;
  if (t.d_rows <= 0 || t.d_rows >= (1ll << 31) || Nq * tc05::kLq >= (1ll << 31)) return false;
  if (t.out_ld * Nq >= (1ll << 31)) return false;
  return tensor_map_encoder() != nullptr;
}

// Work partition and instruction descriptor of a launch whose CTAs take
// `q_per_cta` queries and document tiles of `bn` tokens.  False if the item
// count does not fit 32 bits.
inline bool tc05_fill_params(const PairTable& t, float* scores, int32_t* argmax, int dtype, int sms,
                             int q_per_cta, int bn, tc05::Params* P) {
  const int64_t Nb = t.C, Nq = t.n_pairs / Nb;
  P->doc_offsets = t.ib;
  P->scores = scores;
  P->argmax = argmax;
  P->Nq = (int32_t)Nq;
  P->Nb = (int32_t)Nb;
  P->n_qgroups = (int32_t)((Nq + q_per_cta - 1) / q_per_cta);
  int64_t dpi = (Nb * (int64_t)P->n_qgroups) / (16ll * sms);
  if (dpi < 1) dpi = 1;
  if (dpi > Nb) dpi = Nb;
  P->docs_per_item = (int32_t)dpi;
  const int64_t n_dc = (Nb + dpi - 1) / dpi;
  const int64_t n_items = n_dc * P->n_qgroups;
  if (n_items >= (1ll << 31)) return false;
  P->n_items = (int32_t)n_items;
  P->out_ld = (int32_t)t.out_ld;
  P->out_col0 = (int32_t)t.out_col0;
  const uint32_t fmt = dtype == 2 ? 1u : 0u;  // bf16 : fp16
  P->idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(bn >> 3) << 17) |
             ((uint32_t)(tc05::kBM >> 4) << 24);
  return true;
}

// Opt `kern` in to `smem` bytes of dynamic shared memory once per device.
// `configured` is the kernel's own flag array (one per instantiation).
template <typename Kernel>
int tc05_configure(Kernel kern, size_t smem, std::atomic<unsigned char> (&configured)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -3;
  const bool track = dev >= 0 && dev < 64;
  if (!track || !configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return -3;
    if (track) configured[dev].store(1, std::memory_order_release);  // same value from every racing thread
  }
  return 0;
}

// Returns 0 on success, 1 if the launch could not be prepared (caller falls
// back to another kernel), or a CUDA error code < 0.
template <bool ARGMAX>
int launch_tc05(const PairTable& t, float* scores, int32_t* argmax, int dtype, int sms,
                cudaStream_t st) {
  using C = tc05::Cfg<2, 128>;
  const int64_t Nq = t.n_pairs / t.C;
  CUtensorMap tm_q, tm_d;
  const bool bf16 = dtype == 2;
  if (!encode_rows128(&tm_q, t.queries, Nq * tc05::kLq, tc05::kBM, bf16)) return 1;
  if (!encode_rows128(&tm_d, t.documents, t.d_rows, C::kBN, bf16)) return 1;
  tc05::Params P;
  if (!tc05_fill_params(t, scores, argmax, dtype, sms, C::kQPerCta, C::kBN, &P)) return 1;

  auto kern = tc05::fwd_tc05_kernel<ARGMAX, 2, 128>;
  static std::atomic<unsigned char> configured[64];
  if (int rc = tc05_configure(kern, C::kSmemBytes, configured)) return rc;
  const int grid = (int)(P.n_items < sms ? P.n_items : sms);
  kern<<<grid, C::kThreads, C::kSmemBytes, st>>>(tm_q, tm_d, P);
  return 0;
}

}  // namespace maxsim
