// Contrastive forward on the 5th-generation tensor cores (tcgen05 + TMEM) for
// any query length up to 64 and any dim that is a multiple of 16 up to 128
// (Lq = 32 with dim = 128 takes the specialised kernel of fwd_tc05.cuh).
//
// All-pairs scoring of rectangular queries [Nq, Lq, dim] against packed
// documents [T_d, dim] is a dense contraction with only 2*dim flop per
// similarity value, so the kernel is organised around keeping the tensor pipe
// fed and consuming its output at the rate it is produced:
//
//   * one CTA per SM, M = 256: two accumulators of 128 TMEM lanes, each lane a
//     (query, query-token) row.  A query takes LQP = 16, 32 or 64 lanes (the
//     smallest of those that holds Lq); the query block is fetched through a
//     3-D tensor map [dim, Lq, Nq] whose out-of-range rows TMA fills with
//     zeros, so any Lq <= 64 and a partial last query group need no copy;
//   * dim may be any multiple of 16 up to 128: operands are staged as boxes of
//     64 elements (128-byte swizzle); a box that reaches past dim is zero
//     filled by TMA and the MMA loop runs dim/16 steps, so no tensor work is
//     spent on the fill;
//   * two tilings of an item's document tokens (template PER_DOC): tiles of 128
//     tokens cut from the packed stream regardless of document boundaries (no
//     padded MMA column; the epilogue folds the segments of a tile that belong
//     to different documents separately), or every document tiled on its own,
//     its last tile issued with N rounded up to 16 columns and fetched as
//     32-row boxes (short documents; a full tile then never mixes documents);
//   * warp 0 stages tiles with TMA into a 4-deep shared-memory ring; warp 1
//     issues tcgen05.mma for both accumulators against each staged tile and
//     commits to mbarriers; accumulators are double-buffered in TMEM (512
//     columns) so the tensor pipe runs ahead of the epilogue;
//   * eight epilogue warps read their row's 128 similarities of a tile into
//     registers with tcgen05.ld and hand the TMEM stage back at once, then fold
//     them into a running maximum and first-index argmax held in registers.
//     When a document ends, the row maxima of a query are summed with a warp
//     shuffle tree.  No similarity value is ever written to shared or global
//     memory;
//   * the producer warps sit in a warpgroup of their own (warps 0-3) that
//     hands most of its registers to the epilogue warps (setmaxnreg: 40 and
//     232 per thread), so a whole tile stays in registers without spills.
//
// The argmax fold.  The epilogue, not the tensor pipe, sets the pace, so the
// maximum and its first index come out of ONE pass: each similarity has its
// low 7 mantissa bits replaced by 127 - column (one logic instruction) and the
// keys go through a tree of 3-input maxima.  For a non-negative maximum the
// largest key is the largest value (to 17 significant bits) and, among equal
// values, the lowest column.  A maximum that is negative, at least 64 (where
// 2^-16 relative would exceed 1e-3 absolute), infinite or NaN shows in the
// key itself (max.NaN propagates the NaN that an infinity turns into), and
// the warp then walks that segment column by column on the exact values:
// NaN never wins, +inf does, first index wins.  Values in [0, 64) are compared
// on their upper 25 bits everywhere, so equal similarities tie exactly on
// every path and similarities closer than 2^-16 relative count as ties.
//
// Every wait is bounded; a wait that runs out records a status bit, the role
// that gave up waits (bounded) for the asynchronous work it issued itself,
// pairs it did not finish get NaN scores, and the CTA leaves through the
// common exit where TMEM is released.
#pragma once

#include "fwd_tc05.cuh"

namespace maxsim {
namespace tc05g {

using namespace tc05;  // TMA / MMA / mbarrier wrappers and descriptors are shared

constexpr int kBM = 128;        // rows per accumulator (TMEM lanes)
constexpr int kBN = 128;        // document tokens per tile
constexpr int kMSub = 2;        // accumulators per CTA
constexpr int kAccStages = 2;   // TMEM double buffering
constexpr int kBStages = 4;     // document tile ring
constexpr int kMaxDim = 128;
constexpr int kMaxLq = 64;
constexpr int kEpiWarps = 4 * kMSub;
constexpr int kProducerWarps = 4;  // TMA, MMA, two idle: a whole warpgroup, so that its
                                   // registers can be handed to the epilogue warps
constexpr int kThreads = 32 * (kProducerWarps + kEpiWarps);
constexpr int kTmemCols = kMSub * kBN * kAccStages;
constexpr int kBoxBytes = 128 * 128;        // 128 rows x 64 elements of 2 bytes
constexpr int kBox32Bytes = 32 * 128;       // 32 rows x 64 elements
constexpr int kATileBytes = 2 * kBoxBytes;  // one accumulator's query rows, dim <= 128
constexpr int kBTileBytes = 2 * kBoxBytes;
constexpr size_t kSmemA = (size_t)kMSub * kATileBytes;
constexpr size_t kSmemB = (size_t)kBStages * kBTileBytes;
constexpr size_t kSmemBytes = kSmemA + kSmemB + 1024 /*alignment slack*/ + 512 /*barriers, hand-over rings*/;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kPairRing = 8;
constexpr int kPairBytes = 4 * kPairRing + 16;
static_assert(kTmemCols == 512, "TMEM columns");

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  atomicOr(&g_device_status, 2);
  return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

// TMEM loads of 128, 64 and 16 columns of this warp's 32 lanes.  tcgen05.ld is
// asynchronous; load and wait are ONE statement so that the destination
// registers are plain outputs, defined when the statement ends.
__device__ __forceinline__ void tmem_ld128_sync(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x128.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, %80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95, %96, %97, %98, %99, %100, %101, %102, %103, %104, %105, %106, %107, %108, %109, %110, %111, %112, %113, %114, %115, %116, %117, %118, %119, %120, %121, %122, %123, %124, %125, %126, %127}, [%128];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]), "=r"(r[64]), "=r"(r[65]), "=r"(r[66]), "=r"(r[67]), "=r"(r[68]), "=r"(r[69]), "=r"(r[70]), "=r"(r[71]), "=r"(r[72]), "=r"(r[73]), "=r"(r[74]), "=r"(r[75]), "=r"(r[76]), "=r"(r[77]), "=r"(r[78]), "=r"(r[79]), "=r"(r[80]), "=r"(r[81]), "=r"(r[82]), "=r"(r[83]), "=r"(r[84]), "=r"(r[85]), "=r"(r[86]), "=r"(r[87]), "=r"(r[88]), "=r"(r[89]), "=r"(r[90]), "=r"(r[91]), "=r"(r[92]), "=r"(r[93]), "=r"(r[94]), "=r"(r[95]), "=r"(r[96]), "=r"(r[97]), "=r"(r[98]), "=r"(r[99]), "=r"(r[100]), "=r"(r[101]), "=r"(r[102]), "=r"(r[103]), "=r"(r[104]), "=r"(r[105]), "=r"(r[106]), "=r"(r[107]), "=r"(r[108]), "=r"(r[109]), "=r"(r[110]), "=r"(r[111]), "=r"(r[112]), "=r"(r[113]), "=r"(r[114]), "=r"(r[115]), "=r"(r[116]), "=r"(r[117]), "=r"(r[118]), "=r"(r[119]), "=r"(r[120]), "=r"(r[121]), "=r"(r[122]), "=r"(r[123]), "=r"(r[124]), "=r"(r[125]), "=r"(r[126]), "=r"(r[127])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld64_sync(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16_sync(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ---------------------------------------------------------------------------
// Folding a tile's columns into a row's running maximum and first argmax
// ---------------------------------------------------------------------------
constexpr uint32_t kKeyMask = 0xFFFFFF80u;     // value bits of a key
constexpr uint32_t kPlainLimit = 0x42800000u;  // bits of 64.0f: smaller unsigned patterns are
                                               // the finite values in [0, 64)

// 3-input maxima.  KEYED: NaN propagates (a key that is NaN has to surface);
// otherwise NaN operands are ignored, as the score-only contract wants.
template <bool KEYED>
__device__ __forceinline__ float mx3(float a, float b, float c) {
  float d;
  if constexpr (KEYED) asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  else asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <bool KEYED>
__device__ __forceinline__ float mx2(float a, float b) {
  float d;
  if constexpr (KEYED) asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  else asm("max.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}

// What column C of the tile contributes to a maximum: the similarity itself, or
// (KEYED) the similarity with 127 - C in its low 7 bits.  The key is ONE lop3,
// (bits & mask) | imm: `mask` has to arrive in a register (an opaque value set
// up once per thread) because the instruction takes a single immediate.
template <bool KEYED, int C>
__device__ __forceinline__ float col_term(uint32_t bits, uint32_t mask) {
  if constexpr (KEYED) {
    uint32_t out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(out) : "r"(bits), "r"(mask), "n"(127 - C));
    return __uint_as_float(out);
  } else {
    return __uint_as_float(bits);
  }
}

// Maximum over the 16 columns [16 G, 16 G + 16) of the tile in v: 8 maxima
// after the terms.
template <bool KEYED, int G>
__device__ __forceinline__ float group_max(const uint32_t* v, uint32_t mask) {
#define MAXSIM_TERM(J) col_term<KEYED, 16 * G + (J)>(v[16 * G + (J)], mask)
  const float t0 = mx3<KEYED>(MAXSIM_TERM(0), MAXSIM_TERM(1), MAXSIM_TERM(2));
  const float t1 = mx3<KEYED>(MAXSIM_TERM(3), MAXSIM_TERM(4), MAXSIM_TERM(5));
  const float t2 = mx3<KEYED>(MAXSIM_TERM(6), MAXSIM_TERM(7), MAXSIM_TERM(8));
  const float t3 = mx3<KEYED>(MAXSIM_TERM(9), MAXSIM_TERM(10), MAXSIM_TERM(11));
  const float t4 = mx3<KEYED>(MAXSIM_TERM(12), MAXSIM_TERM(13), MAXSIM_TERM(14));
  return mx2<KEYED>(mx3<KEYED>(t0, t1, t2), mx3<KEYED>(t3, t4, MAXSIM_TERM(15)));
#undef MAXSIM_TERM
}

// Maximum term over the columns [from, to) of group g (0 <= from < to <= 16, all
// warp-uniform), re-read from the accumulator at `taddr0` (column 0 of the
// tile): the group index is a run-time value here, so this code exists once and
// serves whichever group a document boundary falls into.
template <bool KEYED>
__device__ __forceinline__ float group_part_max(uint32_t taddr0, int g, int from, int to,
                                                uint32_t mask) {
  uint32_t w[16];
  tmem_ld16_sync(taddr0 + 16 * g, w);
  // 127 - (16 g + j) = ((7 - g) << 4) | (15 - j)
  const uint32_t hi = (uint32_t)(7 - g) << 4;
  float m0 = neg_inf(), m1 = neg_inf();
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float term;
    if constexpr (KEYED) term = __uint_as_float((w[j] & mask) | hi | (uint32_t)(15 - j));
    else term = __uint_as_float(w[j]);
    if (j >= from && j < to) {
      if (j & 1) m1 = mx2<KEYED>(m1, term);
      else m0 = mx2<KEYED>(m0, term);
    }
  }
  return mx2<KEYED>(m0, m1);
}

// The value a similarity is compared on: finite values in [0, 64) on their
// upper 25 bits (what a key carries), everything else exactly.
__device__ __forceinline__ float compare_value(uint32_t bits) {
  return __uint_as_float(bits < kPlainLimit ? (bits & kKeyMask) : bits);
}

// Column-by-column fold of the columns [a, b) of a tile copied to `tile`
// (thread-local memory): the path of rows whose maximum is negative, 64 or
// more, infinite or NaN.  Rare, so it is kept out of line and out of the
// instruction stream of the hot loop.
__device__ __noinline__ void exact_walk(const uint32_t* tile, int a, int b, int base_ix, float* run,
                                        int* idx) {
  float r = *run;
  int ix = *idx;
  for (int c = a; c < b; ++c) {
    const float x = compare_value(tile[c]);
    if (x > r) { r = x; ix = base_ix + c; }  // false for NaN
  }
  *run = r;
  *idx = ix;
}

// A segment's key maximum `km` (columns [a, b) of the tile in v, one document)
// goes into the row's running maximum and first-index argmax.  `base_ix` is
// the document-local index of the tile's column 0.
__device__ __forceinline__ void commit_segment(float km, const uint32_t* v, int a, int b,
                                               int base_ix, float& run, int& idx) {
  const uint32_t kb = __float_as_uint(km);
  if (__all_sync(0xffffffffu, kb < kPlainLimit)) {
    const float tv = __uint_as_float(kb & kKeyMask);
    if (tv > run) {
      run = tv;
      idx = base_ix + 127 - (int)(kb & 127u);
    }
  } else {
    uint32_t tile[kBN];
#pragma unroll
    for (int c = 0; c < kBN; ++c) tile[c] = v[c];
    exact_walk(tile, a, b, base_ix, &run, &idx);
  }
}

// The MMAs of one document tile against both accumulators, K = 16 * ksteps.
// Inlined into the issuing thread's code on purpose: that thread runs with the
// 40 registers setmaxnreg left it, a budget the compiler keeps only for code
// it compiles as part of the kernel -- an out-of-line callee would be compiled
// to its own, larger, register count.
__device__ __forceinline__ void issue_mmas(uint32_t d_tmem, uint32_t smA, uint32_t b_tile,
                                           uint32_t idesc, int ksteps) {
#pragma unroll
  for (int sub = 0; sub < kMSub; ++sub) {
#pragma unroll
    for (int k = 0; k < kMaxDim / 16; ++k) {
      if (k < ksteps) {
        const uint64_t ad = umma_desc(smA + sub * kATileBytes + (k >> 2) * kBoxBytes + (k & 3) * 32);
        const uint64_t bd = umma_desc(b_tile + (k >> 2) * kBoxBytes + (k & 3) * 32);
        umma_f16(d_tmem + sub * kBN, ad, bd, idesc, k > 0 ? 1u : 0u);
      }
    }
  }
}

struct Params {
  const int32_t* doc_offsets;
  float* scores;
  int32_t* argmax;
  int32_t Nq, Nb, Lq;
  int32_t n_qgroups;      // ceil(Nq / queries per CTA)
  int32_t docs_per_item;
  int32_t n_items;        // document runs x query groups, query group fastest
  int32_t ksteps;         // dim / 16
  int32_t out_ld;         // the pair (q, d) is output slot q * out_ld + out_col0 + d
  int32_t out_col0;
  uint32_t idesc;
  uint32_t wait_limit;
};

// LQP: TMEM lanes per query (16, 32 or 64; Lq <= LQP).
template <bool ARGMAX, int LQP, bool PER_DOC>
__global__ void __launch_bounds__(kThreads, 1)
fwd_tc05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_d,
                const __grid_constant__ CUtensorMap tm_d32, const Params P) {
  static_assert(LQP == 16 || LQP == 32 || LQP == 64, "lanes per query");
  static_assert(kThreads == 384, "register hand-over is sized for 12 warps");
  constexpr int kQPerSub = kBM / LQP;          // queries per accumulator
  extern __shared__ unsigned char tc05_smem_raw[];
  const uint32_t raw_base = smem_u32(tc05_smem_raw);
  const uint32_t base = (raw_base + 1023u) & ~1023u;
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
  const uint32_t drain = t_empty + 8 * kAccStages;     // MMA issuer's own, failure path only
  const uint32_t tmem_slot = drain + 8;                // 4 bytes
  // LQP == 64: a query spans two epilogue warps; the upper one hands its partial
  // sums to the lower one through a ring of kPairRing floats per warp pair,
  // followed by the two progress counters (documents handed over / taken).
  const uint32_t pair_rings = bars + 192;              // [kEpiWarps / 2] x kPairBytes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t limit = P.wait_limit;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kBStages; ++i) { mbar_init(b_full + 8 * i, 1); mbar_init(b_empty + 8 * i, 1); }
    mbar_init(a_full, 1);
    mbar_init(a_empty, 1);
    for (int i = 0; i < kAccStages; ++i) {
      mbar_init(t_full + 8 * i, 1);
      mbar_init(t_empty + 8 * i, kEpiWarps);
    }
    mbar_init(drain, 1);
    for (int i = 0; i < (kEpiWarps / 2) * kPairBytes; i += 4)
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(pair_rings + i), "r"(0u) : "memory");
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
  const int nbox = P.ksteps > 4 ? 2 : 1;  // 64-element boxes per operand row
  // Items are dealt round-robin with the query group varying fastest, so the
  // CTAs running at any moment work on the same run of documents and share its
  // tiles through L2.

  // Register hand-over.  The CTA owns 384 x 168 registers from launch; the producer
  // warpgroup drops to 40 per thread, which frees exactly the 2 x 128 x 64 registers the two
  // epilogue warpgroups need to grow to 232.  setmaxnreg.inc waits, without limit, until
  // that many registers are free: the three numbers have to balance.
  static_assert(128 * (168 - 40) == 256 * (232 - 168), "register hand-over does not balance");
  if (warp < kProducerWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
    if (warp == 0) {
      // ===================== TMA producer ==================================
      if (lane == 0) {
        uint32_t bs = 0, bph = 0, iter = 0;
        uint32_t filled = 0;  // tiles put into the ring so far
        bool ok = true, a_armed = false;
        for (int item = blockIdx.x; ok && item < P.n_items; item += gridDim.x, ++iter) {
          const int dc = item / P.n_qgroups, qg = item - dc * P.n_qgroups;
          const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
          a_armed = false;
          if (!wait_bounded(a_empty, (iter & 1u) ^ 1u, limit)) { ok = false; break; }
          mbar_expect_tx(a_full, (uint32_t)(kMSub * nbox * kBoxBytes));
          a_armed = true;
#pragma unroll
          for (int sub = 0; sub < kMSub; ++sub)
            for (int h = 0; h < nbox; ++h)
              tma_load_3d(smA + sub * kATileBytes + h * kBoxBytes, &tm_q, h * 64, 0,
                          (qg * kMSub + sub) * kQPerSub, a_full);
          if constexpr (!PER_DOC) {
            const int s0 = __ldg(doff + d_lo), s1 = __ldg(doff + d_hi);
            const int ntiles = (s1 - s0 + kBN - 1) / kBN;
            for (int tile = 0; tile < ntiles; ++tile) {
              if (!wait_bounded(b_empty + 8 * bs, bph ^ 1u, limit)) { ok = false; break; }
              mbar_expect_tx(b_full + 8 * bs, (uint32_t)(nbox * kBoxBytes));
              for (int h = 0; h < nbox; ++h)
                tma_load_2d(smB + bs * kBTileBytes + h * kBoxBytes, &tm_d, h * 64,
                            s0 + tile * kBN, b_full + 8 * bs);
              ++filled;
              if (++bs == kBStages) { bs = 0; bph ^= 1u; }
            }
          } else {
            int dbeg = __ldg(doff + d_lo);
            int dend_next = __ldg(doff + d_lo + 1);
            for (int d = d_lo; ok && d < d_hi; ++d) {
              const int dend = dend_next;
              if (d + 1 < d_hi) dend_next = __ldg(doff + d + 2);  // in flight while this document's tiles are issued
              for (int t0 = dbeg; t0 < dend; t0 += kBN) {
                if (!wait_bounded(b_empty + 8 * bs, bph ^ 1u, limit)) { ok = false; break; }
                const int rows = dend - t0;
                if (rows >= kBN) {
                  mbar_expect_tx(b_full + 8 * bs, (uint32_t)(nbox * kBoxBytes));
                  for (int h = 0; h < nbox; ++h)
                    tma_load_2d(smB + bs * kBTileBytes + h * kBoxBytes, &tm_d, h * 64, t0,
                                b_full + 8 * bs);
                } else {
                  // last tile of the document: 32-row boxes, as many as it has tokens.  A box
                  // of 32 rows is four whole swizzle atoms, so it lands exactly where the same
                  // rows of a 128-row box would.
                  const int n32 = (rows + 31) >> 5;
                  mbar_expect_tx(b_full + 8 * bs, (uint32_t)(n32 * nbox * kBox32Bytes));
                  for (int b = 0; b < n32; ++b)
                    for (int h = 0; h < nbox; ++h)
                      tma_load_2d(smB + bs * kBTileBytes + h * kBoxBytes + b * kBox32Bytes,
                                  &tm_d32, h * 64, t0 + b * 32, b_full + 8 * bs);
                }
                ++filled;
                if (++bs == kBStages) { bs = 0; bph ^= 1u; }
              }
              dbeg = dend;
            }
          }
        }
        if (!ok) {
          // Gave up.  Copies this thread issued may still be landing in the CTA's
          // shared memory: wait (bounded) until every ring slot it armed has its bytes.
          const uint32_t n = filled < (uint32_t)kBStages ? filled : (uint32_t)kBStages;
          for (uint32_t k = 0; k < n; ++k) {
            const uint32_t f = filled - 1 - k;  // a fill still possibly in flight
            wait_bounded(b_full + 8 * (f % kBStages), (f / kBStages) & 1u, kWaitLimit);
          }
          if (a_armed) wait_bounded(a_full, iter & 1u, kWaitLimit);  // the query block of the item it stopped in
        }
      }
    } else if (warp == 1) {
      // ===================== MMA issuer ====================================
      if (lane == 0) {
        uint32_t bs = 0, bph = 0, acc = 0, aph = 0, iter = 0;
        const uint32_t idesc0 = P.idesc & ~(0x3Fu << 17);  // everything but the N field
        bool ok = true;
        auto issue_tile = [&](uint32_t idesc) -> bool {
          if (!wait_bounded(t_empty + 8 * acc, aph ^ 1u, limit)) return false;
          if (!wait_bounded(b_full + 8 * bs, bph, limit)) return false;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t b_tile = smB + bs * kBTileBytes;
          const uint32_t d_tmem = tmem_base + acc * (kMSub * kBN);
          issue_mmas(d_tmem, smA, b_tile, idesc, P.ksteps);
          umma_commit(b_empty + 8 * bs);  // slot reusable once these MMAs retire
          umma_commit(t_full + 8 * acc);  // accumulators ready for the epilogue
          if (++bs == kBStages) { bs = 0; bph ^= 1u; }
          if (++acc == kAccStages) { acc = 0; aph ^= 1u; }
          return true;
        };
        for (int item = blockIdx.x; ok && item < P.n_items; item += gridDim.x, ++iter) {
          const int dc = item / P.n_qgroups;
          const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
          if (!wait_bounded(a_full, iter & 1u, limit)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if constexpr (!PER_DOC) {
            const int s0 = __ldg(doff + d_lo), s1 = __ldg(doff + d_hi);
            const int ntiles = (s1 - s0 + kBN - 1) / kBN;
            for (int tile = 0; ok && tile < ntiles; ++tile) ok = issue_tile(P.idesc);
          } else {
            int dbeg = __ldg(doff + d_lo);
            int dend_next = __ldg(doff + d_lo + 1);
            for (int d = d_lo; ok && d < d_hi; ++d) {
              const int dend = dend_next;
              if (d + 1 < d_hi) dend_next = __ldg(doff + d + 2);
              for (int t0 = dbeg; ok && t0 < dend; t0 += kBN) {
                // the last tile of a document: only as many columns as it has tokens, in steps of 16
                const int n16 = min(kBN, (dend - t0 + 15) & ~15);
                ok = issue_tile(idesc0 | ((uint32_t)(n16 >> 3) << 17));
              }
              dbeg = dend;
            }
          }
          if (ok) umma_commit(a_empty);  // query block reusable once this item's MMAs retire
        }
        if (!ok) {
          // Gave up.  MMAs this thread issued may still be writing TMEM, which is
          // released at the common exit: wait (bounded) until they have retired.
          umma_commit(drain);
          wait_bounded(drain, 0u, kWaitLimit);
        }
      }
    }
  } else {
    // ===================== epilogue ========================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
    const int ew = warp - kProducerWarps;
    const int sub = ew >> 2;
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    // this lane's row: query qi of the accumulator, query token `tok`
    const int row = quad * 32 + lane;
    const int qi = row / LQP, tok = row % LQP;
    const uint32_t ring = pair_rings + (uint32_t)(ew >> 1) * kPairBytes;  // LQP == 64 only
    uint32_t key_mask;  // the mask of the argmax keys, in a register (see col_term)
    asm volatile("mov.u32 %0, 0xFFFFFF80;" : "=r"(key_mask));
    uint32_t acc = 0, aph = 0;
    uint32_t n_done = 0;  // documents finished by this warp
    bool ok = true;

    for (int item = blockIdx.x; item < P.n_items; item += gridDim.x) {
      const int dc = item / P.n_qgroups, qg = item - dc * P.n_qgroups;
      const int d_lo = dc * P.docs_per_item, d_hi = min(P.Nb, d_lo + P.docs_per_item);
      const int q = (qg * kMSub + sub) * kQPerSub + qi;  // this lane's query
      const bool row_ok = q < P.Nq && tok < P.Lq;
      const int64_t slot0 = (int64_t)q * P.out_ld + P.out_col0;
      int d = d_lo;
      float run = neg_inf();
      int idx = 0;

      // document d complete for this warp's rows: sum the row maxima of each query, store
      auto finish_document = [&]() {
        float sum = row_ok ? run : 0.0f;
#pragma unroll
        for (int off = (LQP >= 32 ? 16 : LQP / 2); off > 0; off >>= 1)
          sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if constexpr (LQP == 64) {
          // quadrant 2k holds tokens 0-31 of a query, quadrant 2k+1 tokens 32-63: the upper
          // warp hands its partial sum to the lower one through the pair's ring.  Both
          // sides wait with a limit (the upper one for a free entry, the lower one for the
          // sum); running out poisons the score and ends this warp's work.
          bool fine = true;
          if (lane == 0) {
            const uint32_t entry = ring + 4 * (n_done % kPairRing);
            uint32_t it = 0;
            if (quad & 1) {
              uint32_t taken;
              do {
                asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(taken) : "r"(ring + 4 * kPairRing + 4) : "memory");
              } while (n_done - taken >= (uint32_t)kPairRing && ++it < limit);
              fine = it < limit;
              asm volatile("st.volatile.shared.f32 [%0], %1;" ::"r"(entry), "f"(sum) : "memory");
              __threadfence_block();
              asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(ring + 4 * kPairRing), "r"(n_done + 1) : "memory");
            } else {
              uint32_t handed;
              do {
                asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(handed) : "r"(ring + 4 * kPairRing) : "memory");
              } while ((int32_t)(handed - n_done) <= 0 && ++it < limit);
              fine = it < limit;
              __threadfence_block();
              float other;
              asm volatile("ld.volatile.shared.f32 %0, [%1];" : "=f"(other) : "r"(entry) : "memory");
              sum = fine ? sum + other : __int_as_float(0x7fc00000);
              __threadfence_block();
              asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(ring + 4 * kPairRing + 4), "r"(n_done + 1) : "memory");
            }
            if (!fine) atomicOr(&g_device_status, 2);
          }
          if (!__shfl_sync(0xffffffffu, fine, 0)) ok = false;
        }
        if (row_ok && ARGMAX) P.argmax[(slot0 + d) * P.Lq + tok] = idx;
        if (tok == 0 && q < P.Nq) P.scores[slot0 + d] = sum;  // LQP == 64: tok == 0 only in the lower warp
        run = neg_inf();
        idx = 0;
        ++d;
        ++n_done;
      };

      if (ok) {
        const uint32_t taddr_row = tmem_base + ((uint32_t)(quad * 32) << 16) + sub * kBN;
        uint32_t v[kBN];
        // One tile.  Its `n_cols` columns [0, n_cols) hold tokens of the item, the first of
        // them of document d, which ends at column `dend_col` of the tile (beyond n_cols: it
        // continues in the next tile).  Documents that end inside the tile are finished.
        // Returns false if the wait for the accumulator ran out.
        auto do_tile = [&](int n_cols, int tok_tile, int& dstart, int& dend) -> bool {
          const bool got = wait_bounded(t_full + 8 * acc, aph, limit);
          if (!__all_sync(0xffffffffu, got)) return false;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t taddr0 = taddr_row + acc * (kMSub * kBN);
          if (n_cols > 64) tmem_ld128_sync(taddr0, v);
          else tmem_ld64_sync(taddr0, v);
          auto release = [&]() {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(t_empty + 8 * acc);
            if (++acc == kAccStages) { acc = 0; aph ^= 1u; }
          };
          const bool simple = n_cols == kBN && dend - tok_tile >= kBN;  // one document, all 128 columns
          // a simple tile goes back to the tensor pipe before any arithmetic; a tile with a
          // document boundary stays until its boundary groups have been re-read
          if (simple) release();
          // maxima of the 16-column groups that hold columns of the item
          float g[8];
          g[0] = group_max<ARGMAX, 0>(v, key_mask);
          g[1] = n_cols > 16 ? group_max<ARGMAX, 1>(v, key_mask) : neg_inf();
          g[2] = n_cols > 32 ? group_max<ARGMAX, 2>(v, key_mask) : neg_inf();
          g[3] = n_cols > 48 ? group_max<ARGMAX, 3>(v, key_mask) : neg_inf();
          if (n_cols > 64) {
            g[4] = group_max<ARGMAX, 4>(v, key_mask);
            g[5] = n_cols > 80 ? group_max<ARGMAX, 5>(v, key_mask) : neg_inf();
            g[6] = n_cols > 96 ? group_max<ARGMAX, 6>(v, key_mask) : neg_inf();
            g[7] = n_cols > 112 ? group_max<ARGMAX, 7>(v, key_mask) : neg_inf();
          } else {
            g[4] = g[5] = g[6] = g[7] = neg_inf();
          }
          auto commit = [&](float km, int a, int b) {
            if constexpr (ARGMAX) commit_segment(km, v, a, b, tok_tile - dstart, run, idx);
            else run = fmaxf(run, km);
          };
          if (simple) {
            commit(mx3<ARGMAX>(mx3<ARGMAX>(g[0], g[1], g[2]), mx3<ARGMAX>(g[3], g[4], g[5]),
                               mx2<ARGMAX>(g[6], g[7])), 0, kBN);
            if (tok_tile + kBN == dend) {
              finish_document();
              dstart = dend;
              if (d < d_hi) dend = __ldg(doff + d + 1);
            }
            return true;
          }
          int col = 0;
          while (ok && d < d_hi) {
            const int a = col;
            const int e = min(n_cols, dend - tok_tile);  // this document's columns end here
            if (e > a) {
              float km = neg_inf();
              if (col & 15) {  // the segment starts inside a group
                const int gq = col >> 4, hi = min(e, 16 * gq + 16);
                km = group_part_max<ARGMAX>(taddr0, gq, col & 15, hi - 16 * gq, key_mask);
                col = hi;
              }
              const int g_hi = e >> 4;  // whole groups: [col / 16, g_hi)
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (16 * i >= col && i < g_hi) km = mx2<ARGMAX>(km, g[i]);
              col = max(col, 16 * g_hi);
              if (col < e)  // the segment ends inside a group
                km = mx2<ARGMAX>(km, group_part_max<ARGMAX>(taddr0, g_hi, 0, e & 15, key_mask));
              col = e;
              commit(km, a, e);
            }
            if (tok_tile + e < dend) break;  // the document continues in the next tile
            finish_document();
            dstart = dend;
            if (d < d_hi) dend = __ldg(doff + d + 1);
          }
          release();
          return true;
        };

        if constexpr (!PER_DOC) {
          const int s0 = __ldg(doff + d_lo), s1 = __ldg(doff + d_hi);
          const int ntiles = (s1 - s0 + kBN - 1) / kBN;
          int dstart = s0;
          int dend = __ldg(doff + d_lo + 1);
          for (int tile = 0; ok && tile < ntiles; ++tile) {
            const int tok_tile = s0 + tile * kBN;
            if (!do_tile(min(s1 - tok_tile, kBN), tok_tile, dstart, dend)) ok = false;
          }
          while (ok && d < d_hi) finish_document();  // only documents without tokens are left
        } else {
          int dstart = __ldg(doff + d_lo);
          int dend = __ldg(doff + d_lo + 1);
          while (ok && d < d_hi) {
            if (dend == dstart) {  // a document without tokens
              finish_document();
              if (d < d_hi) dend = __ldg(doff + d + 1);
              continue;
            }
            const int d_now = d;
            for (int t0 = dstart; ok && d == d_now; t0 += kBN)
              if (!do_tile(min(dend - t0, kBN), t0, dstart, dend)) ok = false;
          }
        }
      }
      if (!ok) {
        // a wait ran out: the pairs this warp did not finish get NaN scores
        for (; d < d_hi; ++d) {
          const int64_t s = slot0 + d;
          if (row_ok && ARGMAX) P.argmax[s * P.Lq + tok] = 0;
          if (tok == 0 && q < P.Nq) P.scores[s] = __int_as_float(0x7fc00000);
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

// One thread waits `limit` polls for a barrier phase that nothing will ever
// complete, with the same bounded wait the kernels above use: it has to give
// up, record the status bit and return.  Nothing asynchronous is in flight, so
// the wait running out cannot leave anything behind; the next launch finds a
// clean device.  For the test of the time-out reporting path.
__global__ void wait_probe_kernel(uint32_t limit, int* gave_up) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t b = smem_u32(&bar);
  mbar_init(b, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  const bool done = wait_bounded(b, 0u, limit);
  if (gave_up) *gave_up = done ? 0 : 1;
}

}  // namespace tc05g

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// rows x dim row-major matrix of 16-bit elements, boxes of box_rows rows x 64
// elements; elements past dim and rows past the end read as zero
inline bool encode_rows(CUtensorMap* map, const void* base, int64_t rows, int dim, int box_rows,
                        bool bf16) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc || rows <= 0) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)dim, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)dim * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// queries [Nq, Lq, dim] as a 3-D map; a box takes 64 elements x lqp tokens x
// 128 / lqp queries, i.e. 128 accumulator rows, zero filled past Lq, dim, Nq
inline bool encode_queries(CUtensorMap* map, const void* base, int64_t Nq, int Lq, int dim, int lqp,
                           bool bf16) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc || Nq <= 0) return false;
  cuuint64_t gdim[3] = {(cuuint64_t)dim, (cuuint64_t)Lq, (cuuint64_t)Nq};
  cuuint64_t gstride[2] = {(cuuint64_t)dim * 2, (cuuint64_t)Lq * dim * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)lqp, (cuuint32_t)(tc05g::kBM / lqp)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

inline int tc05g_lanes_per_query(int Lq) { return Lq <= 16 ? 16 : (Lq <= 32 ? 32 : 64); }

// fp16 / bf16, Lq <= 64, dim a multiple of 16 up to 128, at least one CTA's
// worth of queries.
inline bool tc05g_eligible(const PairTable& t, int dtype) {
  if (dtype != 1 && dtype != 2) return false;  // fp16 / bf16
  if (t.dim <= 0 || t.dim > tc05g::kMaxDim || t.dim % 16 != 0) return false;
  if (t.q_slots <= 0 || t.q_slots > tc05g::kMaxLq) return false;
  if ((reinterpret_cast<uintptr_t>(t.queries) & 15u) || (reinterpret_cast<uintptr_t>(t.documents) & 15u))
    return false;
  const int64_t Nb = t.C, Nq = t.n_pairs / (Nb > 0 ? Nb : 1);
  if (Nq < 2 * (tc05g::kBM / tc05g_lanes_per_query(t.q_slots)) || Nb < 1) return false;
  if (t.d_rows <= 0 || t.d_rows >= (1ll << 31) || Nq * t.q_slots >= (1ll << 31)) return false;
  if (t.out_ld * Nq >= (1ll << 31)) return false;
  return tensor_map_encoder() != nullptr;
}

// Work partition and instruction descriptor of a launch whose CTAs take
// `q_per_cta` queries.  False if the item count does not fit 32 bits.
inline bool tc05g_fill_params(const PairTable& t, float* scores, int32_t* argmax, int dtype, int sms,
                              int q_per_cta, tc05g::Params* P) {
  const int64_t Nb = t.C, Nq = t.n_pairs / Nb;
  P->doc_offsets = t.ib;
  P->scores = scores;
  P->argmax = argmax;
  P->Nq = (int32_t)Nq;
  P->Nb = (int32_t)Nb;
  P->Lq = t.q_slots;
  P->n_qgroups = (int32_t)((Nq + q_per_cta - 1) / q_per_cta);
  int64_t dpi = (Nb * (int64_t)P->n_qgroups) / (16ll * sms);
  if (dpi < 1) dpi = 1;
  if (dpi > Nb) dpi = Nb;
  P->docs_per_item = (int32_t)dpi;
  const int64_t n_dc = (Nb + dpi - 1) / dpi;
  const int64_t n_items = n_dc * P->n_qgroups;
  if (n_items >= (1ll << 31)) return false;
  P->n_items = (int32_t)n_items;
  P->ksteps = t.dim / 16;
  P->out_ld = (int32_t)t.out_ld;
  P->out_col0 = (int32_t)t.out_col0;
  const uint32_t fmt = dtype == 2 ? 1u : 0u;  // bf16 : fp16
  P->idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(tc05g::kBN >> 3) << 17) |
             ((uint32_t)(tc05g::kBM >> 4) << 24);
  P->wait_limit = tc05g::kWaitLimit;
  return true;
}

// Returns 0 on success, 1 if the launch could not be prepared (caller falls
// back to another kernel), or a CUDA error code < 0.
template <bool ARGMAX, int LQP, bool PER_DOC>
int launch_tc05g_cfg(const PairTable& t, float* scores, int32_t* argmax, int dtype, int sms,
                    cudaStream_t st) {
  const int64_t Nq = t.n_pairs / t.C;
  CUtensorMap tm_q, tm_d, tm_d32;
  const bool bf16 = dtype == 2;
  if (!encode_queries(&tm_q, t.queries, Nq, t.q_slots, t.dim, LQP, bf16)) return 1;
  if (!encode_rows(&tm_d, t.documents, t.d_rows, t.dim, tc05g::kBN, bf16)) return 1;
  if (!encode_rows(&tm_d32, t.documents, t.d_rows, t.dim, 32, bf16)) return 1;
  tc05g::Params P;
  if (!tc05g_fill_params(t, scores, argmax, dtype, sms, 2 * (tc05g::kBM / LQP), &P)) return 1;

  auto kern = tc05g::fwd_tc05_kernel<ARGMAX, LQP, PER_DOC>;
  static std::atomic<unsigned char> configured[64];
  if (int rc = tc05_configure(kern, tc05g::kSmemBytes, configured)) return rc;
  const int grid = (int)(P.n_items < sms ? P.n_items : sms);
  kern<<<grid, tc05g::kThreads, tc05g::kSmemBytes, st>>>(tm_q, tm_d, tm_d32, P);
  return 0;
}

// per_document: every document tiled on its own (argmax launches only).
template <bool ARGMAX>
int launch_tc05g(const PairTable& t, float* scores, int32_t* argmax, int dtype, int sms,
                cudaStream_t st, bool per_document) {
  const int lqp = tc05g_lanes_per_query(t.q_slots);
  if constexpr (ARGMAX) {
    if (per_document) {
      if (lqp == 16) return launch_tc05g_cfg<true, 16, true>(t, scores, argmax, dtype, sms, st);
      if (lqp == 32) return launch_tc05g_cfg<true, 32, true>(t, scores, argmax, dtype, sms, st);
      return launch_tc05g_cfg<true, 64, true>(t, scores, argmax, dtype, sms, st);
    }
  }
  if (lqp == 16) return launch_tc05g_cfg<ARGMAX, 16, false>(t, scores, argmax, dtype, sms, st);
  if (lqp == 32) return launch_tc05g_cfg<ARGMAX, 32, false>(t, scores, argmax, dtype, sms, st);
  return launch_tc05g_cfg<ARGMAX, 64, false>(t, scores, argmax, dtype, sms, st);
}

}  // namespace maxsim
