// Streaming forward kernel for fp16 / bf16 (dim in {32, 64, 96, 128}).
//
// The rerank and packed workloads carry about 32 flop per document byte, so
// they are bound by how fast document tokens stream out of HBM.  This kernel
// is built around that stream:
//
//   * persistent CTAs, one per SM, twelve warps each; every warp owns whole
//     (query, document) pairs, so no cross-warp reduction exists;
//   * each warp keeps its own ring of kStages shared-memory slots of 16
//     document tokens.  Lane 0 feeds the ring with TMA bulk copies
//     (cp.async.bulk global -> shared, completion on an mbarrier), running
//     kStages tiles ahead of the math and straight across pair boundaries, so
//     the memory system always has twelve rings per SM in flight;
//   * padding rows are never fetched: the last tile of a document copies only
//     its valid tokens;
//   * the query (<= 32 rows per pass) lives in registers as mma.sync A
//     fragments and is reloaded only when the query changes;
//   * Q.D^T runs on mma.sync m16n8k16 with fp32 accumulation.  The k index is
//     permuted identically for A and B (each thread feeds the 8 consecutive
//     elements it fetched with one 128-bit load into two k-steps), which lets
//     the B fragments come from unswizzled rows with 128-bit loads;
//   * the epilogue keeps a running maximum and first-index argmax per query
//     row in registers; only the [Lq] argmax and the score reach HBM.
#pragma once

#include <type_traits>

#include "common.cuh"
#include "fwd_simt.cuh"  // merge_best

namespace maxsim {

constexpr int kMmaWarps = 12;
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kTileTokens = 16;
constexpr int kStages = 4;
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and records a status bit) if the phase never
// completes, so a lost copy ends the kernel instead of hanging the device.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  atomicOr(&g_device_status, 1);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// What lane 0 records for the math side about the tile it put in a slot.
// Record A is read for every tile, record B only for the first tile of a
// (pair, query pass).
struct __align__(16) TileMetaA {
  int32_t pair;   // -1: no more work
  int32_t j0;     // first document token of the tile
  int32_t Ld;
  int32_t lq_q0;  // Lq | (q0 << 16): query length and row offset of this pass
};
struct __align__(16) TileMetaB {
  int32_t q_row;  // first query row of this pass
  int32_t pad0, pad1, pad2;
};

struct Geo32 {
  int32_t q_row0, d_row0, Lq, Ld;
  int32_t pair;  // the pair these rows belong to (differs from the grid position under an order)
};

// Pair geometry with 32-bit rows (the dispatcher guarantees every row index
// and pair index fits).
template <int LAYOUT>
__device__ __forceinline__ Geo32 geo32(const PairTable& t, int32_t pos) {
  Geo32 g;
  const int32_t p = (int32_t)pair_at<LAYOUT>(t, pos);
  g.pair = p;
  if constexpr (LAYOUT == kPadded) {
    const int32_t b = (int32_t)((uint32_t)p / (uint32_t)t.C);
    g.q_row0 = b * t.q_slots;
    g.Lq = __ldg(t.ia + b);
    g.d_row0 = p * t.Ld_max;
    g.Ld = __ldg(t.ib + p);
  } else if constexpr (LAYOUT == kPacked) {
    const int32_t qi = __ldg(t.ic + p);
    const int32_t di = __ldg(t.id + p);
    g.q_row0 = __ldg(t.ia + qi);
    g.Lq = __ldg(t.ia + qi + 1) - g.q_row0;
    g.d_row0 = __ldg(t.ib + di);
    g.Ld = __ldg(t.ib + di + 1) - g.d_row0;
  } else {
    const int32_t qi = (int32_t)((uint32_t)p / (uint32_t)t.C);
    const int32_t di = p - qi * t.C;
    g.q_row0 = qi * t.q_slots;
    g.Lq = t.q_slots;
    g.d_row0 = __ldg(t.ib + di);
    g.Ld = __ldg(t.ib + di + 1) - g.d_row0;
  }
  g.Lq = max(0, min(g.Lq, t.q_slots));
  g.Ld = max(0, g.Ld);
  return g;
}

template <int DIM>
constexpr size_t mma_smem_bytes() {
  return (size_t)kMmaWarps * kStages * (kTileTokens * DIM * 2)                        // rings
         + (size_t)kMmaWarps * kStages * (sizeof(TileMetaA) + sizeof(TileMetaB))      // records
         + (size_t)kMmaWarps * kStages * 8;                                           // mbarriers
}

template <typename T, int DIM, int LAYOUT, bool ARGMAX>
__global__ void __launch_bounds__(kMmaThreads, 1)
fwd_mma_kernel(PairTable t, float* __restrict__ scores, int32_t* __restrict__ argmax,
               int pairs_per_chunk) {
  constexpr int kRowBytes = DIM * 2;
  constexpr int kStageBytes = kTileTokens * kRowBytes;
  constexpr int kChunks = DIM / 32;  // 64-byte k chunks per row

  extern __shared__ __align__(128) unsigned char mma_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, tq = lane & 3;

  unsigned char* ring = mma_smem + (size_t)warp * kStages * kStageBytes;
  unsigned char* after_rings = mma_smem + (size_t)kMmaWarps * kStages * kStageBytes;
  TileMetaA* metaA = reinterpret_cast<TileMetaA*>(after_rings) + warp * kStages;
  TileMetaB* metaB =
      reinterpret_cast<TileMetaB*>(after_rings + (size_t)kMmaWarps * kStages * sizeof(TileMetaA)) +
      warp * kStages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(
                       after_rings +
                       (size_t)kMmaWarps * kStages * (sizeof(TileMetaA) + sizeof(TileMetaB))) +
                   warp * kStages;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t bars_u32 = smem_u32(bars);

  __shared__ int s_next_chunk;  // chunks of this CTA handed out so far
  if (threadIdx.x == 0) s_next_chunk = 0;
  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(bars_u32 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // ---- feeding cursor (uniform across the warp) ---------------------------
  // Chunks of `pairs_per_chunk` consecutive pairs are dealt round-robin over
  // the CTAs (CTA b owns chunks b, b + grid, b + 2*grid, ...); inside a CTA the
  // warps take the CTA's chunks from a shared counter as they become free, so
  // ragged documents do not leave some warps idle while others still work.
  const int32_t n_pairs = (int32_t)t.n_pairs;
  const int32_t n_chunks = (n_pairs + pairs_per_chunk - 1) / pairs_per_chunk;
  int32_t fp = -1;     // pair being fed (-1: none left)
  int32_t np = -1;     // the pair after it, geometry already requested
  int32_t np_end = 0;  // end of np's chunk
  Geo32 cur, nxt;
  cur.q_row0 = cur.d_row0 = cur.Lq = cur.Ld = cur.pair = 0;
  nxt = cur;
  int f_q0 = 0, f_j0 = 0;

  auto fetch_next = [&]() {  // np <- successor of np within this warp's chunks; request its geometry
    if (np >= 0 && np + 1 < np_end) {
      ++np;
    } else {
      int k = 0;
      if (lane == 0) k = atomicAdd(&s_next_chunk, 1);
      k = __shfl_sync(0xffffffffu, k, 0);
      const int64_t chunk = (int64_t)k * gridDim.x + blockIdx.x;
      if (chunk < n_chunks) {
        np = (int32_t)chunk * pairs_per_chunk;
        np_end = min(np + pairs_per_chunk, n_pairs);
      } else {
        np = -1;
      }
    }
    if (np >= 0) nxt = geo32<LAYOUT>(t, np);
  };
  auto next_pair = [&]() {
    fp = np;
    cur = nxt;
    if (np >= 0) fetch_next();
  };
  fetch_next();
  next_pair();

  const unsigned char* dbase = reinterpret_cast<const unsigned char*>(t.documents);
  const unsigned char* qbase = reinterpret_cast<const unsigned char*>(t.queries);

  auto feed = [&](int s) {
    if (fp < 0) {
      if (lane == 0) metaA[s].pair = -1;
      return;
    }
    const int n_valid = max(0, min(kTileTokens, cur.Ld - f_j0));
    if (lane == 0) {
      TileMetaA a;
      a.pair = cur.pair;
      a.j0 = f_j0;
      a.Ld = cur.Ld;
      a.lq_q0 = cur.Lq | (f_q0 << 16);
      metaA[s] = a;
      if (f_j0 == 0) metaB[s].q_row = cur.q_row0 + f_q0;
      const uint32_t bytes = (uint32_t)n_valid * kRowBytes;
      mbar_expect_tx(bars_u32 + 8 * s, bytes);
      if (bytes) {
        bulk_g2s(ring_u32 + s * kStageBytes,
                 dbase + (int64_t)(cur.d_row0 + f_j0) * kRowBytes, bytes, bars_u32 + 8 * s);
      }
    }
    f_j0 += kTileTokens;
    if (f_j0 >= cur.Ld) {
      f_j0 = 0;
      f_q0 += 32;
      if (f_q0 >= cur.Lq) {
        f_q0 = 0;
        next_pair();
      }
    }
  };

  // ---- math side ----------------------------------------------------------
  uint32_t afrag[2][DIM / 16][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int ks = 0; ks < DIM / 16; ++ks)
#pragma unroll
      for (int r = 0; r < 4; ++r) afrag[mt][ks][r] = 0u;
  int32_t a_row = -1;  // query row the fragments were loaded from
  int a_rows = 0;      // valid rows in the fragments

  float run[2][2];
  int idx[2][2];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) { run[mt][h] = neg_inf(); idx[mt][h] = 0; }
  float score_acc = 0.0f;

  int s = 0;
  uint32_t parity = 0;
  for (int it = 0;; ++it, ++s) {
    if (s == kStages) { s = 0; if (it > kStages) parity ^= 1u; }
    if (it >= kStages) {
      const TileMetaA m = metaA[s];
      if (m.pair < 0) break;
      const int j0 = m.j0, Ld = m.Ld;
      const int Lq = m.lq_q0 & 0xffff, q0 = m.lq_q0 >> 16;

      if (j0 == 0) {
        const int32_t qrow = metaB[s].q_row;
        const int rows = min(32, Lq - q0);
        if (qrow != a_row || rows != a_rows) {
          a_row = qrow;
          a_rows = rows;
          const unsigned char* qp = qbase + (int64_t)qrow * kRowBytes + tq * 16;
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            const int r_lo = mt * 16 + g, r_hi = r_lo + 8;
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
              uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
              if (r_lo < rows) lo = ldg_nc_v4(qp + r_lo * kRowBytes + c * 64);
              if (r_hi < rows) hi = ldg_nc_v4(qp + r_hi * kRowBytes + c * 64);
              afrag[mt][2 * c][0] = lo.x; afrag[mt][2 * c][1] = hi.x;
              afrag[mt][2 * c][2] = lo.y; afrag[mt][2 * c][3] = hi.y;
              afrag[mt][2 * c + 1][0] = lo.z; afrag[mt][2 * c + 1][1] = hi.z;
              afrag[mt][2 * c + 1][2] = lo.w; afrag[mt][2 * c + 1][3] = hi.w;
            }
          }
        }
        if (q0 == 0) score_acc = 0.0f;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int h = 0; h < 2; ++h) { run[mt][h] = neg_inf(); idx[mt][h] = 0; }
      }
      const int rows = a_rows;

      if (!__all_sync(0xffffffffu, mbar_wait(bars_u32 + 8 * s, parity))) break;  // leave together

      float acc[2][2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[mt][nt][r] = 0.0f;

      const uint32_t stage = ring_u32 + s * kStageBytes + tq * 16;
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        const uint4 b0 = lds_v4(stage + g * kRowBytes + c * 64);
        const uint4 b1 = lds_v4(stage + (8 + g) * kRowBytes + c * 64);
        mma16816<T>(acc[0][0], afrag[0][2 * c][0], afrag[0][2 * c][1], afrag[0][2 * c][2],
                    afrag[0][2 * c][3], b0.x, b0.y);
        mma16816<T>(acc[0][1], afrag[0][2 * c][0], afrag[0][2 * c][1], afrag[0][2 * c][2],
                    afrag[0][2 * c][3], b1.x, b1.y);
        if (rows > 16) {
          mma16816<T>(acc[1][0], afrag[1][2 * c][0], afrag[1][2 * c][1], afrag[1][2 * c][2],
                      afrag[1][2 * c][3], b0.x, b0.y);
          mma16816<T>(acc[1][1], afrag[1][2 * c][0], afrag[1][2 * c][1], afrag[1][2 * c][2],
                      afrag[1][2 * c][3], b1.x, b1.y);
        }
        mma16816<T>(acc[0][0], afrag[0][2 * c + 1][0], afrag[0][2 * c + 1][1],
                    afrag[0][2 * c + 1][2], afrag[0][2 * c + 1][3], b0.z, b0.w);
        mma16816<T>(acc[0][1], afrag[0][2 * c + 1][0], afrag[0][2 * c + 1][1],
                    afrag[0][2 * c + 1][2], afrag[0][2 * c + 1][3], b1.z, b1.w);
        if (rows > 16) {
          mma16816<T>(acc[1][0], afrag[1][2 * c + 1][0], afrag[1][2 * c + 1][1],
                      afrag[1][2 * c + 1][2], afrag[1][2 * c + 1][3], b0.z, b0.w);
          mma16816<T>(acc[1][1], afrag[1][2 * c + 1][0], afrag[1][2 * c + 1][1],
                      afrag[1][2 * c + 1][2], afrag[1][2 * c + 1][3], b1.z, b1.w);
        }
      }

      // running max / first argmax; a thread meets its columns in ascending order
      if (j0 + kTileTokens <= Ld) {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int h = r >> 1;
              const float v = acc[mt][nt][r];
              if (ARGMAX) {
                if (v > run[mt][h]) { run[mt][h] = v; idx[mt][h] = j0 + nt * 8 + tq * 2 + (r & 1); }
              } else {
                run[mt][h] = fmaxf(run[mt][h], v);  // returns the non-NaN operand
              }
            }
      } else {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int col = j0 + nt * 8 + tq * 2 + (r & 1);
              const int h = r >> 1;
              const float v = acc[mt][nt][r];
              if (col < Ld) {
                if (ARGMAX) {
                  if (v > run[mt][h]) { run[mt][h] = v; idx[mt][h] = col; }
                } else {
                  run[mt][h] = fmaxf(run[mt][h], v);
                }
              }
            }
      }

      if (j0 + kTileTokens >= Ld) {
        // document finished for this query pass: fold the quad, sum the rows
        float contrib = 0.0f;
        int my_ix = 0;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v = run[mt][h];
            int ix = idx[mt][h];
#pragma unroll
            for (int off = 1; off <= 2; off <<= 1) {
              const float ov = __shfl_xor_sync(0xffffffffu, v, off);
              if (ARGMAX) {
                const int oi = __shfl_xor_sync(0xffffffffu, ix, off);
                merge_best(v, ix, ov, oi);
              } else {
                v = fmaxf(v, ov);
              }
            }
            const int row = mt * 16 + h * 8 + g;
            if (tq == 0 && row < rows) contrib += v;
            if (tq == mt * 2 + h) my_ix = ix;
          }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, off);
        score_acc += contrib;
        if (ARGMAX) {
          const int row = (tq >> 1) * 16 + (tq & 1) * 8 + g;
          if (row < rows) argmax[(int64_t)m.pair * t.q_slots + q0 + row] = my_ix;
        }
        if (q0 + 32 >= Lq) {
          if (lane == 0) scores[m.pair] = score_acc;
          if (ARGMAX) {
            for (int sl = Lq + lane; sl < t.q_slots; sl += 32)
              argmax[(int64_t)m.pair * t.q_slots + sl] = 0;
          }
        }
      }
      __syncwarp();  // every lane is done with slot s before lane 0 refills it
    }
    feed(s);
    if (it < kStages) __syncwarp();
  }
}

}  // namespace maxsim
