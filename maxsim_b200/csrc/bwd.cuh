// Backward kernels.  The forward saved one int32 argmax per (pair, query
// token); the backward routes g = dscore[pair] through it
// (maxsim_cuda/maxsim.cu:595-611, 1814-1828, 2153-2167):
//     grad_q[i]      += g * d[argmax[i]]
//     grad_d[argmax] += g * q[i]
// The reference issues 2*dim global float atomics per (pair, token).  Here:
//   * grad_q of the padded and contrastive layouts is a gather: every query
//     row has one owner warp that walks its candidates / documents and sums
//     in registers -- no atomics, one store per element, deterministic;
//   * grad_d of the padded layout has one owner warp per document slab;
//   * grad_d of the contrastive layout accumulates per document segment in
//     shared memory (one CTA per document chunk) and stores once;
//   * packed pair grids, whose pair list is arbitrary, use vector reductions
//     (red.global.add) after a zero fill.
#pragma once

#include "common.cuh"

namespace maxsim {

constexpr int kBwdWarps = 4;

template <typename T>
__device__ __forceinline__ void load4(const T* __restrict__ p, bool vec, int k, int dim,
                                      float (&out)[4]) {
  if (vec) {
    if constexpr (sizeof(T) == 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p + k));
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p + k));
      const T* e = reinterpret_cast<const T*>(&raw);
      out[0] = to_f32(e[0]); out[1] = to_f32(e[1]); out[2] = to_f32(e[2]); out[3] = to_f32(e[3]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) out[e] = (k + e < dim) ? to_f32(p[k + e]) : 0.0f;
  }
}

__device__ __forceinline__ void store4(float* __restrict__ p, bool vec, int k, int dim,
                                       const float (&v)[4]) {
  if (vec) {
    *reinterpret_cast<float4*>(p + k) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (k + e < dim) p[k + e] = v[e];
  }
}

// ---------------------------------------------------------------------------
// grad_q by gather (padded: over the C candidates of query b; contrastive:
// over the Nb documents).  One warp per query row; lanes own 4 consecutive
// dims of each 128-wide block.
// ---------------------------------------------------------------------------
template <typename T, int LAYOUT>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_dq_gather_kernel(PairTable t, const float* __restrict__ dscore,
                     const int32_t* __restrict__ argmax, float* __restrict__ dq,
                     int64_t n_rows, int vec_ok) {
  static_assert(LAYOUT == kPadded || LAYOUT == kContrastive, "gather needs grouped pairs");
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int dim = t.dim, slots = t.q_slots, C = t.C;
  const int64_t b = row / slots;  // query index
  const int i = (int)(row - b * slots);
  const int Lq = (LAYOUT == kPadded) ? __ldg(t.ia + b) : slots;
  const T* D = reinterpret_cast<const T*>(t.documents);
  const bool vec = vec_ok != 0;

  for (int kb = 0; kb < dim; kb += 128) {
    const int k = kb + lane * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (i < Lq) {
      for (int c0 = 0; c0 < C; c0 += 32) {
        // lane l stages candidate c0+l: weight and source row (or -1)
        const int c = c0 + lane;
        float gl = 0.f;
        int64_t src = -1;
        if (c < C) {
          const int64_t p = b * C + c;
          const int j = __ldg(argmax + p * slots + i);
          int64_t d_row0;
          int Ld;
          if (LAYOUT == kPadded) {
            d_row0 = p * (int64_t)t.Ld_max;
            Ld = __ldg(t.ib + p);
          } else {
            const int d0 = __ldg(t.ib + c);
            d_row0 = d0;
            Ld = __ldg(t.ib + c + 1) - d0;
          }
          if (j >= 0 && j < Ld) {
            src = d_row0 + j;
            gl = __ldg(dscore + p);
          }
        }
        const int n = min(32, C - c0);
        for (int l = 0; l < n; ++l) {
          const float gv = __shfl_sync(0xffffffffu, gl, l);
          const int64_t sr = __shfl_sync(0xffffffffu, src, l);
          if (sr >= 0 && k < dim) {
            float dv[4];
            load4<T>(D + sr * dim, vec, k, dim, dv);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(gv, dv[e], acc[e]);
          }
        }
      }
    }
    if (k < dim) store4(dq + row * dim, vec, k, dim, acc);
  }
}

// ---------------------------------------------------------------------------
// grad_d of the padded layout: document slab p belongs to pair p alone.
// One warp zero-fills the slab and then adds the (at most Lq) routed rows.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_dd_padded_kernel(PairTable t, const float* __restrict__ dscore,
                     const int32_t* __restrict__ argmax, float* __restrict__ dd, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t p = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (p >= t.n_pairs) return;
  const int dim = t.dim, slots = t.q_slots;
  const PairGeom g = pair_geom<kPadded>(t, p);
  float* slab = dd + p * (int64_t)t.Ld_max * dim;
  const int64_t slab_elems = (int64_t)t.Ld_max * dim;
  const bool vec = vec_ok != 0;
  if (vec) {
    float4* s4 = reinterpret_cast<float4*>(slab);
    for (int64_t e = lane; e < slab_elems / 4; e += 32) s4[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    for (int64_t e = lane; e < slab_elems; e += 32) slab[e] = 0.f;
  }
  __syncwarp();
  const float gv = __ldg(dscore + p);
  const T* Q = reinterpret_cast<const T*>(t.queries) + g.q_row0 * dim;
  for (int i = 0; i < g.Lq; ++i) {
    const int j = __ldg(argmax + p * slots + i);
    if (j < 0 || j >= g.Ld) continue;
    float* dst = slab + (int64_t)j * dim;
    for (int k = lane * 4; k < dim; k += 128) {
      float qv[4], cur[4];
      load4<T>(Q + (int64_t)i * dim, vec, k, dim, qv);
      if (vec) {
        const float4 c4 = *reinterpret_cast<const float4*>(dst + k);
        cur[0] = c4.x; cur[1] = c4.y; cur[2] = c4.z; cur[3] = c4.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) cur[e] = (k + e < dim) ? dst[k + e] : 0.f;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) cur[e] = fmaf(gv, qv[e], cur[e]);
      store4(dst, vec, k, dim, cur);
    }
    // the same lane owns the same dims of every row: no cross-lane hazard
  }
}

// ---------------------------------------------------------------------------
// Atomic routing (any layout).  One warp per pair.  Outputs must be zeroed.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

template <typename T, int LAYOUT, bool DO_DQ, bool DO_DD>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_route_atomic_kernel(PairTable t, const float* __restrict__ dscore,
                        const int32_t* __restrict__ argmax, float* __restrict__ dq,
                        float* __restrict__ dd, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t p = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (p >= t.n_pairs) return;
  const int dim = t.dim, slots = t.q_slots;
  const PairGeom g = pair_geom<LAYOUT>(t, p);
  const float gv = __ldg(dscore + p);
  const T* Q = reinterpret_cast<const T*>(t.queries) + g.q_row0 * dim;
  const T* D = reinterpret_cast<const T*>(t.documents) + g.d_row0 * dim;
  const bool vec = vec_ok != 0;
  for (int i = 0; i < g.Lq; ++i) {
    const int j = __ldg(argmax + p * slots + i);
    if (j < 0 || j >= g.Ld) continue;
    for (int k = lane * 4; k < dim; k += 128) {
      if (DO_DQ) {
        float dv[4];
        load4<T>(D + (int64_t)j * dim, vec, k, dim, dv);
        float* dst = dq + (g.q_row0 + i) * dim + k;
        if (vec) {
          red_add_v4(dst, gv * dv[0], gv * dv[1], gv * dv[2], gv * dv[3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (k + e < dim) atomicAdd(dst + e, gv * dv[e]);
        }
      }
      if (DO_DD) {
        float qv[4];
        load4<T>(Q + (int64_t)i * dim, vec, k, dim, qv);
        float* dst = dd + (g.d_row0 + j) * dim + k;
        if (vec) {
          red_add_v4(dst, gv * qv[0], gv * qv[1], gv * qv[2], gv * qv[3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (k + e < dim) atomicAdd(dst + e, gv * qv[e]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// grad_d of the contrastive layout by per-document shared-memory accumulation.
// CTA (d, chunk) owns kSegTokens document tokens of document d; its warps
// sweep all (query, token) argmax entries of that document, and every entry
// that lands in the chunk adds g * q_row into a shared fp32 tile with
// shared-memory reductions.  The tile is stored once, so grad_d needs no zero
// fill and no global atomics.
// ---------------------------------------------------------------------------
constexpr int kSegTokens = 64;
constexpr int kSegWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kSegWarps * 32)
bwd_dd_contrastive_kernel(PairTable t, const float* __restrict__ dscore,
                          const int32_t* __restrict__ argmax, float* __restrict__ dd,
                          int64_t Nq, int max_chunks, int vec_ok) {
  extern __shared__ __align__(16) float seg_smem[];  // [kSegTokens][dim]
  const int dim = t.dim, Lq = t.q_slots, Nb = t.C;
  const int d = blockIdx.x / max_chunks;
  const int chunk = blockIdx.x - d * max_chunks;
  const int d0 = __ldg(t.ib + d);
  const int Ld = __ldg(t.ib + d + 1) - d0;
  const int tok0 = chunk * kSegTokens;
  if (tok0 >= Ld) return;
  const int ntok = min(kSegTokens, Ld - tok0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool vec = vec_ok != 0;

  for (int e = threadIdx.x; e < ntok * dim; e += kSegWarps * 32) seg_smem[e] = 0.f;
  __syncthreads();

  const T* Q = reinterpret_cast<const T*>(t.queries);
  // entries (q, i) of this document, flattened: e = q*Lq + i.  Each warp takes
  // 32 consecutive entries at a time; lane l inspects entry e0+l.
  const int64_t n_entries = Nq * (int64_t)Lq;
  for (int64_t e0 = (int64_t)warp * 32; e0 < n_entries; e0 += kSegWarps * 32) {
    const int64_t e = e0 + lane;
    int j = -1;
    float gl = 0.f;
    if (e < n_entries) {
      const int64_t q = e / Lq;
      const int i = (int)(e - q * Lq);
      const int a = __ldg(argmax + (q * Nb + d) * (int64_t)Lq + i);
      if (a >= tok0 && a < tok0 + ntok) {
        j = a - tok0;
        gl = __ldg(dscore + q * Nb + d);
      }
    }
    unsigned hits = __ballot_sync(0xffffffffu, j >= 0);
    while (hits) {
      const int l = __ffs(hits) - 1;
      hits &= hits - 1;
      const int jj = __shfl_sync(0xffffffffu, j, l);
      const float gv = __shfl_sync(0xffffffffu, gl, l);
      const T* qrow = Q + (e0 + l) * dim;
      float* dst = seg_smem + jj * dim;
      for (int k = lane * 4; k < dim; k += 128) {
        float qv[4];
        load4<T>(qrow, vec, k, dim, qv);
#pragma unroll
        for (int x = 0; x < 4; ++x)
          if (k + x < dim) atomicAdd(dst + k + x, gv * qv[x]);
      }
    }
  }
  __syncthreads();
  float* out = dd + ((int64_t)d0 + tok0) * dim;
  for (int e = threadIdx.x; e < ntok * dim; e += kSegWarps * 32) out[e] = seg_smem[e];
}

}  // namespace maxsim
