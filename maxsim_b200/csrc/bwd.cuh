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
//   * grad_d of the contrastive layout inverts the argmax per document in
//     shared memory (counting sort of the entries by winning token) and then
//     gathers, one owner warp per document token, one store per row;
//   * packed pair grids, whose pair list is arbitrary: when the caller
//     supplies the list grouped by query and by document (group.cuh), grad_q
//     is the same gather over a query's group and grad_d has one owner warp
//     per document that zero-fills its rows and adds its group's routed rows;
//     otherwise vector reductions (red.global.add) after a zero fill.
#pragma once

#include <type_traits>

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

// Eight consecutive elements of a token row, kept packed in registers until
// they are used (a 16-bit row costs 4 registers, so eight rows can be in flight
// per lane).
template <typename T>
struct Row8 {
  uint4 a;
  __device__ __forceinline__ void load(const T* __restrict__ p) {
    a = __ldg(reinterpret_cast<const uint4*>(p));
  }
  __device__ __forceinline__ void zero() { a = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void fma_into(float g, float (&acc)[8]) const {
    const T* e = reinterpret_cast<const T*>(&a);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(g, to_f32(e[i]), acc[i]);
  }
};
template <>
struct Row8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* __restrict__ p) {
    a = __ldg(reinterpret_cast<const float4*>(p));
    b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void zero() { a = make_float4(0, 0, 0, 0); b = a; }
  __device__ __forceinline__ void fma_into(float g, float (&acc)[8]) const {
    acc[0] = fmaf(g, a.x, acc[0]); acc[1] = fmaf(g, a.y, acc[1]);
    acc[2] = fmaf(g, a.z, acc[2]); acc[3] = fmaf(g, a.w, acc[3]);
    acc[4] = fmaf(g, b.x, acc[4]); acc[5] = fmaf(g, b.y, acc[5]);
    acc[6] = fmaf(g, b.z, acc[6]); acc[7] = fmaf(g, b.w, acc[7]);
  }
};

// Store eight consecutive gradient elements, either as fp32 (the operators'
// contract) or rounded once to the inputs' 16-bit type (what autograd's cast of
// the fp32 gradient would produce, without the extra pass over memory).
template <typename T>
__device__ __forceinline__ void store8(void* row_base, int k, const float (&acc)[8], bool native) {
  if (native) {
    if constexpr (sizeof(T) == 2) {
      T h[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if constexpr (std::is_same<T, __half>::value) h[e] = __float2half_rn(acc[e]);
        else h[e] = __float2bfloat16_rn(acc[e]);
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(row_base) + k) = *reinterpret_cast<const uint4*>(h);
      return;
    }
  }
  float4* out = reinterpret_cast<float4*>(reinterpret_cast<float*>(row_base) + k);
  out[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  out[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
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
        // eight independent row loads in flight per lane before their FMAs
        for (int l0 = 0; l0 < n; l0 += 8) {
          float dv[8][4];
          float gw[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int l = (l0 + u) & 31;
            const float gv = __shfl_sync(0xffffffffu, gl, l);
            const int64_t sr = __shfl_sync(0xffffffffu, src, l);
            const bool ok = (l0 + u < n) && sr >= 0 && k < dim;
            gw[u] = ok ? gv : 0.f;
            if (ok) {
              load4<T>(D + sr * dim, vec, k, dim, dv[u]);
            } else {
              dv[u][0] = dv[u][1] = dv[u][2] = dv[u][3] = 0.f;
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(gw[u], dv[u][e], acc[e]);
        }
      }
    }
    if (k < dim) store4(dq + row * dim, vec, k, dim, acc);
  }
}

// ---------------------------------------------------------------------------
// grad_q gather, 16-bit element types with dim <= 128 and dim % 8 == 0.
// One warp per query row; each half-warp fetches one candidate's winning row
// with 128-bit loads (16 lanes x 8 elements), so a warp step covers two
// candidates and four rows are in flight per lane (more in flight costs
// occupancy and measured slower).
// A variant that cut the L2 traffic 3.5 times was measured and dropped: CTAs of
// 1024 query rows x 32 dims walking all documents, each document's 64-byte
// column slice staged once in shared memory (cp.async, three stages) and the
// rows gathered from there.  1024 x 1024 pairs, bf16: 1.81 ms against 0.76 ms
// for this kernel -- 16-byte reads of random rows keep the shared-memory pipe
// busier than L2 was, with one barrier per document on top.
// ---------------------------------------------------------------------------
// SPLIT > 1: that many warps of a block share a row, each taking every SPLIT-th block of 32
// candidates, and add their sums through shared memory -- for launches with too few rows to
// fill the GPU with one warp per row (a rank's share of the queries in a sharded step).
template <typename T, int LAYOUT, int SPLIT>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_dq_gather16_kernel(PairTable t, const float* __restrict__ dscore,
                       const int32_t* __restrict__ argmax, void* __restrict__ dq,
                       int64_t n_rows, int native) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  static_assert(SPLIT == 1 || SPLIT == 2 || SPLIT == 4, "SPLIT divides the warps of a block");
  const int lane = threadIdx.x & 31, half = lane >> 4, hl = lane & 15;
  const int warp = threadIdx.x >> 5;
  const int64_t row = ((int64_t)blockIdx.x * kBwdWarps + warp) / SPLIT;
  const int part = SPLIT > 1 ? warp % SPLIT : 0;
  const bool row_ok = row < n_rows;
  if (SPLIT == 1 && !row_ok) return;
  const int dim = t.dim, slots = t.q_slots, C = t.C;
  const int64_t b = row / slots;
  const int i = (int)(row - b * slots);
  const int Lq = (LAYOUT == kPadded) ? ((SPLIT == 1 || row_ok) ? __ldg(t.ia + b) : 0) : slots;
  const T* D = reinterpret_cast<const T*>(t.documents);
  const int k = hl * 8;
  const bool k_ok = k < dim;
  // Lanes past the row's last element (dim < 128) fetch column 0 again and their sums are
  // never stored: every load of the inner loops stays unconditional (a per-lane test there
  // cost the kernel three quarters of its rate).
  const int kk = k_ok ? k : 0;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;

  if ((SPLIT == 1 || row_ok) && i < Lq) {
    for (int c0 = part * 32; c0 < C; c0 += 32 * SPLIT) {
      const int c = c0 + lane;
      float gl = 0.f;
      int32_t src = -1;  // winning document row of candidate c0+lane, or -1
      if (c < C) {
        const int64_t p = b * C + c;
        const int j = __ldg(argmax + p * slots + i);
        int32_t d_row0, Ld;
        if (LAYOUT == kPadded) {
          d_row0 = (int32_t)(p * t.Ld_max);
          Ld = __ldg(t.ib + p);
        } else {
          d_row0 = __ldg(t.ib + c);
          Ld = __ldg(t.ib + c + 1) - d_row0;
        }
        if (j >= 0 && j < Ld) {
          src = d_row0 + j;
          gl = __ldg(dscore + p);
        }
      }
      const int n = min(32, C - c0);
      // (only the warp-uniform n == 32 stands before the vote: a lane-dependent test there,
      // such as k_ok with dim < 128, would let lanes skip it.  Taking the vote into a variable
      // ahead of the branch instead measured 1.06 ms against 0.78 ms on 1024 x 1024 pairs.)
      if (n == 32 && __all_sync(0xffffffffu, src >= 0)) {
        // all 32 candidates routed (the usual case): no per-row checks
#pragma unroll 1
        for (int l0 = 0; l0 < 32; l0 += 8) {
          Row8<T> rows[4];
          float gw[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int l = l0 + 2 * u + half;
            gw[u] = __shfl_sync(0xffffffffu, gl, l);
            const int32_t sr = __shfl_sync(0xffffffffu, src, l);
            rows[u].load(D + (int64_t)sr * dim + kk);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) rows[u].fma_into(gw[u], acc);
        }
        continue;
      }
      for (int l0 = 0; l0 < n; l0 += 8) {
        Row8<T> rows[4];
        float gw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int l = (l0 + 2 * u + half) & 31;
          const float gv = __shfl_sync(0xffffffffu, gl, l);
          const int32_t sr = __shfl_sync(0xffffffffu, src, l);
          const bool ok = (l0 + 2 * u + half < n) && sr >= 0;
          gw[u] = ok ? gv : 0.f;
          rows[u].zero();
          if (ok) rows[u].load(D + (int64_t)sr * dim + kk);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) rows[u].fma_into(gw[u], acc);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 16);
  if constexpr (SPLIT > 1) {
    __shared__ float partial[kBwdWarps][16][8];
    if (part != 0 && half == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) partial[warp][hl][e] = acc[e];
    }
    __syncthreads();
    if (part != 0 || !row_ok) return;
    if (half == 0) {
#pragma unroll
      for (int w = 1; w < SPLIT; ++w)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += partial[warp + w][hl][e];
    }
  }
  if (half == 0 && k_ok) {
    void* row_base = native ? static_cast<void*>(reinterpret_cast<T*>(dq) + row * dim)
                            : static_cast<void*>(reinterpret_cast<float*>(dq) + row * dim);
    store8<T>(row_base, k, acc, native != 0);
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

// grad_d of the padded layout, rows written once in the inputs' 16-bit type.
// One warp per slab, for Lq_max <= 32 and Ld_max <= 1024: lane i holds the
// winning token of query token i; tokens that won the same document token are
// found with a warp match, their query rows are summed in registers and the
// row is stored once, rounded once; rows nobody won are zero-filled from a
// bitmap.  Same values as casting the fp32 operator's result, without its
// read-modify-writes, its fp32 tensor and the cast's pass over it.
template <typename T>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_dd_padded_native_kernel(PairTable t, const float* __restrict__ dscore,
                            const int32_t* __restrict__ argmax, T* __restrict__ dd) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  const int lane = threadIdx.x & 31;
  const int64_t p = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (p >= t.n_pairs) return;
  const int dim = t.dim, slots = t.q_slots, Ld_max = t.Ld_max;
  const PairGeom g = pair_geom<kPadded>(t, p);
  T* slab = dd + p * (int64_t)Ld_max * dim;
  const float gv = __ldg(dscore + p);
  const T* Q = reinterpret_cast<const T*>(t.queries) + g.q_row0 * dim;

  int jl = -1;
  if (lane < g.Lq) {
    jl = __ldg(argmax + p * slots + lane);
    if (jl < 0 || jl >= g.Ld) jl = -1;
  }
  const unsigned same = __match_any_sync(0xffffffffu, jl);
  const bool leader = jl >= 0 && lane == (__ffs(same) - 1);
  unsigned leaders = __ballot_sync(0xffffffffu, leader);
  uint32_t written = 0u;  // lane w: rows 32w .. 32w+31
  while (leaders) {
    const int l = __ffs(leaders) - 1;
    leaders &= leaders - 1;
    const int j = __shfl_sync(0xffffffffu, jl, l);
    unsigned members = __shfl_sync(0xffffffffu, same, l);
    if (lane == (j >> 5)) written |= 1u << (j & 31);
    for (int k = lane * 4; k < dim; k += 128) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned mm = members;
      while (mm) {
        const int i = __ffs(mm) - 1;
        mm &= mm - 1;
        float qv[4];
        load4<T>(Q + (int64_t)i * dim, true, k, dim, qv);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = fmaf(gv, qv[e], acc[e]);  // same order as the fp32 kernel
      }
      T h[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if constexpr (std::is_same<T, __half>::value) h[e] = __float2half_rn(acc[e]);
        else h[e] = __float2bfloat16_rn(acc[e]);
      }
      *reinterpret_cast<uint2*>(slab + (int64_t)j * dim + k) = *reinterpret_cast<const uint2*>(h);
    }
  }
  for (int w = 0; w * 32 < Ld_max; ++w) {
    uint32_t missing = ~__shfl_sync(0xffffffffu, written, w);
    if (Ld_max - w * 32 < 32) missing &= (1u << (Ld_max - w * 32)) - 1u;
    while (missing) {
      const int r = w * 32 + __ffs(missing) - 1;
      missing &= missing - 1;
      for (int k = lane * 4; k < dim; k += 128)
        *reinterpret_cast<uint2*>(slab + (int64_t)r * dim + k) = make_uint2(0u, 0u);
    }
  }
}

// ---------------------------------------------------------------------------
// Packed pair lists with groups (t.order_q / ends_q / order_d / ends_d set).
// Needs dim % 8 == 0 and 16-byte aligned bases.  Both kernels write every
// output row exactly once: no zero fill, no atomics, same sums on every run up
// to the order of a group's members.
// ---------------------------------------------------------------------------

// grad_q: one warp per (query, token slot).  Each half-warp fetches one pair's
// winning document row with 128-bit loads; four rows in flight per lane.
template <typename T>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_dq_packed_kernel(PairTable t, const float* __restrict__ dscore,
                     const int32_t* __restrict__ argmax, void* __restrict__ dq,
                     int64_t n_queries, int native) {
  const int lane = threadIdx.x & 31, half = lane >> 4, hl = lane & 15;
  const int dim = t.dim, slots = t.q_slots;
  const int64_t row = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (row >= n_queries * slots) return;
  const int64_t b = row / slots;
  const int i = (int)(row - b * slots);
  const int q0 = __ldg(t.ia + b);
  const int Lq = min(__ldg(t.ia + b + 1) - q0, slots);
  if (i >= Lq) return;
  const int beg = b ? __ldg(t.ends_q + b - 1) : 0;
  const int C = __ldg(t.ends_q + b) - beg;
  const T* D = reinterpret_cast<const T*>(t.documents);

  for (int kb = 0; kb < dim; kb += 128) {
    const int k = kb + hl * 8;
    const bool k_ok = k < dim;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int c0 = 0; c0 < C; c0 += 32) {
      const int c = c0 + lane;
      float gl = 0.f;
      int32_t src = -1;  // winning document row of the group's member c0+lane, or -1
      if (c < C) {
        const int64_t p = __ldg(t.order_q + beg + c);
        const int j = __ldg(argmax + p * slots + i);
        const int di = __ldg(t.id + p);
        const int d0 = __ldg(t.ib + di);
        const int Ld = __ldg(t.ib + di + 1) - d0;
        if (j >= 0 && j < Ld) {
          src = d0 + j;
          gl = __ldg(dscore + p);
        }
      }
      const int n = min(32, C - c0);
      for (int l0 = 0; l0 < n; l0 += 8) {
        Row8<T> rows[4];
        float gw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int l = (l0 + 2 * u + half) & 31;
          const float gv = __shfl_sync(0xffffffffu, gl, l);
          const int32_t sr = __shfl_sync(0xffffffffu, src, l);
          const bool ok = (l0 + 2 * u + half < n) && sr >= 0 && k_ok;
          gw[u] = ok ? gv : 0.f;
          rows[u].zero();
          if (ok) rows[u].load(D + (int64_t)sr * dim + k);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) rows[u].fma_into(gw[u], acc);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 16);
    if (half == 0 && k_ok) {
      const int64_t r = (int64_t)q0 + i;
      void* row_base = native ? static_cast<void*>(reinterpret_cast<T*>(dq) + r * dim)
                              : static_cast<void*>(reinterpret_cast<float*>(dq) + r * dim);
      store8<T>(row_base, k, acc, native != 0);
    }
  }
}

// grad_d: one warp per document.  The warp walks the document's group: for
// every pair, the winning token of each query token receives g * q_i.  A bitmap
// (lane w keeps the word of rows 32w .. 32w+31) records which rows were
// written: the first contribution to a row is a plain store, later ones
// read-modify-write it, and rows that got none are zero-filled at the end --
// so most rows are written exactly once and there is no window between a
// zero-fill pass and the updates in which the lines could leave L2.  Lane l
// owns dims [4l, 4l+4) (+128 m) of every row, so an update is private to a
// lane and needs no atomics; the query rows of four tokens are fetched ahead
// of their updates.
constexpr int kDdPassRows = 1024;  // rows covered by one pass of the bitmap

template <typename T>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_dd_packed_kernel(PairTable t, const float* __restrict__ dscore,
                     const int32_t* __restrict__ argmax, float* __restrict__ dd,
                     int64_t n_documents) {
  const int lane = threadIdx.x & 31;
  const int dim = t.dim, slots = t.q_slots;
  const int64_t b = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (b >= n_documents) return;
  const int d0 = __ldg(t.ib + b);
  const int Ld = max(0, __ldg(t.ib + b + 1) - d0);
  const int beg = b ? __ldg(t.ends_d + b - 1) : 0;
  const int C = __ldg(t.ends_d + b) - beg;
  const T* Q = reinterpret_cast<const T*>(t.queries);
  const int dim4 = dim >> 2;

  for (int row0 = 0; row0 < Ld; row0 += kDdPassRows) {
    const int nrows = min(kDdPassRows, Ld - row0);
    float4* base4 = reinterpret_cast<float4*>(dd + ((int64_t)d0 + row0) * dim);
    uint32_t written = 0u;  // this lane's word of the bitmap
    int32_t m_p = 0, m_q0 = 0, m_Lq = 0;
    float m_g = 0.f;
    for (int c = 0; c < C; ++c) {
      // lane l fetches the geometry of the group's member c + l: one chain of
      // dependent loads per 32 pairs instead of one per pair
      if ((c & 31) == 0) {
        m_p = 0; m_g = 0.f; m_q0 = 0; m_Lq = 0;
        if (c + lane < C) {
          m_p = __ldg(t.order_d + beg + c + lane);
          m_g = __ldg(dscore + m_p);
          const int qi = __ldg(t.ic + m_p);
          m_q0 = __ldg(t.ia + qi);
          m_Lq = min(__ldg(t.ia + qi + 1) - m_q0, slots);
        }
      }
      const int64_t p = __shfl_sync(0xffffffffu, m_p, c & 31);
      const float gv = __shfl_sync(0xffffffffu, m_g, c & 31);
      const int q0 = __shfl_sync(0xffffffffu, m_q0, c & 31);
      const int Lq = __shfl_sync(0xffffffffu, m_Lq, c & 31);
      for (int i0 = 0; i0 < Lq; i0 += 32) {
        int jl = -1;
        if (i0 + lane < Lq) {
          jl = __ldg(argmax + p * slots + i0 + lane) - row0;
          if (jl < 0 || jl >= nrows) jl = -1;
        }
        const int n = min(32, Lq - i0);
        const T* qrow = Q + ((int64_t)q0 + i0) * dim;
        for (int kb = 0; kb < dim; kb += 128) {
          const int k = kb + lane * 4;
          const bool k_ok = k < dim;
          uint32_t seen = written;  // rows written before this (pair, i0) block
          for (int u0 = 0; u0 < n; u0 += 4) {
            int j[4];
            float qv[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              j[u] = __shfl_sync(0xffffffffu, jl, (u0 + u) & 31);
              if (u0 + u >= n) j[u] = -1;
              qv[u][0] = qv[u][1] = qv[u][2] = qv[u][3] = 0.f;
              if (j[u] >= 0 && k_ok) load4<T>(qrow + (u0 + u) * dim, true, k, dim, qv[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (j[u] < 0) continue;  // uniform: j comes from a shuffle
              const uint32_t word = __shfl_sync(0xffffffffu, seen, j[u] >> 5);
              const bool fresh = ((word >> (j[u] & 31)) & 1u) == 0u;
              if (lane == (j[u] >> 5)) seen |= 1u << (j[u] & 31);
              if (k_ok) {
                float4* dst = base4 + j[u] * dim4 + (k >> 2);
                float4 cur = make_float4(0.f, 0.f, 0.f, 0.f);
                if (!fresh) cur = *dst;
                cur.x = fmaf(gv, qv[u][0], cur.x);
                cur.y = fmaf(gv, qv[u][1], cur.y);
                cur.z = fmaf(gv, qv[u][2], cur.z);
                cur.w = fmaf(gv, qv[u][3], cur.w);
                *dst = cur;
              }
            }
          }
          if (kb + 128 >= dim) written = seen;  // every 128-wide block replays the same rows
        }
      }
    }
    // rows nobody routed to
    for (int w = 0; w * 32 < nrows; ++w) {
      uint32_t missing = ~__shfl_sync(0xffffffffu, written, w);
      if (nrows - w * 32 < 32) missing &= (1u << (nrows - w * 32)) - 1u;
      while (missing) {
        const int r = w * 32 + __ffs(missing) - 1;
        missing &= missing - 1;
        for (int k = lane * 4; k < dim; k += 128)
          base4[r * dim4 + (k >> 2)] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  }
}

// grad_d of a grouped packed list with every row written once, in the inputs'
// 16-bit type.  One warp per document.  The warp collects the routed terms of
// the document's pairs -- (winning token, query row, weight) -- in its slice of
// shared memory, one lane threads them into per-token lists (last term first,
// so every list runs in the order of the pair list: the same sums on every
// run), and the two half-warps walk the tokens, each summing a token's list in
// registers and storing the row once, rounded once; tokens nobody won are
// stored as zeros.  No read-modify-write of the gradient, no zero-fill pass, no
// fp32 tensor for autograd to cast afterwards.
// The slice holds kPdnCap terms.  A document with more routed terms is done in
// ranges of tokens: when the terms of a range do not fit, the range is halved
// and collected again, so every row still meets all of its terms in one piece;
// a single token with more than kPdnCap terms is summed over several batches
// in the registers of the half-warp that owns it.  Documents longer than
// kPdnMaxTok tokens take one window of tokens at a time.
constexpr int kPdnCap = 512;
constexpr int kPdnMaxTok = 1024;
struct __align__(16) PdnWarp {
  float g[kPdnCap];
  int32_t qrow[kPdnCap];
  uint16_t tok[kPdnCap];
  uint16_t next[kPdnCap];
  uint16_t head[kPdnMaxTok];
};
constexpr uint16_t kPdnNil = 0xFFFF;

template <typename T>
__global__ void __launch_bounds__(kBwdWarps * 32)
bwd_dd_packed_native_kernel(PairTable t, const float* __restrict__ dscore,
                            const int32_t* __restrict__ argmax, T* __restrict__ dd,
                            int64_t n_documents) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  extern __shared__ __align__(16) unsigned char pdn_smem[];
  PdnWarp& W = reinterpret_cast<PdnWarp*>(pdn_smem)[threadIdx.x >> 5];
  const int lane = threadIdx.x & 31, half = lane >> 4, hl = lane & 15;
  const int dim = t.dim, slots = t.q_slots;
  const int64_t b = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (b >= n_documents) return;
  const int d0 = __ldg(t.ib + b);
  const int Ld = max(0, __ldg(t.ib + b + 1) - d0);
  const int beg = b ? __ldg(t.ends_d + b - 1) : 0;
  const int C = __ldg(t.ends_d + b) - beg;
  const T* Q = reinterpret_cast<const T*>(t.queries);
  const int k = hl * 8;
  const bool k_ok = k < dim;

  // Collect the terms whose token lies in [lo, lo + width) of the document, starting at block
  // (c, i0) of the group (pair c, query tokens from i0), until the group ends or the slice is
  // full; the lists are then threaded.  Returns the number of terms; c < C afterwards means
  // that terms were left out.
  auto collect = [&](int lo, int width, int& c, int& i0) -> int {
    for (int h = lane; h < width; h += 32) W.head[h] = kPdnNil;
    int E = 0;
    while (c < C && E + 32 <= kPdnCap) {
      const int p = __ldg(t.order_d + beg + c);
      const int qi = __ldg(t.ic + p);
      const int q0 = __ldg(t.ia + qi);
      const int Lq = min(__ldg(t.ia + qi + 1) - q0, slots);
      const int i = i0 + lane;
      int tk = -1;
      if (i < Lq) {
        const int a = __ldg(argmax + (int64_t)p * slots + i);
        if (a >= lo && a < lo + width && a < Ld) tk = a - lo;
      }
      const unsigned routed = __ballot_sync(0xffffffffu, tk >= 0);
      if (tk >= 0) {
        const int pos = E + __popc(routed & ((1u << lane) - 1u));
        W.tok[pos] = (uint16_t)tk;
        W.qrow[pos] = q0 + i;
        W.g[pos] = __ldg(dscore + p);
      }
      E += __popc(routed);
      i0 += 32;
      if (i0 >= Lq) { ++c; i0 = 0; }
    }
    __syncwarp();
    if (lane == 0) {
      for (int e = E - 1; e >= 0; --e) {
        const int tk = W.tok[e];
        W.next[e] = W.head[tk];
        W.head[tk] = (uint16_t)e;
      }
    }
    __syncwarp();
    return E;
  };
  // acc += the terms of the list that starts at e (this half-warp's 8 dims per lane)
  auto sum_list = [&](int e, float (&acc)[8]) {
    while (e != kPdnNil) {
      Row8<T> rows[4];  // up to four terms fetched together
      float gw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        rows[u].zero();
        gw[u] = 0.f;
        if (e != kPdnNil) {
          gw[u] = W.g[e];
          if (k_ok) rows[u].load(Q + (int64_t)W.qrow[e] * dim + k);
          e = W.next[e];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) rows[u].fma_into(gw[u], acc);
    }
  };

  for (int w0 = 0; w0 < Ld; w0 += kPdnMaxTok) {
    const int nw = min(kPdnMaxTok, Ld - w0);
    int lo = 0, width = nw;
    while (lo < nw) {
      width = min(width, nw - lo);
      int c = 0, i0 = 0;
      collect(w0 + lo, width, c, i0);
      if (c < C && width > 1) {  // the terms of this range do not fit: a narrower one
        width >>= 1;
        continue;
      }
      if (c >= C) {
        // every term of the range is in the lists: one store per row
        for (int j = half; j < width; j += 2) {
          float acc[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) acc[x] = 0.f;
          sum_list(W.head[j], acc);
          if (k_ok) store8<T>(dd + ((int64_t)d0 + w0 + lo + j) * dim, k, acc, true);
        }
        __syncwarp();
      } else {
        // one token with more terms than the slice holds: batches, summed in registers
        float acc[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) acc[x] = 0.f;
        for (;;) {
          if (half == 0) sum_list(W.head[0], acc);
          __syncwarp();
          if (c >= C) break;
          collect(w0 + lo, 1, c, i0);
        }
        if (half == 0 && k_ok) store8<T>(dd + ((int64_t)d0 + w0 + lo) * dim, k, acc, true);
      }
      lo += width;
      width = min(2 * width, nw);  // try a wider range again
    }
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
  const int64_t pos = (int64_t)blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
  if (pos >= t.n_pairs) return;
  const int64_t p = pair_at<LAYOUT>(t, pos);
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
// grad_d of the contrastive layout: invert the argmax in shared memory, then
// gather.  grad_d[d, j] = sum over the (query, token) entries whose argmax is
// j of g[q, d] * Q[q, i].  A scatter of that sum would need atomics; instead
// one CTA per document counting-sorts the document's Nq*Lq argmax entries by
// winning token inside shared memory (histogram, scan, scatter of entry ids),
// after which every document token owns a contiguous list of the query rows
// routed to it.  Warps then take tokens one at a time and sum their lists in
// registers -- a pure gather (two 128-bit row loads per warp step, eight rows
// in flight per lane) with exactly one store per gradient row.  No global
// atomics, no scratch in global memory, no zero-fill pass.
//
// Entries are processed in passes of at most kInvEntries (query blocks) and
// documents longer than kInvBins tokens in token chunks; later passes add to
// the rows the first pass stored.
// ---------------------------------------------------------------------------
// Sized for two CTAs per SM (88 KB of shared memory and at most 64 registers
// per thread), so that one document's histogram / scan / scatter phases, which
// wait on memory and barriers, overlap the other's gather.
constexpr int kInvThreads = 512;
constexpr int kInvEntries = 32768;  // entry ids held per pass (16-bit ids: 64 KB)
constexpr int kInvBins = 2048;      // document tokens per chunk
constexpr int kInvMaxQ = 2048;      // queries per pass (g column held in shared memory)

constexpr size_t inv_smem_bytes() {
  return (size_t)kInvEntries * 2 + (size_t)kInvMaxQ * 4 + (size_t)(2 * kInvBins + 2) * 4 + 16;
}
static_assert(kInvEntries <= 65536, "entry ids are stored in 16 bits");

// Grid rows per document for `documents` documents of `mean_tokens` tokens on
// `sms` SMs (two CTAs each).  With at least half as many documents as CTA slots:
// one CTA per document (two for very long documents), chunks of kInvBins tokens.
// With fewer: up to eight CTAs per document, each taking an even share of its
// tokens (*split = 1).
inline void inv_grid_shape(int64_t documents, int64_t mean_tokens, int sms, int* gy, int* split) {
  const int64_t slots = 2ll * sms;
  *gy = mean_tokens > kInvBins ? 2 : 1;
  *split = 0;
  if (documents > 0 && documents * 2 <= slots && mean_tokens <= kInvBins) {
    int64_t rows = slots / documents;
    if (rows > 8) rows = 8;
    *gy = (int)rows;
    *split = 1;
  }
}

template <typename T>
__global__ void __launch_bounds__(kInvThreads, 2)
bwd_dd_invert_kernel(PairTable t, const float* __restrict__ dscore,
                     const int32_t* __restrict__ argmax, void* __restrict__ dd_out, int Nq,
                     int native, int split, int rec_stride) {
  // rec_stride > 0: `argmax` holds one record of rec_stride words per pair -- the Lq
  // winning tokens followed by the bits of the pair's score gradient -- and `dscore`
  // is not read (the form in which a rank receives the pairs of its own documents
  // from the ranks that hold the queries).
  // CTA (d, y) takes the token chunks y, y + gridDim.y, ... of document d.  A chunk
  // is kInvBins tokens, or, with `split` set (few documents, several CTAs per
  // document), an even share of the document.
  // `native` (rows stored once, in the inputs' type) is only given when all
  // entries of a document fit one pass; the fp32 form adds later passes in place.
  float* dd = reinterpret_cast<float*>(dd_out);
  extern __shared__ __align__(16) unsigned char inv_smem[];
  uint16_t* list = reinterpret_cast<uint16_t*>(inv_smem);               // [kInvEntries]
  float* gcol = reinterpret_cast<float*>(list + kInvEntries);          // [kInvMaxQ]
  int32_t* bin_start = reinterpret_cast<int32_t*>(gcol + kInvMaxQ);    // [kInvBins + 1]
  int32_t* cursor = bin_start + kInvBins + 1;                          // [kInvBins]
  int32_t* next_tok = cursor + kInvBins;                               // [1]

  const int dim = t.dim, Lq = t.q_slots, Nb = t.C;
  const int d = blockIdx.x;
  const int d0 = __ldg(t.ib + d);
  const int Ld = __ldg(t.ib + d + 1) - d0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = lane >> 4, hl = lane & 15;
  const T* Q = reinterpret_cast<const T*>(t.queries);
  int q_block = kInvEntries / Lq;
  if (q_block > kInvMaxQ) q_block = kInvMaxQ;
  if (q_block < 1) q_block = 1;  // the dispatcher guarantees Lq <= kInvEntries

  const int bins = split ? min(kInvBins, (Ld + (int)gridDim.y - 1) / (int)gridDim.y) : kInvBins;
  for (int tok0 = blockIdx.y * bins; tok0 < Ld; tok0 += gridDim.y * bins) {
    const int ntok = min(bins, Ld - tok0);
    for (int q0 = 0; q0 < Nq; q0 += q_block) {
      const int nq = min(q_block, Nq - q0);
      const int n_e = nq * Lq;
      const int rs = rec_stride > 0 ? rec_stride : Lq;                // words per pair in `argmax`
      const int32_t* amax = argmax + ((int64_t)q0 * Nb + d) * rs;     // entry (q, i) at amax[q*Nb*rs + i]
      __syncthreads();
      for (int b = tid; b < ntok; b += kInvThreads) cursor[b] = 0;
      for (int qq = tid; qq < nq; qq += kInvThreads)
        gcol[qq] = rec_stride > 0 ? __int_as_float(__ldg(amax + (int64_t)qq * Nb * rs + Lq))
                                  : __ldg(dscore + (int64_t)(q0 + qq) * Nb + d);
      if (tid == 0) *next_tok = 0;
      __syncthreads();
      // histogram of winning tokens
      for (int e0 = tid; e0 < n_e; e0 += 4 * kInvThreads) {
        int a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {  // four independent loads in flight
          const int e = e0 + u * kInvThreads;
          a[u] = -1;
          if (e < n_e) {
            const int qq = e / Lq, i = e - qq * Lq;
            a[u] = __ldg(amax + (int64_t)qq * Nb * rs + i) - tok0;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (a[u] >= 0 && a[u] < ntok) atomicAdd(&cursor[a[u]], 1);
      }
      __syncthreads();
      // exclusive scan over the bins (one warp, contiguous slices per lane)
      if (warp == 0) {
        const int per = (ntok + 31) / 32;
        const int b0 = lane * per, b1 = min(ntok, b0 + per);
        int sum = 0;
        for (int b = b0; b < b1; ++b) sum += cursor[b];
        int incl = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int o = __shfl_up_sync(0xffffffffu, incl, off);
          if (lane >= off) incl += o;
        }
        int run = incl - sum;
        for (int b = b0; b < b1; ++b) {
          const int c = cursor[b];
          bin_start[b] = run;
          cursor[b] = run;
          run += c;
        }
        if (lane == 31) bin_start[ntok] = incl;
      }
      __syncthreads();
      // scatter entry ids into their token's list
      for (int e0 = tid; e0 < n_e; e0 += 4 * kInvThreads) {
        int a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int e = e0 + u * kInvThreads;
          a[u] = -1;
          if (e < n_e) {
            const int qq = e / Lq, i = e - qq * Lq;
            a[u] = __ldg(amax + (int64_t)qq * Nb * rs + i) - tok0;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (a[u] >= 0 && a[u] < ntok)
            list[atomicAdd(&cursor[a[u]], 1)] = (uint16_t)(e0 + u * kInvThreads);
      }
      __syncthreads();
      // gather: warps claim tokens; each half-warp fetches one routed query row
      const int lq_shift = (Lq & (Lq - 1)) == 0 ? (31 - __clz(Lq)) : -1;  // Lq a power of two
      const T* qpass = Q + (int64_t)q0 * Lq * dim;
      for (;;) {
        int j = 0;
        if (lane == 0) j = atomicAdd(next_tok, 1);
        j = __shfl_sync(0xffffffffu, j, 0);
        if (j >= ntok) break;
        const int beg = bin_start[j], end = bin_start[j + 1];
        float* out = dd + ((int64_t)d0 + tok0 + j) * dim;
        for (int kb = 0; kb < dim; kb += 128) {
          const int k = kb + hl * 8;
          const bool k_ok = k < dim;
          const T* qk = qpass + k;
          float acc[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) acc[x] = 0.f;
          constexpr int kFlight = sizeof(T) == 2 ? 4 : 2;  // rows in flight per lane
          int p = beg + half;
          if (k_ok) {
            // full groups: no bounds checks
            for (; p + 2 * (kFlight - 1) < end; p += 2 * kFlight) {
              Row8<T> rows[kFlight];
              float gw[kFlight];
#pragma unroll
              for (int u = 0; u < kFlight; ++u) {
                const int e = list[p + 2 * u];
                gw[u] = gcol[lq_shift >= 0 ? (e >> lq_shift) : (e / Lq)];
                rows[u].load(qk + (int64_t)e * dim);
              }
#pragma unroll
              for (int u = 0; u < kFlight; ++u) rows[u].fma_into(gw[u], acc);
            }
            // tail: one more group with its loads issued together, absent rows weighted 0
            if (p < end) {
              Row8<T> rows[kFlight];
              float gw[kFlight];
#pragma unroll
              for (int u = 0; u < kFlight; ++u) {
                const bool has = p + 2 * u < end;
                const int e = has ? list[p + 2 * u] : 0;
                gw[u] = has ? gcol[lq_shift >= 0 ? (e >> lq_shift) : (e / Lq)] : 0.f;
                rows[u].zero();
                if (has) rows[u].load(qk + (int64_t)e * dim);
              }
#pragma unroll
              for (int u = 0; u < kFlight; ++u) rows[u].fma_into(gw[u], acc);
            }
          }
#pragma unroll
          for (int x = 0; x < 8; ++x) acc[x] += __shfl_xor_sync(0xffffffffu, acc[x], 16);
          if (half == 0 && k_ok && native) {
            store8<T>(reinterpret_cast<T*>(dd_out) + ((int64_t)d0 + tok0 + j) * dim, k, acc, true);
          } else if (half == 0 && k_ok) {
            float4* o4 = reinterpret_cast<float4*>(out + k);
            if (q0 == 0) {
              o4[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
              o4[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            } else {
              float4 c0 = o4[0], c1 = o4[1];
              o4[0] = make_float4(c0.x + acc[0], c0.y + acc[1], c0.z + acc[2], c0.w + acc[3]);
              o4[1] = make_float4(c1.x + acc[4], c1.y + acc[5], c1.z + acc[6], c1.w + acc[7]);
            }
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Sharded contrastive training, owner exchange: the pairs of this rank's
// queries are regrouped by the rank that owns the document.  Owner o's block
// starts at word col_start[o] * Nq * (Lq + 1) of `send` and is laid out
// [query][document of o][Lq + 1]: the Lq winning tokens of the pair and the
// bits of its score gradient.  Blocks of all ranks' queries, concatenated in
// rank order by the all-to-all, are the [all queries][own documents][Lq + 1]
// tensor that bwd_dd_invert_kernel reads with rec_stride = Lq + 1.
// One thread per word of `send`; blockIdx.y is the owner, so that its column
// range is uniform over the block and both sides of the copy are coalesced.
// ---------------------------------------------------------------------------
// With `owner_blocks` the block of owner o is written to owner_blocks[o] instead: the
// pointers are into the owners' own memory (peer mappings), so the kernel's stores are the
// transfer and no send buffer or all-to-all exists.
__global__ void __launch_bounds__(256)
pack_owner_records_kernel(const int32_t* __restrict__ argmax, const float* __restrict__ dscore,
                          const int32_t* __restrict__ col_start, int Nq, int Nb, int Lq,
                          int32_t* __restrict__ send, int32_t* const* __restrict__ owner_blocks) {
  const int o = blockIdx.y;
  const int c0 = __ldg(col_start + o), n_o = __ldg(col_start + o + 1) - c0;
  const int rec = Lq + 1;
  const int64_t words = (int64_t)Nq * n_o * rec;          // of this owner's block
  int32_t* dst = owner_blocks ? owner_blocks[o] : send + (int64_t)c0 * Nq * rec;
  const int64_t per_query = (int64_t)n_o * rec;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words;
       w += (int64_t)gridDim.x * blockDim.x) {
    const int q = (int)(w / per_query);
    const int r = (int)(w - (int64_t)q * per_query);
    const int dl = r / rec, slot = r - dl * rec;
    const int64_t pair = (int64_t)q * Nb + c0 + dl;
    dst[w] = slot < Lq ? __ldg(argmax + pair * Lq + slot) : __float_as_int(__ldg(dscore + pair));
  }
}

// ---------------------------------------------------------------------------
// Barrier between the ranks of one node over flags in peer-mapped memory.
// flags[r] points at rank r's flag words (one per rank) as mapped into this
// process; thread t tells rank t that this rank has reached its next barrier
// (a release store at system scope into flags[t][rank], after the stream's
// earlier stores to peer memory) and waits until rank t has said the same
// (flags[rank][t] >= epoch; epochs only grow, so a peer that is already one
// barrier ahead satisfies the wait too).  The epoch is the number of barriers
// this rank has passed plus one, kept in `counter` on the device -- not a
// launch argument, so that a barrier captured in a CUDA graph counts on at
// every replay.  The wait is bounded: after `limit` polls the kernel sets bit 4
// of the status word and returns.
// ---------------------------------------------------------------------------
__global__ void peer_barrier_kernel(uint32_t* const* __restrict__ flags, int rank, int world,
                                    uint32_t* __restrict__ counter, uint32_t limit) {
  const int t = threadIdx.x;
  const uint32_t epoch = *counter + 1;
  __syncthreads();  // every thread has read the old count
  if (t == 0) *counter = epoch;
  if (t >= world || t == rank) return;
  __threadfence_system();
  uint32_t* theirs = flags[t] + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const uint32_t* mine = flags[rank] + t;
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - epoch) >= 0) break;
    if (it >= limit) {
      atomicOr(&g_device_status, 4);
      break;
    }
    __nanosleep(200);
  }
}

// ---------------------------------------------------------------------------
// Gather of small segments out of peer-mapped memory with plain loads: the
// document lengths and the queries of all ranks in one launch each instead of
// one copy per rank.  table[s] = {source address, which destination (0 / 1),
// byte offset in it, bytes}; bytes are a multiple of 4, and 16-byte words are
// used when source, destination and size allow.  blockIdx.y is the segment.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
peer_gather_kernel(const int64_t* __restrict__ table, void* __restrict__ dst0,
                   void* __restrict__ dst1) {
  const int64_t* row = table + 4 * (int64_t)blockIdx.y;
  const char* src = reinterpret_cast<const char*>(row[0]);
  char* dst = reinterpret_cast<char*>(row[1] ? dst1 : dst0) + row[2];
  const int64_t bytes = row[3];
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  const bool wide = (((uintptr_t)src | (uintptr_t)dst | (uintptr_t)bytes) & 15) == 0;
  if (wide) {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
    for (int64_t w = first; w < bytes / 16; w += step) d4[w] = s4[w];
  } else {
    const int32_t* s1 = reinterpret_cast<const int32_t*>(src);
    int32_t* d1 = reinterpret_cast<int32_t*>(dst);
    for (int64_t w = first; w < bytes / 4; w += step) d1[w] = s1[w];
  }
}

}  // namespace maxsim
