// Portable forward kernel: any dtype (fp32 / fp16 / bf16), any dim, any query
// length.  One CTA per (query, document) pair; every thread owns document
// tokens tid, tid+128, ... and forms their dot products with up to 32 query
// rows held in shared memory, in ascending-k fp32 FMA order (the order of the
// reference's scalar path, maxsim_cuda/maxsim.cu:59-66).  This is the fp32
// path and the fallback for shapes the tensor-core kernels do not take.
#pragma once

#include "common.cuh"

namespace maxsim {

constexpr int kSimtThreads = 128;
constexpr int kSimtRows = 32;  // query rows per pass

template <typename T>
__device__ __forceinline__ void load_chunk8(const T* __restrict__ row, int k0, int dim,
                                            bool vec_ok, float (&out)[8]) {
  if (vec_ok && k0 + 8 <= dim) {
    if constexpr (sizeof(T) == 4) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(row + k0));
      const float4 b = __ldg(reinterpret_cast<const float4*>(row + k0 + 4));
      out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
      out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    } else {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + k0));
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = to_f32(e[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = (k0 + i < dim) ? to_f32(row[k0 + i]) : 0.0f;
  }
}

// Order used everywhere a (value, index) pair is merged: larger value wins,
// equal values keep the lower index (first document token wins a tie).
__device__ __forceinline__ void merge_best(float& v, int& ix, float ov, int oi) {
  if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
}

template <typename T, int LAYOUT, bool ARGMAX>
__global__ void __launch_bounds__(kSimtThreads)
fwd_simt_kernel(PairTable t, float* __restrict__ scores, int32_t* __restrict__ argmax,
                int vec_ok) {
  extern __shared__ __align__(16) float simt_smem[];
  const int dim = t.dim;
  const int dimp = (dim + 7) & ~7;
  float* sq = simt_smem;                                    // [32][dimp]
  float* red_v = sq + kSimtRows * dimp;                     // [4][32]
  int* red_i = reinterpret_cast<int*>(red_v + 4 * kSimtRows);  // [4][32]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int64_t pos = blockIdx.x; pos < t.n_pairs; pos += gridDim.x) {
    const int64_t p = pair_at<LAYOUT>(t, pos);
    const PairGeom g = pair_geom<LAYOUT>(t, p);
    const T* Q = reinterpret_cast<const T*>(t.queries) + g.q_row0 * dim;
    const T* D = reinterpret_cast<const T*>(t.documents) + g.d_row0 * dim;
    float score = 0.0f;  // meaningful in warp 0

    for (int q0 = 0; q0 < g.Lq; q0 += kSimtRows) {
      const int rows = min(kSimtRows, g.Lq - q0);
      __syncthreads();
      for (int e = tid; e < kSimtRows * dimp; e += kSimtThreads) {
        const int r = e / dimp, k = e - r * dimp;
        sq[e] = (r < rows && k < dim) ? to_f32(Q[(int64_t)(q0 + r) * dim + k]) : 0.0f;
      }
      __syncthreads();

      float run[kSimtRows];
      int idx[kSimtRows];
#pragma unroll
      for (int i = 0; i < kSimtRows; ++i) { run[i] = neg_inf(); idx[i] = 0; }

      for (int j = tid; j < g.Ld; j += kSimtThreads) {
        const T* drow = D + (int64_t)j * dim;
        float acc[kSimtRows];
#pragma unroll
        for (int i = 0; i < kSimtRows; ++i) acc[i] = 0.0f;
        for (int k0 = 0; k0 < dimp; k0 += 8) {
          float dv[8];
          load_chunk8<T>(drow, k0, dim, vec_ok != 0, dv);
#pragma unroll
          for (int i = 0; i < kSimtRows; ++i) {
            const float4 qa = *reinterpret_cast<const float4*>(sq + i * dimp + k0);
            const float4 qb = *reinterpret_cast<const float4*>(sq + i * dimp + k0 + 4);
            float a = acc[i];
            a = fmaf(qa.x, dv[0], a); a = fmaf(qa.y, dv[1], a);
            a = fmaf(qa.z, dv[2], a); a = fmaf(qa.w, dv[3], a);
            a = fmaf(qb.x, dv[4], a); a = fmaf(qb.y, dv[5], a);
            a = fmaf(qb.z, dv[6], a); a = fmaf(qb.w, dv[7], a);
            acc[i] = a;
          }
        }
#pragma unroll
        for (int i = 0; i < kSimtRows; ++i) {
          if (acc[i] > run[i]) { run[i] = acc[i]; idx[i] = j; }  // NaN never wins
        }
      }

      // Reduce over the 128 threads, one query row at a time.
#pragma unroll
      for (int i = 0; i < kSimtRows; ++i) {
        float v = run[i];
        int ix = idx[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, off);
          const int oi = __shfl_xor_sync(0xffffffffu, ix, off);
          merge_best(v, ix, ov, oi);
        }
        if (lane == 0) { red_v[warp * kSimtRows + i] = v; red_i[warp * kSimtRows + i] = ix; }
      }
      __syncthreads();
      if (warp == 0) {
        float v = red_v[lane];
        int ix = red_i[lane];
#pragma unroll
        for (int w = 1; w < kSimtThreads / 32; ++w)
          merge_best(v, ix, red_v[w * kSimtRows + lane], red_i[w * kSimtRows + lane]);
        float contrib = (lane < rows) ? v : 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, off);
        score += contrib;
        if (ARGMAX && lane < rows) argmax[p * t.q_slots + q0 + lane] = ix;
      }
    }
    if (warp == 0) {
      if (lane == 0) scores[p] = score;
      if (ARGMAX) {
        for (int s = g.Lq + lane; s < t.q_slots; s += 32) argmax[p * t.q_slots + s] = 0;
      }
    }
  }
}

}  // namespace maxsim
