// Device-side reduction used by the host-side layout validation: instead of
// copying whole offset / id tensors to the host (the reference's Python layer
// does, torch-ext/maxsim/__init__.py:184-223, 858-877), one small kernel
// reduces them to eight integers that come back in a single transfer.
#pragma once

#include "common.cuh"

namespace maxsim {

constexpr int kStatsThreads = 512;

template <typename I>
__device__ __forceinline__ long long load_index(const void* p, long long i) {
  return (long long)reinterpret_cast<const I*>(p)[i];
}

// out[0] = offsets[0], out[1] = offsets[n-1], out[2] = min segment, out[3] = max segment,
// out[4] = min id, out[5] = max id, out[6] = n_offsets, out[7] = n_ids.
// Absent arrays leave neutral values (min = LLONG_MAX, max = LLONG_MIN).
template <typename I>
__global__ void __launch_bounds__(kStatsThreads)
layout_stats_kernel(const void* offsets, long long n_off, const void* ids, long long n_ids,
                    long long* __restrict__ out) {
  __shared__ long long s_min[kStatsThreads / 32], s_max[kStatsThreads / 32];
  __shared__ long long s_imin[kStatsThreads / 32], s_imax[kStatsThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long mn = 0x7fffffffffffffffLL, mx = -0x7fffffffffffffffLL - 1;
  for (long long i = tid; i + 1 < n_off; i += kStatsThreads) {
    const long long seg = load_index<I>(offsets, i + 1) - load_index<I>(offsets, i);
    mn = seg < mn ? seg : mn;
    mx = seg > mx ? seg : mx;
  }
  long long imn = 0x7fffffffffffffffLL, imx = -0x7fffffffffffffffLL - 1;
  for (long long i = tid; i < n_ids; i += kStatsThreads) {
    const long long v = load_index<I>(ids, i);
    imn = v < imn ? v : imn;
    imx = v > imx ? v : imx;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const long long a = __shfl_xor_sync(0xffffffffu, mn, off), b = __shfl_xor_sync(0xffffffffu, mx, off);
    const long long c = __shfl_xor_sync(0xffffffffu, imn, off), d = __shfl_xor_sync(0xffffffffu, imx, off);
    mn = a < mn ? a : mn; mx = b > mx ? b : mx;
    imn = c < imn ? c : imn; imx = d > imx ? d : imx;
  }
  if (lane == 0) { s_min[warp] = mn; s_max[warp] = mx; s_imin[warp] = imn; s_imax[warp] = imx; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kStatsThreads / 32; ++w) {
      mn = s_min[w] < mn ? s_min[w] : mn; mx = s_max[w] > mx ? s_max[w] : mx;
      imn = s_imin[w] < imn ? s_imin[w] : imn; imx = s_imax[w] > imx ? s_imax[w] : imx;
    }
    out[0] = n_off > 0 ? load_index<I>(offsets, 0) : 0;
    out[1] = n_off > 0 ? load_index<I>(offsets, n_off - 1) : 0;
    out[2] = mn; out[3] = mx; out[4] = imn; out[5] = imx;
    out[6] = n_off; out[7] = n_ids;
  }
}

}  // namespace maxsim
