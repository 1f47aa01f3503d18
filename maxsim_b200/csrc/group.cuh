// Grouping a packed pair list by document.
//
// The packed operators take an arbitrary list of (query, document) pairs
// (maxsim_cuda/maxsim.cu:70-126 of the reference launches one CTA per list
// entry, in list order).  When several pairs name the same document, working
// through the list in document order makes the repeats hit in L2 instead of
// streaming the document from HBM once per pair.  These kernels build that
// order with a counting sort on the document id:
//   1. group_count_kernel    bins[id] += 1                (bins zeroed before)
//   2. group_scan_kernel     bins <- exclusive prefix sum (one CTA)
//   3. group_scatter_kernel  order[bins[id]++] = pair
// `bins` (n_documents ints) is scratch; `order` (n_pairs ints) is read by
// the operator kernels.  The order of pairs inside a group is whatever the
// atomics produce; results do not depend on it, because every pair writes
// only its own output slot (gradients are sums either way).
#pragma once

#include "common.cuh"

namespace maxsim {

constexpr int kGroupThreads = 256;
constexpr int kGroupScanThreads = 1024;

__device__ __forceinline__ int32_t group_bin(int32_t id, int32_t n_bins) {
  return id < 0 ? 0 : (id >= n_bins ? n_bins - 1 : id);  // validated ids are in range
}

__global__ void __launch_bounds__(kGroupThreads)
group_count_kernel(const int32_t* __restrict__ ids, int64_t n, int32_t n_bins,
                   int32_t* __restrict__ bins) {
  for (int64_t i = (int64_t)blockIdx.x * kGroupThreads + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * kGroupThreads)
    atomicAdd(bins + group_bin(__ldg(ids + i), n_bins), 1);
}

// In-place exclusive prefix sum of bins[0 .. n_bins): afterwards bins[b] is the
// number of pairs whose bin is below b.  One CTA; every thread owns a
// contiguous slice, which it alone reads and writes.
__global__ void __launch_bounds__(kGroupScanThreads)
group_scan_kernel(int32_t* __restrict__ bins, int32_t n_bins) {
  __shared__ int32_t s_warp[kGroupScanThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (n_bins + kGroupScanThreads - 1) / kGroupScanThreads;
  const int lo = min(per * tid, n_bins), hi = min(lo + per, n_bins);
  int32_t sum = 0;
  for (int i = lo; i < hi; ++i) sum += bins[i];
  int32_t incl = sum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int32_t up = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += up;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int32_t w = s_warp[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int32_t up = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += up;
    }
    s_warp[lane] = w;
  }
  __syncthreads();
  int32_t run = incl - sum + (warp ? s_warp[warp - 1] : 0);
  for (int i = lo; i < hi; ++i) {
    const int32_t c = bins[i];
    bins[i] = run;
    run += c;
  }
}

__global__ void __launch_bounds__(kGroupThreads)
group_scatter_kernel(const int32_t* __restrict__ ids, int64_t n, int32_t n_bins,
                     int32_t* __restrict__ bins, int32_t* __restrict__ order) {
  for (int64_t i = (int64_t)blockIdx.x * kGroupThreads + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * kGroupThreads) {
    const int32_t pos = atomicAdd(bins + group_bin(__ldg(ids + i), n_bins), 1);
    order[pos] = (int32_t)i;
  }
}

}  // namespace maxsim
