// The steps either side of the operators.
//
// Packing: an encoder emits padded token rows [N, L_max, row]; the
// contrastive and packed operators take the valid rows back to back with
// int32 offsets (README.md:185-192 of the reference packs with a Python loop
// of slices and torch.cat; torch-ext/maxsim/__init__.py:516-620 with a boolean
// mask gather).  Here the offsets come from one scan kernel and the rows from
// one copy kernel: segment n's valid rows are contiguous on both sides, so the
// gather is N contiguous copies of lengths[n] * row_bytes bytes.  The reverse
// copy (packed -> padded, padding zero-filled) is the gradient of the first
// and also turns packed gradients back into the encoder's layout.
//
// Ranking: README.md:270-274 of the reference sorts the [B, K] score matrix
// with argsort(descending); topk_rows_kernel sorts one row per CTA in shared
// memory and writes the best k (k = K gives the full ranking).
#pragma once

#include "common.cuh"

namespace maxsim {

constexpr int kScanThreads = 1024;
constexpr int kCopyThreads = 256;

// offsets[0] = 0, offsets[n+1] = offsets[n] + clamp(lengths[n], 0, L_max); the
// 64-bit total goes to *total (it can exceed what int32 offsets hold; the host
// checks it).  One CTA: each thread owns a contiguous slice, slices are
// combined by a warp/CTA scan.
__global__ void __launch_bounds__(kScanThreads)
offsets_from_lengths_kernel(const int32_t* __restrict__ lengths, long long n, int L_max,
                            int32_t* __restrict__ offsets, long long* __restrict__ total) {
  __shared__ long long s_warp[kScanThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long per = (n + kScanThreads - 1) / kScanThreads;
  const long long lo = per * tid < n ? per * tid : n;
  const long long hi = lo + per < n ? lo + per : n;
  long long sum = 0;
  for (long long i = lo; i < hi; ++i) {
    const int v = lengths[i];
    sum += v < 0 ? 0 : (v > L_max ? L_max : v);
  }
  long long incl = sum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const long long up = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += up;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    long long w = s_warp[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const long long up = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += up;
    }
    s_warp[lane] = w;
  }
  __syncthreads();
  long long run = incl - sum + (warp ? s_warp[warp - 1] : 0);
  if (tid == 0) offsets[0] = 0;
  for (long long i = lo; i < hi; ++i) {
    const int v = lengths[i];
    run += v < 0 ? 0 : (v > L_max ? L_max : v);
    offsets[i + 1] = (int32_t)run;
  }
  if (tid == kScanThreads - 1 && total) *total = s_warp[kScanThreads / 32 - 1];
}

// Segment copies between the padded and the packed layout.  V is the access
// width (16, 4 or 1 bytes; the host picks the widest the addresses allow).
// grid.x walks segments, grid.y splits a segment's bytes so that long segments
// and small N both fill the device.  TO_PACKED: packed[off[n] ...] = padded[n, :len];
// otherwise padded[n, :len] = packed[off[n] ...] and padded[n, len:] = 0.
// Rows at or beyond packed_rows are never touched (a caller-supplied row count
// smaller than the offsets' end cannot overrun the packed buffer).
template <typename V, bool TO_PACKED>
__global__ void __launch_bounds__(kCopyThreads)
segment_copy_kernel(const void* __restrict__ src, void* __restrict__ dst,
                    const int32_t* __restrict__ offsets, long long n_seg, int L_max,
                    long long row_bytes, long long packed_rows) {
  const long long slab = (long long)L_max * row_bytes / (long long)sizeof(V);  // V units per padded segment
  const long long rowv = row_bytes / (long long)sizeof(V);
  for (long long n = blockIdx.x; n < n_seg; n += gridDim.x) {
    long long o0 = offsets[n], o1 = offsets[n + 1];
    o0 = o0 < 0 ? 0 : (o0 > packed_rows ? packed_rows : o0);
    o1 = o1 < o0 ? o0 : (o1 > packed_rows ? packed_rows : o1);
    long long len = o1 - o0;
    if (len > L_max) len = L_max;
    const long long valid = len * rowv;
    const long long start = (long long)blockIdx.y * kCopyThreads + threadIdx.x;
    const long long step = (long long)gridDim.y * kCopyThreads;
    if (TO_PACKED) {
      const V* s = reinterpret_cast<const V*>(src) + n * slab;
      V* d = reinterpret_cast<V*>(dst) + o0 * rowv;
      long long i = start;
      for (; i + 3 * step < valid; i += 4 * step) {
        const V a = s[i], b = s[i + step], c = s[i + 2 * step], e = s[i + 3 * step];
        d[i] = a; d[i + step] = b; d[i + 2 * step] = c; d[i + 3 * step] = e;
      }
      for (; i < valid; i += step) d[i] = s[i];
    } else {
      const V* s = reinterpret_cast<const V*>(src) + o0 * rowv;
      V* d = reinterpret_cast<V*>(dst) + n * slab;
      long long i = start;
      for (; i + 3 * step < valid; i += 4 * step) {
        const V a = s[i], b = s[i + step], c = s[i + 2 * step], e = s[i + 3 * step];
        d[i] = a; d[i + step] = b; d[i + 2 * step] = c; d[i + 3 * step] = e;
      }
      for (; i < valid; i += step) d[i] = s[i];
      V zero;
      memset(&zero, 0, sizeof(V));
      // first padding unit owned by this thread: smallest i >= valid with i = start (mod step)
      long long z = start + ((valid - start + step - 1) / step) * step;
      if (valid <= start) z = start;
      for (; z < slab; z += step) d[z] = zero;
    }
  }
}

// Valid-row copy between two padded tensors of the same shape: segment n's
// first lengths[n] rows go from src to dst, the padding rows are not touched.
// Made for sources in pinned host memory (the kernel reads it over PCIe through
// the device mapping of the allocation): a padded rerank batch is about one
// third padding, which a plain host-to-device copy would move as well.  Eight
// independent 16-byte loads are in flight per thread before the first store.
template <typename V>
__global__ void __launch_bounds__(kCopyThreads)
valid_rows_copy_kernel(const void* __restrict__ src, void* __restrict__ dst,
                       const int32_t* __restrict__ lengths, long long n_seg, int L_max,
                       long long row_bytes) {
  const long long slab = (long long)L_max * row_bytes / (long long)sizeof(V);
  const long long rowv = row_bytes / (long long)sizeof(V);
  const long long start = (long long)blockIdx.y * kCopyThreads + threadIdx.x;
  const long long step = (long long)gridDim.y * kCopyThreads;
  for (long long n = blockIdx.x; n < n_seg; n += gridDim.x) {
    int len = __ldg(lengths + n);
    len = len < 0 ? 0 : (len > L_max ? L_max : len);
    const long long valid = (long long)len * rowv;
    const V* s = reinterpret_cast<const V*>(src) + n * slab;
    V* d = reinterpret_cast<V*>(dst) + n * slab;
    long long i = start;
    for (; i + 7 * step < valid; i += 8 * step) {
      V v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = s[i + u * step];
#pragma unroll
      for (int u = 0; u < 8; ++u) d[i + u * step] = v[u];
    }
    for (; i < valid; i += step) d[i] = s[i];
  }
}

// ---------------------------------------------------------------------------
// Ranking.  One CTA sorts one score row in shared memory (bitonic network over
// 64-bit keys) and writes the best k entries, best first.  Key = order-
// preserving image of the float in the high word, ~index in the low word, so
// a descending sort puts the larger score first and, among equal scores, the
// LOWER index first.  NaN ranks above +inf (torch.sort's convention); -0 and
// +0 are equal.
// ---------------------------------------------------------------------------
constexpr int kTopkThreads = 512;
constexpr int kTopkMaxCols = 16384;  // 128 KB of keys

__device__ __forceinline__ unsigned long long rank_key(float v, unsigned idx) {
  unsigned hi;
  if (v != v) {
    hi = 0xffffffffu;
  } else {
    const unsigned b = __float_as_uint(v + 0.0f);  // -0 -> +0
    hi = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
  return ((unsigned long long)hi << 32) | (unsigned long long)(~idx);
}

__global__ void __launch_bounds__(kTopkThreads)
topk_rows_kernel(const float* __restrict__ scores, long long cols, int n_pow2, int k,
                 float* __restrict__ values, long long* __restrict__ indices) {
  extern __shared__ unsigned long long s_keys[];
  const float* row = scores + (long long)blockIdx.x * cols;
  for (int i = threadIdx.x; i < n_pow2; i += kTopkThreads)
    s_keys[i] = i < cols ? rank_key(row[i], (unsigned)i) : 0ull;  // 0 sorts last: below every real key
  __syncthreads();
  for (int size = 2; size <= n_pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (n_pow2 >> 1); t += kTopkThreads) {
        const int i = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
        const int j = i | stride;
        const bool desc = (i & size) == 0;
        const unsigned long long a = s_keys[i], b = s_keys[j];
        if ((a < b) == desc) { s_keys[i] = b; s_keys[j] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < k; i += kTopkThreads) {
    const unsigned idx = ~(unsigned)(s_keys[i] & 0xffffffffull);
    values[(long long)blockIdx.x * k + i] = row[idx];
    indices[(long long)blockIdx.x * k + i] = (long long)idx;
  }
}

}  // namespace maxsim
