// extern "C" entry points of libmaxsim_b200.so and the host-side dispatch.
// No torch headers: the boundary is plain pointers, sizes and a stream.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <string>
#include <type_traits>

#include "../../include/maxsim_b200.h"
#include "bwd.cuh"
#include "common.cuh"
#include "fwd_mma.cuh"
#include "fwd_simt.cuh"
#include "fwd_tc05_any.cuh"
#include "fwd_tc05_doc.cuh"
#include "group.cuh"
#include "layout_stats.cuh"
#include "loss.cuh"
#include "pack.cuh"

namespace maxsim {

namespace {

thread_local std::string t_last_error;
std::atomic<int64_t> g_launches{0};
std::atomic<int> g_forward_path{0};

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_last_error = buf;
  return code;
}

#define MAXSIM_CUDA(expr)                                                         \
  do {                                                                            \
    cudaError_t e_ = (expr);                                                      \
    if (e_ != cudaSuccess)                                                        \
      return fail(MAXSIM_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

int launch_check(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(MAXSIM_ECUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  return MAXSIM_OK;
}

// Per-device caches below are written with the same value by every thread that
// races on them, through atomics, so concurrent first calls are harmless.
constexpr int kMaxDevices = 64;

int sm_count() {
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Opt a kernel in to `smem` bytes of dynamic shared memory, once per device.
template <typename Kernel>
int ensure_smem(Kernel kern, size_t smem, std::atomic<unsigned char>* done) {
  int dev = 0;
  MAXSIM_CUDA(cudaGetDevice(&dev));
  const bool track = dev >= 0 && dev < kMaxDevices;
  if (track && done[dev].load(std::memory_order_acquire)) return MAXSIM_OK;
  MAXSIM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (track) done[dev].store(1, std::memory_order_release);
  return MAXSIM_OK;
}

// Mean document length up to which contrastive argmax launches tile every
// document on its own.  Measured on 1024 x 1024 pairs, bf16, per-document tiles
// against boundary-agnostic ones: 32-256 tokens 1.43 / 1.77 ms, 64-512 tokens
// (mean 288) 2.43 / 2.56 ms, 300-1000 tokens 4.9-5.4 / 4.9-5.0 ms.
constexpr int64_t kPerDocMaxMean = 320;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool valid_dtype(int dtype) { return dtype == MAXSIM_F32 || dtype == MAXSIM_F16 || dtype == MAXSIM_BF16; }

// ---------------------------------------------------------------------------
// Forward dispatch
// ---------------------------------------------------------------------------
template <typename T, int LAYOUT, bool ARGMAX>
int launch_simt(const PairTable& t, float* scores, int32_t* argmax, cudaStream_t st) {
  const int dimp = (t.dim + 7) & ~7;
  const size_t smem = ((size_t)kSimtRows * dimp + 8 * kSimtRows) * sizeof(float);
  if (smem > 200 * 1024) return fail(MAXSIM_EUNSUPPORTED, "dim=%d too large for the SIMT kernel", t.dim);
  auto kern = fwd_simt_kernel<T, LAYOUT, ARGMAX>;
  if (smem > 48 * 1024)
    MAXSIM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int elems16 = 16 / (int)sizeof(T);
  const int vec_ok = (t.dim % elems16 == 0) && aligned16(t.documents);
  const int64_t grid = t.n_pairs < (1 << 22) ? t.n_pairs : (1 << 22);
  kern<<<(unsigned)grid, kSimtThreads, smem, st>>>(t, scores, argmax, vec_ok);
  return launch_check("fwd_simt_kernel");
}

template <typename T, int DIM, int LAYOUT, bool ARGMAX>
int launch_mma_dim(const PairTable& t, float* scores, int32_t* argmax, cudaStream_t st) {
  auto kern = fwd_mma_kernel<T, DIM, LAYOUT, ARGMAX>;
  constexpr size_t smem = mma_smem_bytes<DIM>();
  static std::atomic<unsigned char> configured[kMaxDevices];
  if (int rc = ensure_smem(kern, smem, configured)) return rc;
  const int sms = sm_count();
  const int64_t warps_full = (int64_t)sms * kMmaWarps;
  int ppc = (int)(t.n_pairs / (warps_full * 4));
  if (ppc < 1) ppc = 1;
  if (ppc > 8) ppc = 8;
  if (t.order && ppc > 2) ppc = 2;  // same-document pairs to different warps at about the same time
  const int64_t n_chunks = (t.n_pairs + ppc - 1) / ppc;
  int64_t grid = (n_chunks + kMmaWarps - 1) / kMmaWarps;
  if (grid > sms) grid = sms;
  if (grid < 1) grid = 1;
  kern<<<(unsigned)grid, kMmaThreads, smem, st>>>(t, scores, argmax, ppc);
  return launch_check("fwd_mma_kernel");
}

template <typename T, int LAYOUT, bool ARGMAX>
int launch_mma(const PairTable& t, float* scores, int32_t* argmax, cudaStream_t st) {
  switch (t.dim) {
    case 32: return launch_mma_dim<T, 32, LAYOUT, ARGMAX>(t, scores, argmax, st);
    case 64: return launch_mma_dim<T, 64, LAYOUT, ARGMAX>(t, scores, argmax, st);
    case 96: return launch_mma_dim<T, 96, LAYOUT, ARGMAX>(t, scores, argmax, st);
    case 128: return launch_mma_dim<T, 128, LAYOUT, ARGMAX>(t, scores, argmax, st);
    default: return fail(MAXSIM_EUNSUPPORTED, "warp-MMA kernel does not take dim=%d", t.dim);
  }
}

bool mma_eligible(const PairTable& t, int dtype) {
  if (dtype == MAXSIM_F32) return false;
  if (!(t.dim == 32 || t.dim == 64 || t.dim == 96 || t.dim == 128)) return false;
  if (!aligned16(t.queries) || !aligned16(t.documents)) return false;
  if (t.n_pairs >= (1ll << 31)) return false;
  if (t.q_slots > 32767) return false;
  // the streaming kernel indexes token rows with 32 bits
  if (t.Ld_max > 0 && t.n_pairs * (int64_t)t.Ld_max >= (1ll << 31)) return false;
  if ((t.n_pairs / t.C + 1) * (int64_t)t.q_slots >= (1ll << 31)) return false;
  return true;
}

template <int LAYOUT, bool ARGMAX>
int run_forward(const PairTable& t, float* scores, int32_t* argmax, int dtype, void* stream) {
  if (!valid_dtype(dtype)) return fail(MAXSIM_EINVAL, "unknown dtype code %d", dtype);
  if (t.n_pairs < 0 || t.dim <= 0 || t.q_slots <= 0)
    return fail(MAXSIM_EINVAL, "sizes must be positive (pairs=%lld dim=%d q_slots=%d)",
                (long long)t.n_pairs, t.dim, t.q_slots);
  if (t.n_pairs == 0) return MAXSIM_OK;
  if (!t.queries || !t.documents || !scores || (ARGMAX && !argmax))
    return fail(MAXSIM_EINVAL, "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int path = g_forward_path.load(std::memory_order_relaxed);

  if (LAYOUT == kContrastive && path != 1 && path != 2 &&
      (tc05_eligible(t, dtype) || tc05g_eligible(t, dtype))) {
    // Tiles that start at document starts pay one short tile per document and
    // spare the epilogue the cuts at document boundaries inside a tile; they are
    // taken for argmax launches whose documents average at most kPerDocMaxMean
    // tokens.  Path 8 forces them, path 9 forces the boundary-agnostic tiles.
    const bool per_document =
        ARGMAX && (path == 8 || (path != 9 && t.block_rows <= kPerDocMaxMean * (int64_t)t.C));
    int rc;
    // the persistent kernels take one CTA per SM; a launch that runs beside a collective
    // leaves t.reserve_sms of them to the collective's kernels
    int sms = sm_count() - t.reserve_sms;
    if (sms < 8) sms = 8;
    if (tc05_eligible(t, dtype))  // Lq = 32, dim = 128
      rc = per_document ? launch_tc05_doc<ARGMAX>(t, scores, argmax, dtype, sms, st)
                        : launch_tc05<ARGMAX>(t, scores, argmax, dtype, sms, st);
    else
      rc = launch_tc05g<ARGMAX>(t, scores, argmax, dtype, sms, st, per_document);
    if (rc == 0) return launch_check("fwd_tc05_kernel");
    if (rc < 0) return fail(MAXSIM_ECUDA, "could not configure the tcgen05 kernel");
    // rc == 1: tensor maps could not be encoded; use the streaming kernel
  }
  if ((path == 3 || path == 8 || path == 9) && LAYOUT == kContrastive)
    return fail(MAXSIM_EUNSUPPORTED, "tcgen05 kernel forced but shape not eligible");
  if (LAYOUT == kContrastive && (t.out_ld != t.C || t.out_col0 != 0))
    return fail(MAXSIM_EUNSUPPORTED, "a column block of a wider score matrix needs the tcgen05 kernel "
                                     "(float16 / bfloat16, Lq <= 64, dim %% 16 == 0, dim <= 128)");

  if (path != 1 && mma_eligible(t, dtype)) {
    if (dtype == MAXSIM_F16) return launch_mma<__half, LAYOUT, ARGMAX>(t, scores, argmax, st);
    return launch_mma<__nv_bfloat16, LAYOUT, ARGMAX>(t, scores, argmax, st);
  }
  switch (dtype) {
    case MAXSIM_F32: return launch_simt<float, LAYOUT, ARGMAX>(t, scores, argmax, st);
    case MAXSIM_F16: return launch_simt<__half, LAYOUT, ARGMAX>(t, scores, argmax, st);
    default: return launch_simt<__nv_bfloat16, LAYOUT, ARGMAX>(t, scores, argmax, st);
  }
}

// ---------------------------------------------------------------------------
// Backward dispatch
// ---------------------------------------------------------------------------

// grad_queries of 16-bit inputs (dim % 8 == 0, dim <= 128): one owner warp per query row.
template <typename T, int LAYOUT>
int launch_dq16(const PairTable& t, const float* dscore, const int32_t* argmax, void* dq,
                int64_t q_rows, int native, cudaStream_t st) {
  // One warp per row fills the GPU from about three waves of warps up (36 resident per SM);
  // with fewer rows and enough candidates, 2 or 4 warps share a row.
  const int64_t full = (int64_t)sm_count() * 36 * 3;
  const int split = (q_rows >= full || t.C < 256) ? 1 : (2 * q_rows >= full || t.C < 512) ? 2 : 4;
  const int64_t grid = (q_rows * split + kBwdWarps - 1) / kBwdWarps;
  const unsigned threads = kBwdWarps * 32;
  if (split == 1)
    bwd_dq_gather16_kernel<T, LAYOUT, 1><<<(unsigned)grid, threads, 0, st>>>(t, dscore, argmax, dq, q_rows, native);
  else if (split == 2)
    bwd_dq_gather16_kernel<T, LAYOUT, 2><<<(unsigned)grid, threads, 0, st>>>(t, dscore, argmax, dq, q_rows, native);
  else
    bwd_dq_gather16_kernel<T, LAYOUT, 4><<<(unsigned)grid, threads, 0, st>>>(t, dscore, argmax, dq, q_rows, native);
  return launch_check("bwd_dq_gather16_kernel");
}

template <typename T, int LAYOUT>
int run_backward_t(const PairTable& t, const float* dscore, const int32_t* argmax, float* dq,
                   float* dd, int64_t q_rows, int64_t d_rows, int64_t Nq, cudaStream_t st,
                   int64_t n_queries, int64_t n_documents) {
  const int dim = t.dim;
  const int vec_ok = (dim % 4 == 0) && aligned16(t.queries) && aligned16(t.documents) &&
                     aligned16(dq) && aligned16(dd);
  const unsigned threads = kBwdWarps * 32;
  if constexpr (LAYOUT == kPacked) {
    if (t.order_q && vec_ok && dim % 8 == 0 && t.n_pairs > 0 &&
        n_queries * (int64_t)t.q_slots < (1ll << 33)) {
      // grouped lists: owner warps, every output row written once
      if (n_queries > 0) {
        const int64_t rows = n_queries * (int64_t)t.q_slots;
        bwd_dq_packed_kernel<T><<<(unsigned)((rows + kBwdWarps - 1) / kBwdWarps), threads, 0, st>>>(
            t, dscore, argmax, dq, n_queries, 0);
        if (int rc = launch_check("bwd_dq_packed_kernel")) return rc;
      }
      if (n_documents > 0) {
        bwd_dd_packed_kernel<T><<<(unsigned)((n_documents + kBwdWarps - 1) / kBwdWarps), threads, 0, st>>>(
            t, dscore, argmax, dd, n_documents);
        if (int rc = launch_check("bwd_dd_packed_kernel")) return rc;
      }
      return MAXSIM_OK;
    }
    MAXSIM_CUDA(cudaMemsetAsync(dq, 0, (size_t)q_rows * dim * sizeof(float), st));
    MAXSIM_CUDA(cudaMemsetAsync(dd, 0, (size_t)d_rows * dim * sizeof(float), st));
    if (t.n_pairs == 0) return MAXSIM_OK;
    const int64_t grid = (t.n_pairs + kBwdWarps - 1) / kBwdWarps;
    bwd_route_atomic_kernel<T, LAYOUT, true, true><<<(unsigned)grid, threads, 0, st>>>(
        t, dscore, argmax, dq, dd, vec_ok);
    return launch_check("bwd_route_atomic_kernel");
  } else {
    if (t.n_pairs == 0) {
      if (dq) MAXSIM_CUDA(cudaMemsetAsync(dq, 0, (size_t)q_rows * dim * sizeof(float), st));
      if (dd) MAXSIM_CUDA(cudaMemsetAsync(dd, 0, (size_t)d_rows * dim * sizeof(float), st));
      return MAXSIM_OK;
    }
    if (dq) {
      bool fast = false;
      if constexpr (sizeof(T) == 2) {
        fast = vec_ok && dim <= 128 && dim % 8 == 0 && d_rows < (1ll << 31);
        if (fast)
          if (int rc = launch_dq16<T, LAYOUT>(t, dscore, argmax, dq, q_rows, 0, st)) return rc;
      }
      if (!fast) {
        const int64_t grid = (q_rows + kBwdWarps - 1) / kBwdWarps;
        bwd_dq_gather_kernel<T, LAYOUT><<<(unsigned)grid, threads, 0, st>>>(t, dscore, argmax, dq,
                                                                             q_rows, vec_ok);
        if (int rc = launch_check("bwd_dq_gather_kernel")) return rc;
      }
    }
    if constexpr (LAYOUT == kPadded) {
      const int64_t grid = (t.n_pairs + kBwdWarps - 1) / kBwdWarps;
      bwd_dd_padded_kernel<T><<<(unsigned)grid, threads, 0, st>>>(t, dscore, argmax, dd, vec_ok);
      return launch_check("bwd_dd_padded_kernel");
    } else {
      if (!dd) return MAXSIM_OK;
      const int64_t Nb = t.C;
      if (vec_ok && dim % 8 == 0 && t.q_slots <= kInvEntries && Nq < (1ll << 31) &&
          Nb < (1ll << 31) && Nq * (int64_t)t.q_slots < (1ll << 31)) {
        auto kern = bwd_dd_invert_kernel<T>;
        constexpr size_t smem = inv_smem_bytes();
        static std::atomic<unsigned char> configured[kMaxDevices];
        if (int rc = ensure_smem(kern, smem, configured)) return rc;
        int gy, split;
        inv_grid_shape(Nb, d_rows / Nb, sm_count(), &gy, &split);
        dim3 grid((unsigned)Nb, (unsigned)gy);
        kern<<<grid, kInvThreads, smem, st>>>(t, dscore, argmax, dd, (int)Nq, 0, split, 0);
        return launch_check("bwd_dd_invert_kernel");
      }
      MAXSIM_CUDA(cudaMemsetAsync(dd, 0, (size_t)d_rows * dim * sizeof(float), st));
      const int64_t grid = (t.n_pairs + kBwdWarps - 1) / kBwdWarps;
      bwd_route_atomic_kernel<T, LAYOUT, false, true><<<(unsigned)grid, threads, 0, st>>>(
          t, dscore, argmax, dq, dd, vec_ok);
      return launch_check("bwd_route_atomic_kernel");
    }
  }
}

template <int LAYOUT>
int run_backward(const PairTable& t, const float* dscore, const int32_t* argmax, float* dq,
                 float* dd, int64_t q_rows, int64_t d_rows, int64_t Nq, int dtype, void* stream,
                 int64_t n_queries = 0, int64_t n_documents = 0) {
  if (!valid_dtype(dtype)) return fail(MAXSIM_EINVAL, "unknown dtype code %d", dtype);
  if (t.dim <= 0 || t.q_slots <= 0 || t.n_pairs < 0 || q_rows < 0 || d_rows < 0)
    return fail(MAXSIM_EINVAL, "sizes must be positive");
  // The contrastive operator may be asked for one gradient only (the other
  // pointer NULL): the sharded driver computes grad_queries where the queries
  // live and grad_documents where the documents live.
  if (LAYOUT != kContrastive && ((q_rows && !dq) || (d_rows && !dd)))
    return fail(MAXSIM_EINVAL, "null gradient pointer");
  if (LAYOUT == kContrastive && !dq && !dd) return MAXSIM_OK;
  if (t.n_pairs && (!dscore || !argmax || !t.queries || !t.documents))
    return fail(MAXSIM_EINVAL, "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MAXSIM_F32: return run_backward_t<float, LAYOUT>(t, dscore, argmax, dq, dd, q_rows, d_rows, Nq, st,
                                                  n_queries, n_documents);
    case MAXSIM_F16: return run_backward_t<__half, LAYOUT>(t, dscore, argmax, dq, dd, q_rows, d_rows, Nq, st,
                                                  n_queries, n_documents);
    default: return run_backward_t<__nv_bfloat16, LAYOUT>(t, dscore, argmax, dq, dd, q_rows, d_rows, Nq, st,
                                                  n_queries, n_documents);
  }
}

// Gradients written once, in the inputs' 16-bit element type.  Only for the
// shapes whose kernels store every gradient row exactly once; anything else is
// MAXSIM_EUNSUPPORTED and the caller uses the fp32 operator.
template <typename T, int LAYOUT>
int run_backward_native_t(const PairTable& t, const float* dscore, const int32_t* argmax, void* dq,
                          void* dd, int64_t q_rows, int64_t d_rows, int64_t Nq, cudaStream_t st) {
  static_assert(LAYOUT == kPadded || LAYOUT == kContrastive, "padded and contrastive only");
  const int dim = t.dim;
  const bool ok = dim % 8 == 0 && dim <= 128 && aligned16(t.queries) && aligned16(t.documents) &&
                  aligned16(dq) && aligned16(dd) && d_rows < (1ll << 31) && t.n_pairs > 0 &&
                  (dd || LAYOUT == kContrastive);
  if (!ok) return fail(MAXSIM_EUNSUPPORTED, "native-type gradients need dim %% 8 == 0, dim <= 128 and aligned tensors");
  const unsigned threads = kBwdWarps * 32;
  if constexpr (LAYOUT == kPadded) {
    if (t.q_slots > 32 || t.Ld_max > 1024)
      return fail(MAXSIM_EUNSUPPORTED, "native-type gradients need Lq_max <= 32 and Ld_max <= 1024");
  } else {
    const int64_t Nb = t.C;
    if (dd && ((int64_t)Nq * t.q_slots > kInvEntries || Nq > kInvMaxQ || Nb >= (1ll << 31)))
      return fail(MAXSIM_EUNSUPPORTED, "native-type gradients need Nq * Lq <= %d", kInvEntries);
  }
  if (int rc = launch_dq16<T, LAYOUT>(t, dscore, argmax, dq, q_rows, 1, st)) return rc;
  if constexpr (LAYOUT == kPadded) {
    const int64_t grid = (t.n_pairs + kBwdWarps - 1) / kBwdWarps;
    bwd_dd_padded_native_kernel<T><<<(unsigned)grid, threads, 0, st>>>(t, dscore, argmax,
                                                                       reinterpret_cast<T*>(dd));
    return launch_check("bwd_dd_padded_native_kernel");
  } else {
    if (!dd) return MAXSIM_OK;  // grad_queries only
    const int64_t Nb = t.C;
    auto kern = bwd_dd_invert_kernel<T>;
    constexpr size_t smem = inv_smem_bytes();
    static std::atomic<unsigned char> configured[kMaxDevices];
    if (int rc = ensure_smem(kern, smem, configured)) return rc;
    int gy, split;
    inv_grid_shape(Nb, d_rows / Nb, sm_count(), &gy, &split);
    dim3 grid((unsigned)Nb, (unsigned)gy);
    kern<<<grid, kInvThreads, smem, st>>>(t, dscore, argmax, dd, (int)Nq, 1, split, 0);
    return launch_check("bwd_dd_invert_kernel");
  }
}

template <int LAYOUT>
int run_backward_native(const PairTable& t, const float* dscore, const int32_t* argmax, void* dq,
                        void* dd, int64_t q_rows, int64_t d_rows, int64_t Nq, int dtype,
                        void* stream) {
  if (t.dim <= 0 || t.q_slots <= 0 || t.n_pairs < 0 || q_rows < 0 || d_rows < 0)
    return fail(MAXSIM_EINVAL, "sizes must be positive");
  // the contrastive operator may be asked for grad_queries alone (grad_documents NULL)
  if (!dq || (!dd && LAYOUT != kContrastive) || !dscore || !argmax)
    return fail(MAXSIM_EUNSUPPORTED, "empty problem");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MAXSIM_F16: return run_backward_native_t<__half, LAYOUT>(t, dscore, argmax, dq, dd, q_rows, d_rows, Nq, st);
    case MAXSIM_BF16: return run_backward_native_t<__nv_bfloat16, LAYOUT>(t, dscore, argmax, dq, dd, q_rows, d_rows, Nq, st);
    default: return fail(MAXSIM_EUNSUPPORTED, "native-type gradients are for float16 / bfloat16 inputs");
  }
}

template <typename T>
int launch_dd_from_records(const PairTable& t, const int32_t* records, void* dd, int64_t Nq,
                           int native, cudaStream_t st) {
  auto kern = bwd_dd_invert_kernel<T>;
  constexpr size_t smem = inv_smem_bytes();
  static std::atomic<unsigned char> configured[kMaxDevices];
  if (int rc = ensure_smem(kern, smem, configured)) return rc;
  int gy, split;
  inv_grid_shape(t.C, t.d_rows / t.C, sm_count(), &gy, &split);
  dim3 grid((unsigned)t.C, (unsigned)gy);
  kern<<<grid, kInvThreads, smem, st>>>(t, nullptr, records, dd, (int)Nq, native, split,
                                        t.q_slots + 1);
  return launch_check("bwd_dd_invert_kernel");
}

PairTable packed_table(const void* q, const int32_t* qoff, const void* d, const int32_t* doff,
                       const int32_t* pq, const int32_t* pd, int64_t n_pairs, int64_t dim,
                       int64_t max_q_len, int64_t q_rows, int64_t d_rows,
                       const int32_t* order = nullptr) {
  PairTable t{};
  t.queries = q; t.documents = d;
  t.ia = qoff; t.ib = doff; t.ic = pq; t.id = pd; t.order = order;
  t.n_pairs = n_pairs; t.dim = (int32_t)dim; t.q_slots = (int32_t)max_q_len;
  t.q_rows = q_rows; t.d_rows = d_rows;
  t.Ld_max = 0; t.C = 1;
  return t;
}

PairTable padded_table(const void* q, const int32_t* qlen, const void* d, const int32_t* dlen,
                       int64_t B, int64_t C, int64_t Lq_max, int64_t Ld_max, int64_t dim) {
  PairTable t{};
  t.queries = q; t.documents = d;
  t.ia = qlen; t.ib = dlen; t.ic = nullptr; t.id = nullptr;
  t.n_pairs = B * C; t.dim = (int32_t)dim; t.q_slots = (int32_t)Lq_max;
  t.q_rows = B * Lq_max; t.d_rows = B * C * Ld_max;
  t.Ld_max = (int32_t)Ld_max; t.C = (int32_t)(C > 0 ? C : 1);
  return t;
}

PairTable contrastive_table(const void* q, const void* d, const int32_t* doff, int64_t Nq,
                            int64_t Lq, int64_t Nb, int64_t dim, int64_t d_rows) {
  PairTable t{};
  t.queries = q; t.documents = d;
  t.ia = nullptr; t.ib = doff; t.ic = nullptr; t.id = nullptr;
  t.n_pairs = Nq * Nb; t.dim = (int32_t)dim; t.q_slots = (int32_t)Lq;
  t.q_rows = Nq * Lq; t.d_rows = d_rows;
  t.Ld_max = 0; t.C = (int32_t)(Nb > 0 ? Nb : 1);
  t.out_ld = t.C; t.out_col0 = 0; t.block_rows = d_rows; t.reserve_sms = 0;
  return t;
}

bool fits_i32(int64_t v) { return v >= 0 && v < (1ll << 31); }

template <bool TO_PACKED>
int run_segment_copy(const void* src, void* dst, const int32_t* offsets, int64_t n_segments,
                     int64_t L_max, int64_t row_bytes, int64_t packed_rows, void* stream) {
  if (n_segments < 0 || L_max < 0 || row_bytes <= 0 || packed_rows < 0 || !fits_i32(L_max))
    return fail(MAXSIM_EINVAL, "sizes must be >= 0 (row_bytes > 0) and L_max must fit int32");
  if (n_segments == 0 || L_max == 0) return MAXSIM_OK;
  if (!src || !dst || !offsets) return fail(MAXSIM_EINVAL, "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  const int64_t slab_bytes = L_max * row_bytes;
  int64_t gy = (slab_bytes + 16 * 4 * kCopyThreads - 1) / (16 * 4 * kCopyThreads);
  gy = gy < 1 ? 1 : (gy > 8 ? 8 : gy);
  int64_t gx = n_segments;
  const int64_t cap = (int64_t)sms * 64;
  if (gx * gy > cap) gx = cap / gy;
  dim3 grid((unsigned)gx, (unsigned)gy);
  const bool a16 = aligned16(src) && aligned16(dst) && row_bytes % 16 == 0;
  const bool a4 = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 3u) == 0 &&
                  row_bytes % 4 == 0;
  if (a16)
    segment_copy_kernel<uint4, TO_PACKED><<<grid, kCopyThreads, 0, st>>>(
        src, dst, offsets, n_segments, (int)L_max, row_bytes, packed_rows);
  else if (a4)
    segment_copy_kernel<uint32_t, TO_PACKED><<<grid, kCopyThreads, 0, st>>>(
        src, dst, offsets, n_segments, (int)L_max, row_bytes, packed_rows);
  else
    segment_copy_kernel<uint8_t, TO_PACKED><<<grid, kCopyThreads, 0, st>>>(
        src, dst, offsets, n_segments, (int)L_max, row_bytes, packed_rows);
  return launch_check("segment_copy_kernel");
}

}  // namespace
}  // namespace maxsim

using namespace maxsim;

extern "C" {

const char* maxsim_b200_version(void) { return "maxsim_b200 0.1 (sm_100a)"; }
const char* maxsim_b200_last_error(void) { return t_last_error.c_str(); }
int64_t maxsim_b200_launch_count(void) { return g_launches.load(); }
void maxsim_b200_set_forward_path(int path) { g_forward_path.store(path); }

int maxsim_b200_device_status(void* stream) {
  int v = 0, zero = 0;
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return MAXSIM_ECUDA;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return MAXSIM_ECUDA;
  if (v != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  return v;
}

int maxsim_b200_wait_probe(int64_t polls, int* gave_up, void* stream) {
  if (polls < 1 || polls > (1 << 20)) return fail(MAXSIM_EINVAL, "polls must be in [1, 2^20]");
  tc05g::wait_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>((uint32_t)polls, gave_up);
  return launch_check("wait_probe_kernel");
}

int maxsim_b200_layout_stats(const void* offsets, int64_t n_offsets, const void* ids, int64_t n_ids,
                             int index_bytes, int64_t* out8, void* stream) {
  if (!out8) return fail(MAXSIM_EINVAL, "null output pointer");
  if ((n_offsets > 0 && !offsets) || (n_ids > 0 && !ids) || n_offsets < 0 || n_ids < 0)
    return fail(MAXSIM_EINVAL, "null index array");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long* out = reinterpret_cast<long long*>(out8);
  if (index_bytes == 4)
    layout_stats_kernel<int32_t><<<1, kStatsThreads, 0, st>>>(offsets, n_offsets, ids, n_ids, out);
  else if (index_bytes == 8)
    layout_stats_kernel<int64_t><<<1, kStatsThreads, 0, st>>>(offsets, n_offsets, ids, n_ids, out);
  else
    return fail(MAXSIM_EINVAL, "index_bytes must be 4 or 8");
  return launch_check("layout_stats_kernel");
}

int maxsim_b200_contrastive_ce(const float* scores, const int64_t* targets, float* loss_rows,
                               float* dscore, int64_t Nq, int64_t Nb, float temperature,
                               float grad_scale, void* stream) {
  if (Nq < 0 || Nb <= 0 || Nb >= (1ll << 31) || Nq >= (1ll << 31))
    return fail(MAXSIM_EINVAL, "score matrix sizes must be positive and fit int32");
  if (!(temperature > 0.f)) return fail(MAXSIM_EINVAL, "temperature must be > 0");
  if (Nq == 0) return MAXSIM_OK;
  if (!scores || !targets || !loss_rows) return fail(MAXSIM_EINVAL, "null pointer argument");
  contrastive_ce_kernel<<<(unsigned)Nq, kLossThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      scores, targets, loss_rows, dscore, (int)Nb, 1.0f / temperature, grad_scale);
  return launch_check("contrastive_ce_kernel");
}

int maxsim_b200_offsets_from_lengths(const int32_t* lengths, int64_t n, int64_t L_max,
                                     int32_t* offsets, int64_t* total, void* stream) {
  if (n < 0 || L_max < 0 || !fits_i32(L_max)) return fail(MAXSIM_EINVAL, "sizes must be >= 0 and fit int32");
  if (!offsets || (n > 0 && !lengths)) return fail(MAXSIM_EINVAL, "null pointer argument");
  offsets_from_lengths_kernel<<<1, kScanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      lengths, n, (int)L_max, offsets, reinterpret_cast<long long*>(total));
  return launch_check("offsets_from_lengths_kernel");
}

int maxsim_b200_pack_rows(const void* padded, const int32_t* offsets, void* packed,
                          int64_t n_segments, int64_t L_max, int64_t row_bytes,
                          int64_t packed_rows, void* stream) {
  return run_segment_copy<true>(padded, packed, offsets, n_segments, L_max, row_bytes, packed_rows,
                                stream);
}

int maxsim_b200_unpack_rows(const void* packed, const int32_t* offsets, void* padded,
                            int64_t n_segments, int64_t L_max, int64_t row_bytes,
                            int64_t packed_rows, void* stream) {
  return run_segment_copy<false>(packed, padded, offsets, n_segments, L_max, row_bytes, packed_rows,
                                 stream);
}

int maxsim_b200_copy_valid_rows(const void* src, int src_is_host, const int32_t* lengths,
                                void* dst, int64_t n_segments, int64_t L_max, int64_t row_bytes,
                                void* stream) {
  if (n_segments < 0 || L_max < 0 || row_bytes <= 0 || !fits_i32(L_max))
    return fail(MAXSIM_EINVAL, "sizes must be >= 0 (row_bytes > 0) and L_max must fit int32");
  if (n_segments == 0 || L_max == 0) return MAXSIM_OK;
  if (!src || !dst || !lengths) return fail(MAXSIM_EINVAL, "null pointer argument");
  const void* dsrc = src;
  if (src_is_host) {
    void* mapped = nullptr;
    cudaError_t e = cudaHostGetDevicePointer(&mapped, const_cast<void*>(src), 0);
    if (e != cudaSuccess || !mapped) {
      (void)cudaGetLastError();
      return fail(MAXSIM_EINVAL,
                  "source is not page-locked host memory mapped for this device (%s)",
                  cudaGetErrorString(e));
    }
    dsrc = mapped;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  const int64_t slab_bytes = L_max * row_bytes;
  // one CTA per segment at a time unless the segments are few and long
  int64_t gy = 1;
  if (n_segments < 2 * sms) {
    gy = (slab_bytes + 16 * 8 * kCopyThreads - 1) / (16 * 8 * kCopyThreads);
    gy = gy < 1 ? 1 : (gy > 16 ? 16 : gy);
  }
  int64_t gx = n_segments;
  const int64_t cap = (int64_t)sms * 32;
  if (gx * gy > cap) gx = cap / gy;
  dim3 grid((unsigned)gx, (unsigned)gy);
  const bool a16 = aligned16(dsrc) && aligned16(dst) && row_bytes % 16 == 0;
  const bool a4 = ((reinterpret_cast<uintptr_t>(dsrc) | reinterpret_cast<uintptr_t>(dst)) & 3u) == 0 &&
                  row_bytes % 4 == 0;
  if (a16)
    valid_rows_copy_kernel<uint4><<<grid, kCopyThreads, 0, st>>>(dsrc, dst, lengths, n_segments,
                                                                 (int)L_max, row_bytes);
  else if (a4)
    valid_rows_copy_kernel<uint32_t><<<grid, kCopyThreads, 0, st>>>(dsrc, dst, lengths, n_segments,
                                                                    (int)L_max, row_bytes);
  else
    valid_rows_copy_kernel<uint8_t><<<grid, kCopyThreads, 0, st>>>(dsrc, dst, lengths, n_segments,
                                                                   (int)L_max, row_bytes);
  return launch_check("valid_rows_copy_kernel");
}

int maxsim_b200_topk_rows(const float* scores, int64_t rows, int64_t cols, int64_t k,
                          float* values, int64_t* indices, void* stream) {
  if (rows < 0 || cols < 0 || k < 0 || k > cols) return fail(MAXSIM_EINVAL, "need 0 <= k <= cols");
  if (cols > kTopkMaxCols)
    return fail(MAXSIM_EUNSUPPORTED, "topk_rows sorts at most %d columns per row; got %lld",
                kTopkMaxCols, (long long)cols);
  if (rows >= (1ll << 31)) return fail(MAXSIM_EINVAL, "too many rows");
  if (rows == 0 || k == 0) return MAXSIM_OK;
  if (!scores || !values || !indices) return fail(MAXSIM_EINVAL, "null pointer argument");
  int n_pow2 = 2;
  while (n_pow2 < cols) n_pow2 <<= 1;
  const size_t smem = (size_t)n_pow2 * sizeof(unsigned long long);
  static std::atomic<unsigned char> configured[kMaxDevices];
  if (int rc = ensure_smem(topk_rows_kernel, (size_t)kTopkMaxCols * sizeof(unsigned long long), configured))
    return rc;
  topk_rows_kernel<<<(unsigned)rows, kTopkThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      scores, cols, n_pow2, (int)k, values, reinterpret_cast<long long*>(indices));
  return launch_check("topk_rows_kernel");
}

int maxsim_b200_group_pairs(const int32_t* pair_document_ids, int64_t n_pairs,
                            int64_t n_documents, int32_t* bins_scratch, int32_t* order,
                            void* stream) {
  if (n_pairs < 0 || n_documents <= 0 || !fits_i32(n_pairs) || !fits_i32(n_documents))
    return fail(MAXSIM_EINVAL, "n_pairs must be >= 0, n_bins > 0, both within int32");
  if (!bins_scratch) return fail(MAXSIM_EINVAL, "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MAXSIM_CUDA(cudaMemsetAsync(bins_scratch, 0, (size_t)n_documents * sizeof(int32_t), st));
  if (n_pairs == 0) return MAXSIM_OK;
  if (!pair_document_ids || !order) return fail(MAXSIM_EINVAL, "null pointer argument");
  int64_t grid = (n_pairs + kGroupThreads - 1) / kGroupThreads;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (grid > cap) grid = cap;
  group_count_kernel<<<(unsigned)grid, kGroupThreads, 0, st>>>(pair_document_ids, n_pairs,
                                                               (int32_t)n_documents, bins_scratch);
  if (int rc = launch_check("group_count_kernel")) return rc;
  group_scan_kernel<<<1, kGroupScanThreads, 0, st>>>(bins_scratch, (int32_t)n_documents);
  if (int rc = launch_check("group_scan_kernel")) return rc;
  group_scatter_kernel<<<(unsigned)grid, kGroupThreads, 0, st>>>(
      pair_document_ids, n_pairs, (int32_t)n_documents, bins_scratch, order);
  return launch_check("group_scatter_kernel");
}

// Counters of maxsim_b200_group_pairs_static.  In host code the array's name is
// only a handle: its device address comes from cudaGetSymbolAddress, looked up
// once per device with that device current.
constexpr int64_t kStaticGroupBins = 1 << 20;
static __device__ __align__(256) int32_t g_static_group_bins[kStaticGroupBins];

static int static_group_bins(int32_t** out) {
  static std::atomic<int32_t*> cached[kMaxDevices];
  int dev = 0;
  MAXSIM_CUDA(cudaGetDevice(&dev));
  const bool track = dev >= 0 && dev < kMaxDevices;
  int32_t* p = track ? cached[dev].load(std::memory_order_acquire) : nullptr;
  if (!p) {
    MAXSIM_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_group_bins));
    if (track) cached[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return MAXSIM_OK;
}

int maxsim_b200_group_pairs_static(const int32_t* ids, int64_t n_pairs, int64_t n_bins,
                                   int32_t* order, void* stream) {
  if (n_pairs < 0 || n_bins <= 0 || !fits_i32(n_pairs))
    return fail(MAXSIM_EINVAL, "n_pairs must be >= 0 and within int32, n_bins > 0");
  if (n_bins > kStaticGroupBins)
    return fail(MAXSIM_EUNSUPPORTED,
                "n_bins=%lld exceeds the %lld ids the built-in scratch array holds; use "
                "maxsim_b200_group_pairs with caller-provided memory",
                (long long)n_bins, (long long)kStaticGroupBins);
  if (n_pairs == 0) return MAXSIM_OK;
  if (!ids || !order) return fail(MAXSIM_EINVAL, "null pointer argument");
  int32_t* bins = nullptr;
  if (int rc = static_group_bins(&bins)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MAXSIM_CUDA(cudaMemsetAsync(bins, 0, (size_t)n_bins * sizeof(int32_t), st));
  int64_t grid = (n_pairs + kGroupThreads - 1) / kGroupThreads;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (grid > cap) grid = cap;
  group_count_kernel<<<(unsigned)grid, kGroupThreads, 0, st>>>(ids, n_pairs, (int32_t)n_bins, bins);
  if (int rc = launch_check("group_count_kernel")) return rc;
  group_scan_kernel<<<1, kGroupScanThreads, 0, st>>>(bins, (int32_t)n_bins);
  if (int rc = launch_check("group_scan_kernel")) return rc;
  group_scatter_kernel<<<(unsigned)grid, kGroupThreads, 0, st>>>(ids, n_pairs, (int32_t)n_bins, bins,
                                                                 order);
  return launch_check("group_scatter_kernel");
}

int maxsim_forward_ordered(const void* queries, const int32_t* query_offsets,
                           const void* documents, const int32_t* document_offsets,
                           const int32_t* pair_query_ids, const int32_t* pair_document_ids,
                           const int32_t* pair_order, float* scores, int64_t n_pairs,
                           int64_t n_queries, int64_t n_documents, int64_t total_q_tokens,
                           int64_t total_d_tokens, int64_t dim, int64_t max_q_len, int dtype,
                           void* stream) {
  (void)n_queries; (void)n_documents;
  if (!fits_i32(dim) || !fits_i32(max_q_len) || !fits_i32(total_q_tokens) || !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "packed sizes must fit int32 offsets");
  if (max_q_len <= 0) return fail(MAXSIM_EINVAL, "max_q_len must be > 0; got %lld", (long long)max_q_len);
  PairTable t = packed_table(queries, query_offsets, documents, document_offsets, pair_query_ids,
                             pair_document_ids, n_pairs, dim, max_q_len, total_q_tokens,
                             total_d_tokens, pair_order);
  return run_forward<kPacked, false>(t, scores, nullptr, dtype, stream);
}

int maxsim_forward(const void* queries, const int32_t* query_offsets, const void* documents,
                   const int32_t* document_offsets, const int32_t* pair_query_ids,
                   const int32_t* pair_document_ids, float* scores, int64_t n_pairs,
                   int64_t n_queries, int64_t n_documents, int64_t total_q_tokens,
                   int64_t total_d_tokens, int64_t dim, int64_t max_q_len, int dtype,
                   void* stream) {
  return maxsim_forward_ordered(queries, query_offsets, documents, document_offsets,
                                pair_query_ids, pair_document_ids, nullptr, scores, n_pairs,
                                n_queries, n_documents, total_q_tokens, total_d_tokens, dim,
                                max_q_len, dtype, stream);
}

int maxsim_packed_forward_with_argmax_ordered(
    const void* queries, const int32_t* query_offsets, const void* documents,
    const int32_t* document_offsets, const int32_t* pair_query_ids,
    const int32_t* pair_document_ids, const int32_t* pair_order, float* scores, int32_t* argmax,
    int64_t n_pairs, int64_t n_queries, int64_t n_documents, int64_t total_q_tokens,
    int64_t total_d_tokens, int64_t dim, int64_t max_q_len, int dtype, void* stream) {
  (void)n_queries; (void)n_documents;
  if (!fits_i32(dim) || !fits_i32(max_q_len) || !fits_i32(total_q_tokens) || !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "packed sizes must fit int32 offsets");
  if (max_q_len <= 0) return fail(MAXSIM_EINVAL, "max_q_len must be > 0; got %lld", (long long)max_q_len);
  PairTable t = packed_table(queries, query_offsets, documents, document_offsets, pair_query_ids,
                             pair_document_ids, n_pairs, dim, max_q_len, total_q_tokens,
                             total_d_tokens, pair_order);
  return run_forward<kPacked, true>(t, scores, argmax, dtype, stream);
}

int maxsim_packed_forward_with_argmax(const void* queries, const int32_t* query_offsets,
                                      const void* documents, const int32_t* document_offsets,
                                      const int32_t* pair_query_ids,
                                      const int32_t* pair_document_ids, float* scores,
                                      int32_t* argmax, int64_t n_pairs, int64_t n_queries,
                                      int64_t n_documents, int64_t total_q_tokens,
                                      int64_t total_d_tokens, int64_t dim, int64_t max_q_len,
                                      int dtype, void* stream) {
  return maxsim_packed_forward_with_argmax_ordered(
      queries, query_offsets, documents, document_offsets, pair_query_ids, pair_document_ids,
      nullptr, scores, argmax, n_pairs, n_queries, n_documents, total_q_tokens, total_d_tokens,
      dim, max_q_len, dtype, stream);
}

int maxsim_packed_backward_grouped(const float* dscore, const void* queries,
                                   const int32_t* query_offsets, const void* documents,
                                   const int32_t* document_offsets,
                                   const int32_t* pair_query_ids,
                                   const int32_t* pair_document_ids,
                                   const int32_t* order_by_query, const int32_t* ends_by_query,
                                   const int32_t* order_by_document,
                                   const int32_t* ends_by_document, const int32_t* argmax,
                                   float* grad_queries, float* grad_documents, int64_t n_pairs,
                                   int64_t n_queries, int64_t n_documents,
                                   int64_t total_q_tokens, int64_t total_d_tokens, int64_t dim,
                                   int64_t max_q_len, int dtype, void* stream) {
  if (!fits_i32(dim) || !fits_i32(max_q_len) || !fits_i32(total_q_tokens) || !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "packed sizes must fit int32 offsets");
  if (n_queries < 0 || n_documents < 0) return fail(MAXSIM_EINVAL, "sizes must be positive");
  PairTable t = packed_table(queries, query_offsets, documents, document_offsets, pair_query_ids,
                             pair_document_ids, n_pairs, dim, max_q_len, total_q_tokens,
                             total_d_tokens);
  if (order_by_query && ends_by_query && order_by_document && ends_by_document) {
    t.order_q = order_by_query; t.ends_q = ends_by_query;
    t.order_d = order_by_document; t.ends_d = ends_by_document;
  }
  return run_backward<kPacked>(t, dscore, argmax, grad_queries, grad_documents, total_q_tokens,
                               total_d_tokens, 0, dtype, stream, n_queries, n_documents);
}

int maxsim_packed_backward_grouped_native(
    const float* dscore, const void* queries, const int32_t* query_offsets, const void* documents,
    const int32_t* document_offsets, const int32_t* pair_query_ids,
    const int32_t* pair_document_ids, const int32_t* order_by_query, const int32_t* ends_by_query,
    const int32_t* order_by_document, const int32_t* ends_by_document, const int32_t* argmax,
    void* grad_queries, void* grad_documents, int64_t n_pairs, int64_t n_queries,
    int64_t n_documents, int64_t total_q_tokens, int64_t total_d_tokens, int64_t dim,
    int64_t max_q_len, int dtype, void* stream) {
  if (!fits_i32(dim) || !fits_i32(max_q_len) || !fits_i32(total_q_tokens) || !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "packed sizes must fit int32 offsets");
  if (n_queries < 0 || n_documents < 0 || max_q_len <= 0) return fail(MAXSIM_EINVAL, "sizes must be positive");
  const bool ok = (dtype == MAXSIM_F16 || dtype == MAXSIM_BF16) && dim % 8 == 0 && dim <= 128 &&
                  order_by_query && ends_by_query && order_by_document && ends_by_document &&
                  n_pairs > 0 && n_pairs < (1ll << 31) && aligned16(queries) && aligned16(documents) &&
                  aligned16(grad_queries) && aligned16(grad_documents) &&
                  n_queries * max_q_len < (1ll << 33);
  if (!ok)
    return fail(MAXSIM_EUNSUPPORTED, "native-type packed gradients need float16 / bfloat16, grouped "
                                     "pair lists, dim %% 8 == 0, dim <= 128 and aligned tensors");
  if (!dscore || !argmax || !query_offsets || !document_offsets || !pair_query_ids || !pair_document_ids)
    return fail(MAXSIM_EINVAL, "null pointer argument");
  PairTable t = packed_table(queries, query_offsets, documents, document_offsets, pair_query_ids,
                             pair_document_ids, n_pairs, dim, max_q_len, total_q_tokens,
                             total_d_tokens);
  t.order_q = order_by_query; t.ends_q = ends_by_query;
  t.order_d = order_by_document; t.ends_d = ends_by_document;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned threads = kBwdWarps * 32;
  if (n_queries > 0) {
    const int64_t rows = n_queries * max_q_len;
    if (dtype == MAXSIM_F16)
      bwd_dq_packed_kernel<__half><<<(unsigned)((rows + kBwdWarps - 1) / kBwdWarps), threads, 0, st>>>(
          t, dscore, argmax, grad_queries, n_queries, 1);
    else
      bwd_dq_packed_kernel<__nv_bfloat16><<<(unsigned)((rows + kBwdWarps - 1) / kBwdWarps), threads, 0, st>>>(
          t, dscore, argmax, grad_queries, n_queries, 1);
    if (int rc = launch_check("bwd_dq_packed_kernel")) return rc;
  }
  if (n_documents > 0) {
    const size_t smem = (size_t)kBwdWarps * sizeof(PdnWarp);
    const unsigned grid = (unsigned)((n_documents + kBwdWarps - 1) / kBwdWarps);
    if (dtype == MAXSIM_F16)
      bwd_dd_packed_native_kernel<__half><<<grid, threads, smem, st>>>(
          t, dscore, argmax, reinterpret_cast<__half*>(grad_documents), n_documents);
    else
      bwd_dd_packed_native_kernel<__nv_bfloat16><<<grid, threads, smem, st>>>(
          t, dscore, argmax, reinterpret_cast<__nv_bfloat16*>(grad_documents), n_documents);
    if (int rc = launch_check("bwd_dd_packed_native_kernel")) return rc;
  }
  return MAXSIM_OK;
}

int maxsim_packed_backward(const float* dscore, const void* queries, const int32_t* query_offsets,
                           const void* documents, const int32_t* document_offsets,
                           const int32_t* pair_query_ids, const int32_t* pair_document_ids,
                           const int32_t* argmax, float* grad_queries, float* grad_documents,
                           int64_t n_pairs, int64_t n_queries, int64_t n_documents,
                           int64_t total_q_tokens, int64_t total_d_tokens, int64_t dim,
                           int64_t max_q_len, int dtype, void* stream) {
  return maxsim_packed_backward_grouped(dscore, queries, query_offsets, documents, document_offsets,
                                        pair_query_ids, pair_document_ids, nullptr, nullptr,
                                        nullptr, nullptr, argmax, grad_queries, grad_documents,
                                        n_pairs, n_queries, n_documents, total_q_tokens,
                                        total_d_tokens, dim, max_q_len, dtype, stream);
}

int maxsim_padded_forward(const void* queries, const int32_t* query_lengths, const void* documents,
                          const int32_t* doc_lengths, float* scores, int64_t B, int64_t C,
                          int64_t Lq_max, int64_t Ld_max, int64_t dim, int dtype, void* stream) {
  if (B < 0 || C < 0 || Lq_max <= 0 || Ld_max <= 0 || !fits_i32(dim) || !fits_i32(Lq_max) ||
      !fits_i32(Ld_max) || !fits_i32(C))
    return fail(MAXSIM_EINVAL, "Lq_max/Ld_max/num_candidates must all be > 0");
  PairTable t = padded_table(queries, query_lengths, documents, doc_lengths, B, C, Lq_max, Ld_max, dim);
  return run_forward<kPadded, false>(t, scores, nullptr, dtype, stream);
}

int maxsim_padded_forward_with_argmax(const void* queries, const int32_t* query_lengths,
                                      const void* documents, const int32_t* doc_lengths,
                                      float* scores, int32_t* argmax, int64_t B, int64_t C,
                                      int64_t Lq_max, int64_t Ld_max, int64_t dim, int dtype,
                                      void* stream) {
  if (B < 0 || C < 0 || Lq_max <= 0 || Ld_max <= 0 || !fits_i32(dim) || !fits_i32(Lq_max) ||
      !fits_i32(Ld_max) || !fits_i32(C))
    return fail(MAXSIM_EINVAL, "Lq_max/Ld_max/num_candidates must all be > 0");
  PairTable t = padded_table(queries, query_lengths, documents, doc_lengths, B, C, Lq_max, Ld_max, dim);
  return run_forward<kPadded, true>(t, scores, argmax, dtype, stream);
}

int maxsim_padded_backward(const float* dscore, const void* queries, const void* documents,
                           const int32_t* query_lengths, const int32_t* doc_lengths,
                           const int32_t* argmax, float* grad_queries, float* grad_documents,
                           int64_t B, int64_t C, int64_t Lq_max, int64_t Ld_max, int64_t dim,
                           int dtype, void* stream) {
  if (B < 0 || C < 0 || Lq_max <= 0 || Ld_max <= 0 || !fits_i32(dim) || !fits_i32(Lq_max) ||
      !fits_i32(Ld_max) || !fits_i32(C))
    return fail(MAXSIM_EINVAL, "Lq_max/Ld_max/num_candidates must all be > 0");
  PairTable t = padded_table(queries, query_lengths, documents, doc_lengths, B, C, Lq_max, Ld_max, dim);
  return run_backward<kPadded>(t, dscore, argmax, grad_queries, grad_documents, B * Lq_max,
                               B * C * Ld_max, B, dtype, stream);
}

int maxsim_padded_backward_native(const float* dscore, const void* queries, const void* documents,
                                  const int32_t* query_lengths, const int32_t* doc_lengths,
                                  const int32_t* argmax, void* grad_queries, void* grad_documents,
                                  int64_t B, int64_t C, int64_t Lq_max, int64_t Ld_max,
                                  int64_t dim, int dtype, void* stream) {
  if (B < 0 || C < 0 || Lq_max <= 0 || Ld_max <= 0 || !fits_i32(dim) || !fits_i32(Lq_max) ||
      !fits_i32(Ld_max) || !fits_i32(C))
    return fail(MAXSIM_EINVAL, "Lq_max/Ld_max/num_candidates must all be > 0");
  PairTable t = padded_table(queries, query_lengths, documents, doc_lengths, B, C, Lq_max, Ld_max, dim);
  return run_backward_native<kPadded>(t, dscore, argmax, grad_queries, grad_documents, B * Lq_max,
                                      B * C * Ld_max, B, dtype, stream);
}

int maxsim_contrastive_forward(const void* queries, const void* documents,
                               const int32_t* document_offsets, float* scores, int64_t Nq,
                               int64_t Lq, int64_t Nb, int64_t dim, int64_t total_d_tokens,
                               int dtype, void* stream) {
  if (Nq < 0 || Nb < 0 || Lq <= 0 || !fits_i32(dim) || !fits_i32(Lq) || !fits_i32(Nb) ||
      !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "Lq and dim must be > 0 and sizes must fit int32");
  PairTable t = contrastive_table(queries, documents, document_offsets, Nq, Lq, Nb, dim,
                                  total_d_tokens);
  return run_forward<kContrastive, false>(t, scores, nullptr, dtype, stream);
}

int maxsim_contrastive_forward_with_argmax(const void* queries, const void* documents,
                                           const int32_t* document_offsets, float* scores,
                                           int32_t* argmax, int64_t Nq, int64_t Lq, int64_t Nb,
                                           int64_t dim, int64_t total_d_tokens, int dtype,
                                           void* stream) {
  if (Nq < 0 || Nb < 0 || Lq <= 0 || !fits_i32(dim) || !fits_i32(Lq) || !fits_i32(Nb) ||
      !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "Lq and dim must be > 0 and sizes must fit int32");
  PairTable t = contrastive_table(queries, documents, document_offsets, Nq, Lq, Nb, dim,
                                  total_d_tokens);
  return run_forward<kContrastive, true>(t, scores, argmax, dtype, stream);
}

int maxsim_contrastive_forward_with_argmax_block(
    const void* queries, const void* documents, const int32_t* document_offsets, float* scores,
    int32_t* argmax, int64_t Nq, int64_t Lq, int64_t Nb, int64_t dim, int64_t total_d_tokens,
    int64_t block_tokens, int64_t out_ld, int64_t out_col0, int64_t reserve_sms, int dtype,
    void* stream) {
  if (Nq < 0 || Nb < 0 || Lq <= 0 || !fits_i32(dim) || !fits_i32(Lq) || !fits_i32(Nb) ||
      !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "Lq and dim must be > 0 and sizes must fit int32");
  if (out_col0 < 0 || out_ld < out_col0 + Nb || !fits_i32(out_ld))
    return fail(MAXSIM_EINVAL, "the block's columns [%lld, %lld) do not fit a row of %lld",
                (long long)out_col0, (long long)(out_col0 + Nb), (long long)out_ld);
  PairTable t = contrastive_table(queries, documents, document_offsets, Nq, Lq, Nb, dim,
                                  total_d_tokens);
  t.out_ld = out_ld;
  t.out_col0 = out_col0;
  t.block_rows = block_tokens > 0 ? block_tokens : total_d_tokens;
  t.reserve_sms = reserve_sms > 0 ? (int32_t)(reserve_sms < 1024 ? reserve_sms : 1024) : 0;
  return run_forward<kContrastive, true>(t, scores, argmax, dtype, stream);
}

namespace {
int launch_pack_owner_records(const int32_t* argmax, const float* dscore, const int32_t* col_start,
                              int64_t n_owners, int64_t Nq, int64_t Nb, int64_t Lq, int32_t* send,
                              int32_t* const* owner_blocks, void* stream) {
  if (n_owners <= 0 || Nq < 0 || Nb < 0 || Lq <= 0 || !fits_i32(Nq) || !fits_i32(Nb) ||
      !fits_i32(Lq) || !fits_i32(n_owners))
    return fail(MAXSIM_EINVAL, "sizes must be >= 0 (Lq, n_owners > 0) and fit int32");
  if (Nq * Nb == 0) return MAXSIM_OK;
  if (!argmax || !dscore || !col_start || (!send && !owner_blocks))
    return fail(MAXSIM_EINVAL, "null pointer argument");
  if (n_owners > 65535) return fail(MAXSIM_EINVAL, "too many owners");
  // about one wave of CTAs over all owners, each thread copying several words
  int64_t gx = ((int64_t)sm_count() * 8 + n_owners - 1) / n_owners;
  const int64_t need = (Nq * Nb * (Lq + 1) / n_owners + 255) / 256;
  if (gx > need) gx = need > 0 ? need : 1;
  dim3 grid((unsigned)gx, (unsigned)n_owners);
  pack_owner_records_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      argmax, dscore, col_start, (int)Nq, (int)Nb, (int)Lq, send, owner_blocks);
  return launch_check("pack_owner_records_kernel");
}
}  // namespace

int maxsim_b200_pack_owner_records(const int32_t* argmax, const float* dscore,
                                   const int32_t* col_start, int64_t n_owners, int64_t Nq,
                                   int64_t Nb, int64_t Lq, int32_t* send, void* stream) {
  return launch_pack_owner_records(argmax, dscore, col_start, n_owners, Nq, Nb, Lq, send, nullptr,
                                   stream);
}

int maxsim_b200_pack_owner_records_to(const int32_t* argmax, const float* dscore,
                                      const int32_t* col_start, int32_t* const* owner_blocks,
                                      int64_t n_owners, int64_t Nq, int64_t Nb, int64_t Lq,
                                      void* stream) {
  return launch_pack_owner_records(argmax, dscore, col_start, n_owners, Nq, Nb, Lq, nullptr,
                                   owner_blocks, stream);
}

int maxsim_b200_peer_gather(const int64_t* table, int64_t n_segments, int64_t max_bytes, void* dst0,
                            void* dst1, void* stream) {
  if (n_segments < 0 || n_segments > 65535 || max_bytes < 0)
    return fail(MAXSIM_EINVAL, "segment count out of range");
  if (n_segments == 0 || max_bytes == 0) return MAXSIM_OK;
  if (!table || !dst0) return fail(MAXSIM_EINVAL, "null pointer argument");
  // enough CTAs per segment to keep a few loads in flight on every link, never more than the
  // largest segment has 4 KB pieces
  int64_t gx = (max_bytes + 4095) / 4096;
  const int64_t cap = ((int64_t)sm_count() * 4 + n_segments - 1) / n_segments;
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  dim3 grid((unsigned)gx, (unsigned)n_segments);
  peer_gather_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(table, dst0, dst1);
  return launch_check("peer_gather_kernel");
}

int maxsim_b200_copy_many(void* const* dst, const void* const* src, const int64_t* bytes,
                          int64_t n, void* stream) {
  if (n < 0) return fail(MAXSIM_EINVAL, "negative count");
  if (n == 0) return MAXSIM_OK;
  if (!dst || !src || !bytes) return fail(MAXSIM_EINVAL, "null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int64_t i = 0; i < n; ++i) {
    if (bytes[i] < 0) return fail(MAXSIM_EINVAL, "negative size");
    if (bytes[i] == 0) continue;
    if (!dst[i] || !src[i]) return fail(MAXSIM_EINVAL, "null pointer argument");
    MAXSIM_CUDA(cudaMemcpyAsync(dst[i], src[i], (size_t)bytes[i], cudaMemcpyDeviceToDevice, st));
  }
  return MAXSIM_OK;
}

int maxsim_b200_peer_barrier(uint32_t* const* flags, int64_t rank, int64_t world,
                             uint32_t* counter, uint32_t polls, void* stream) {
  if (world <= 0 || world > 1024 || rank < 0 || rank >= world)
    return fail(MAXSIM_EINVAL, "rank / world out of range");
  if (!flags || !counter) return fail(MAXSIM_EINVAL, "null pointer argument");
  const unsigned threads = (unsigned)((world + 31) / 32 * 32);
  peer_barrier_kernel<<<1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      flags, (int)rank, (int)world, counter, polls ? polls : (1u << 24));
  return launch_check("peer_barrier_kernel");
}

int maxsim_contrastive_backward_documents_from_records(
    const int32_t* records, const void* queries, const void* documents,
    const int32_t* document_offsets, void* grad_documents, int64_t Nq, int64_t Lq, int64_t Nb,
    int64_t dim, int64_t total_d_tokens, int dtype, int native, void* stream) {
  if (Nq < 0 || Nb < 0 || Lq <= 0 || !fits_i32(dim) || !fits_i32(Lq) || !fits_i32(Nb) ||
      !fits_i32(total_d_tokens) || !fits_i32(Nq))
    return fail(MAXSIM_EINVAL, "Lq and dim must be > 0 and sizes must fit int32");
  if (!valid_dtype(dtype)) return fail(MAXSIM_EINVAL, "unknown dtype code %d", dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t elem = native ? (dtype == MAXSIM_F32 ? 4 : 2) : 4;
  if (Nq * Nb == 0) {
    if (grad_documents && total_d_tokens)
      MAXSIM_CUDA(cudaMemsetAsync(grad_documents, 0, (size_t)total_d_tokens * dim * elem, st));
    return MAXSIM_OK;
  }
  if (!records || !queries || !documents || !document_offsets || !grad_documents)
    return fail(MAXSIM_EINVAL, "null pointer argument");
  PairTable t = contrastive_table(queries, documents, document_offsets, Nq, Lq, Nb, dim,
                                  total_d_tokens);
  const bool ok = dim % 8 == 0 && aligned16(queries) && aligned16(grad_documents) &&
                  Lq <= kInvEntries && Nq * Lq < (1ll << 31) && (Nq + 1) * Nb * (Lq + 1) < (1ll << 62);
  if (!ok) return fail(MAXSIM_EUNSUPPORTED, "record routing needs dim %% 8 == 0 and aligned tensors");
  if (native && (dtype == MAXSIM_F32 || Nq * Lq > kInvEntries || Nq > kInvMaxQ || dim > 128))
    return fail(MAXSIM_EUNSUPPORTED, "native-type gradients need float16 / bfloat16, Nq * Lq <= %d and dim <= 128",
                kInvEntries);
  switch (dtype) {
    case MAXSIM_F32: return launch_dd_from_records<float>(t, records, grad_documents, Nq, 0, st);
    case MAXSIM_F16: return launch_dd_from_records<__half>(t, records, grad_documents, Nq, native, st);
    default: return launch_dd_from_records<__nv_bfloat16>(t, records, grad_documents, Nq, native, st);
  }
}

int maxsim_contrastive_backward(const float* dscore, const void* queries, const void* documents,
                                const int32_t* document_offsets, const int32_t* argmax,
                                float* grad_queries, float* grad_documents, int64_t Nq, int64_t Lq,
                                int64_t Nb, int64_t dim, int64_t total_d_tokens, int dtype,
                                void* stream) {
  if (Nq < 0 || Nb < 0 || Lq <= 0 || !fits_i32(dim) || !fits_i32(Lq) || !fits_i32(Nb) ||
      !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "Lq and dim must be > 0 and sizes must fit int32");
  PairTable t = contrastive_table(queries, documents, document_offsets, Nq, Lq, Nb, dim,
                                  total_d_tokens);
  return run_backward<kContrastive>(t, dscore, argmax, grad_queries, grad_documents, Nq * Lq,
                                    total_d_tokens, Nq, dtype, stream);
}

int maxsim_contrastive_backward_native(const float* dscore, const void* queries,
                                       const void* documents, const int32_t* document_offsets,
                                       const int32_t* argmax, void* grad_queries,
                                       void* grad_documents, int64_t Nq, int64_t Lq, int64_t Nb,
                                       int64_t dim, int64_t total_d_tokens, int dtype,
                                       void* stream) {
  if (Nq < 0 || Nb < 0 || Lq <= 0 || !fits_i32(dim) || !fits_i32(Lq) || !fits_i32(Nb) ||
      !fits_i32(total_d_tokens))
    return fail(MAXSIM_EINVAL, "Lq and dim must be > 0 and sizes must fit int32");
  PairTable t = contrastive_table(queries, documents, document_offsets, Nq, Lq, Nb, dim,
                                  total_d_tokens);
  return run_backward_native<kContrastive>(t, dscore, argmax, grad_queries, grad_documents,
                                           Nq * Lq, total_d_tokens, Nq, dtype, stream);
}

}  // extern "C"
