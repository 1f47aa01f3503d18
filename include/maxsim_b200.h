/*
 * maxsim_b200 -- C ABI of the sm_100a MaxSim library (libmaxsim_b200.so).
 *
 *   score(q, d) = sum_i max_j <q_i, d_j>
 *
 * One entry point per operator of the reference's torch extension.  The
 * reference declares its nine operators in torch-ext/torch_binding.h:21-165
 * (schemas in torch-ext/torch_binding.cpp:7-90) with torch::Tensor arguments;
 * here every tensor becomes a device pointer plus explicit sizes so that the
 * library carries no torch types.  Conventions shared by all entry points:
 *
 *   - every pointer is a device pointer on the CUDA device that is current
 *     when the call is made; inputs are borrowed and never written;
 *   - outputs are caller-allocated and need no initialisation: each call
 *     defines every element of every output (argmax slots past a pair's query
 *     length are 0, gradient rows nothing routes to are 0);
 *   - `dtype` is a maxsim_dtype value and names the element type of
 *     `queries` and `documents`; scores and gradients are always float,
 *     argmax and all index arrays are int32_t;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL is
 *     the legacy default stream) and the call returns without synchronising;
 *   - the return value is MAXSIM_OK or a negative maxsim_status;
 *     maxsim_b200_last_error() gives a thread-local message for the last
 *     failure.  No C++ exception crosses the boundary;
 *   - empty problems (zero pairs) return MAXSIM_OK without launching.
 *
 * Tie and non-finite semantics (reference: maxsim_cuda/maxsim.cu:416-443,
 * 517-528; tests/test_nan_inf.py:33-92): the first document token reaching
 * the maximum wins; a NaN similarity never wins, so a NaN query token yields
 * a -inf score with argmax 0 and a NaN document token is ignored.
 */
#ifndef MAXSIM_B200_H_
#define MAXSIM_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define MAXSIM_API __attribute__((visibility("default")))
#else
#define MAXSIM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum maxsim_dtype {
  MAXSIM_F32 = 0,
  MAXSIM_F16 = 1,
  MAXSIM_BF16 = 2
} maxsim_dtype;

typedef enum maxsim_status {
  MAXSIM_OK = 0,
  MAXSIM_EINVAL = -1,       /* bad size, null pointer, misaligned base         */
  MAXSIM_EUNSUPPORTED = -2, /* shape outside what the kernels implement        */
  MAXSIM_ECUDA = -3,        /* a CUDA runtime call or launch failed            */
  MAXSIM_EWORKSPACE = -4,   /* workspace missing or too small                  */
  MAXSIM_EDEVICE = -5       /* a kernel reported a bounded wait that ran out   */
} maxsim_status;

/* Library identification and diagnostics (no reference counterpart). */
MAXSIM_API const char* maxsim_b200_version(void);
MAXSIM_API const char* maxsim_b200_last_error(void);
/* Synchronises `stream`, then returns and clears the device-side status word
 * that kernels set when one of their bounded waits gave up (0 = clean). */
MAXSIM_API int maxsim_b200_device_status(void* stream);
/* Exercises the time-out reporting path without putting anything at risk
 * (no reference counterpart): one thread waits `polls` polls (1 .. 2^20) on a
 * barrier nothing arrives at, through the same bounded wait the tensor-core
 * kernels use, gives up, sets the status bit maxsim_b200_device_status
 * reports and writes 1 to *gave_up (device memory, may be NULL).  No copy or
 * MMA is in flight in that kernel, so the device is clean afterwards. */
MAXSIM_API int maxsim_b200_wait_probe(int64_t polls, int* gave_up, void* stream);
/* Number of kernel launches this process has enqueued through the library. */
MAXSIM_API int64_t maxsim_b200_launch_count(void);
/* Selects the forward implementation: 0 = automatic, 1 = force the portable
 * SIMT kernel, 2 = force the warp-MMA streaming kernel where eligible,
 * 3 = the contrastive operators fail instead of leaving the tcgen05 kernel,
 * 8 = as 3 with every document tiled on its own, 9 = as 3 with 128-token tiles
 * that ignore document boundaries (0 and 3 choose between 8 and 9 by average
 * document length).  A process-wide switch for tests and profiling: do not
 * change it while another thread is calling an operator. */
MAXSIM_API void maxsim_b200_set_forward_path(int path);

/* Host-side validation helper (no reference counterpart: the reference copies
 * whole offset / id tensors to the host, torch-ext/maxsim/__init__.py:184-223).
 * Reduces a CSR offsets array and/or an id array (either may be NULL with
 * count 0; elements are int32 when index_bytes == 4, int64 when 8) to eight
 * int64 values written to device memory out8: offsets[0], offsets[n-1],
 * smallest segment, largest segment, smallest id, largest id, n_offsets,
 * n_ids. */
MAXSIM_API int maxsim_b200_layout_stats(const void* offsets, int64_t n_offsets,
                                        const void* ids, int64_t n_ids,
                                        int index_bytes, int64_t* out8, void* stream);

/* Fused in-batch contrastive loss over a score matrix (no reference
 * counterpart; callers of the reference build it from softmax / nll kernels,
 * tests/test_train_convergence.py:34-45).  scores [Nq, Nb] float, targets [Nq]
 * int64 column of each query's positive.  Writes loss_rows [Nq] =
 * logsumexp(scores[q]/T) - scores[q, target]/T and, when dscore is not NULL,
 * dscore [Nq, Nb] = (softmax(scores[q]/T) - onehot(target)) * grad_scale / T. */
MAXSIM_API int maxsim_b200_contrastive_ce(const float* scores, const int64_t* targets,
                                          float* loss_rows, float* dscore,
                                          int64_t Nq, int64_t Nb, float temperature,
                                          float grad_scale, void* stream);

/* Either side of the operators (no compiled reference counterpart: the
 * reference's callers pack with Python slicing and torch.cat, README.md:185-192,
 * or with a boolean-mask gather, torch-ext/maxsim/__init__.py:516-620, and
 * rank with argsort, README.md:270-274).
 *
 * offsets_from_lengths: offsets[0] = 0, offsets[n+1] = offsets[n] +
 * clamp(lengths[n], 0, L_max), int32; *total (device, may be NULL) receives
 * the 64-bit sum.
 * pack_rows: packed[offsets[n] + j] = padded[n, j] for j < offsets[n+1] -
 * offsets[n]; rows are row_bytes bytes of any element type.
 * unpack_rows: the reverse copy; padded[n, j] = 0 for j beyond the segment.
 * Rows at or beyond packed_rows are never read or written.
 * topk_rows: for each of `rows` score rows of `cols` floats the k best
 * entries, best first, equal scores by ascending index, NaN above +inf;
 * values [rows, k] float, indices [rows, k] int64.  cols <= 16384. */
MAXSIM_API int maxsim_b200_offsets_from_lengths(const int32_t* lengths, int64_t n,
                                                int64_t L_max, int32_t* offsets,
                                                int64_t* total, void* stream);
MAXSIM_API int maxsim_b200_pack_rows(const void* padded, const int32_t* offsets, void* packed,
                                     int64_t n_segments, int64_t L_max, int64_t row_bytes,
                                     int64_t packed_rows, void* stream);
MAXSIM_API int maxsim_b200_unpack_rows(const void* packed, const int32_t* offsets, void* padded,
                                       int64_t n_segments, int64_t L_max, int64_t row_bytes,
                                       int64_t packed_rows, void* stream);
/* copy_valid_rows: both tensors are padded [n_segments, L_max, row]; segment
 * n's first lengths[n] rows (lengths on the device) are copied from src to
 * dst, padding rows of dst are left as they are.  src may be device memory or
 * page-locked host memory (its host pointer; the library asks the driver for
 * the device-side mapping and fails with MAXSIM_EINVAL if there is none), in
 * which case the kernel reads it over PCIe and padding never crosses the bus. */
MAXSIM_API int maxsim_b200_copy_valid_rows(const void* src, int src_is_host,
                                           const int32_t* lengths, void* dst,
                                           int64_t n_segments, int64_t L_max,
                                           int64_t row_bytes, void* stream);
MAXSIM_API int maxsim_b200_topk_rows(const float* scores, int64_t rows, int64_t cols, int64_t k,
                                     float* values, int64_t* indices, void* stream);

/* ------------------------------------------------------------------------
 * Packed pair grids.
 * queries [total_q_tokens, dim], query_offsets [n_queries+1],
 * documents [total_d_tokens, dim], document_offsets [n_documents+1],
 * pair_query_ids / pair_document_ids [n_pairs].
 * ---------------------------------------------------------------------- */

/* Replaces maxsim_forward (torch-ext/torch_binding.h, host function
 * maxsim_cuda/maxsim.cu:819-922).  scores [n_pairs]. */
MAXSIM_API int maxsim_forward(const void* queries, const int32_t* query_offsets,
                   const void* documents, const int32_t* document_offsets,
                   const int32_t* pair_query_ids, const int32_t* pair_document_ids,
                   float* scores,
                   int64_t n_pairs, int64_t n_queries, int64_t n_documents,
                   int64_t total_q_tokens, int64_t total_d_tokens,
                   int64_t dim, int64_t max_q_len, int dtype, void* stream);

/* Replaces maxsim_packed_forward_with_argmax (maxsim_cuda/maxsim.cu:2039-2108).
 * scores [n_pairs], argmax [n_pairs, max_q_len]. */
MAXSIM_API int maxsim_packed_forward_with_argmax(
    const void* queries, const int32_t* query_offsets,
    const void* documents, const int32_t* document_offsets,
    const int32_t* pair_query_ids, const int32_t* pair_document_ids,
    float* scores, int32_t* argmax,
    int64_t n_pairs, int64_t n_queries, int64_t n_documents,
    int64_t total_q_tokens, int64_t total_d_tokens,
    int64_t dim, int64_t max_q_len, int dtype, void* stream);

/* Replaces maxsim_packed_backward (maxsim_cuda/maxsim.cu:2201-2286).
 * dscore [n_pairs]; grad_queries [total_q_tokens, dim] and
 * grad_documents [total_d_tokens, dim], both float. */
MAXSIM_API int maxsim_packed_backward(
    const float* dscore,
    const void* queries, const int32_t* query_offsets,
    const void* documents, const int32_t* document_offsets,
    const int32_t* pair_query_ids, const int32_t* pair_document_ids,
    const int32_t* argmax,
    float* grad_queries, float* grad_documents,
    int64_t n_pairs, int64_t n_queries, int64_t n_documents,
    int64_t total_q_tokens, int64_t total_d_tokens,
    int64_t dim, int64_t max_q_len, int dtype, void* stream);

/* Grouping of a packed pair list (no reference counterpart: the reference
 * works through the list in list order, one CTA per entry, and routes
 * gradients with global atomics, maxsim_cuda/maxsim.cu:70-126, 1933-2010,
 * 2122-2169).
 *
 * group_pairs sorts the pair indices by an id (counting sort): order [n_pairs]
 * receives a permutation of [0, n_pairs) in which pairs with the same id are
 * adjacent, ids ascending; ends [n_bins] is scratch memory during the call and
 * afterwards holds, for every id b, the end of its group: the group of b is
 * order[(b ? ends[b-1] : 0) .. ends[b]).  Call it with pair_document_ids /
 * n_documents and with pair_query_ids / n_queries.
 *
 * The *_ordered forward operators are the packed forward operators given the
 * by-document permutation as pair_order (NULL = list order): they visit the
 * pairs in that order, so that a document named by several pairs is read from
 * HBM once and found in L2 afterwards.  maxsim_packed_backward_grouped is
 * maxsim_packed_backward given both groupings: grad_queries is gathered per
 * query and grad_documents is owned by one warp per document, so there is no
 * zero-fill pass, no atomic and no run-to-run difference in the sums' order
 * beyond the order inside a group.  It needs dim % 8 == 0 and 16-byte aligned
 * tensors; otherwise, or with a NULL grouping, it falls back to the plain
 * operator.  Results are those of the plain operators. */
MAXSIM_API int maxsim_b200_group_pairs(const int32_t* ids, int64_t n_pairs, int64_t n_bins,
                                       int32_t* ends, int32_t* order, void* stream);
MAXSIM_API int maxsim_forward_ordered(const void* queries, const int32_t* query_offsets,
                   const void* documents, const int32_t* document_offsets,
                   const int32_t* pair_query_ids, const int32_t* pair_document_ids,
                   const int32_t* pair_order, float* scores,
                   int64_t n_pairs, int64_t n_queries, int64_t n_documents,
                   int64_t total_q_tokens, int64_t total_d_tokens,
                   int64_t dim, int64_t max_q_len, int dtype, void* stream);
MAXSIM_API int maxsim_packed_forward_with_argmax_ordered(
    const void* queries, const int32_t* query_offsets,
    const void* documents, const int32_t* document_offsets,
    const int32_t* pair_query_ids, const int32_t* pair_document_ids,
    const int32_t* pair_order, float* scores, int32_t* argmax,
    int64_t n_pairs, int64_t n_queries, int64_t n_documents,
    int64_t total_q_tokens, int64_t total_d_tokens,
    int64_t dim, int64_t max_q_len, int dtype, void* stream);
MAXSIM_API int maxsim_packed_backward_grouped(
    const float* dscore,
    const void* queries, const int32_t* query_offsets,
    const void* documents, const int32_t* document_offsets,
    const int32_t* pair_query_ids, const int32_t* pair_document_ids,
    const int32_t* order_by_query, const int32_t* ends_by_query,
    const int32_t* order_by_document, const int32_t* ends_by_document,
    const int32_t* argmax,
    float* grad_queries, float* grad_documents,
    int64_t n_pairs, int64_t n_queries, int64_t n_documents,
    int64_t total_q_tokens, int64_t total_d_tokens,
    int64_t dim, int64_t max_q_len, int dtype, void* stream);

/* group_pairs for callers that cannot allocate device memory (no counterpart
 * in the reference).  Same result in `order` as maxsim_b200_group_pairs, but
 * the n_bins counters live in a 4 MB array inside the library (one per GPU
 * that loads it, held until the process exits) instead of caller memory, and
 * the call performs no allocation of any kind.  It is meant for hosts that
 * bind this ABI without a device allocator of their own (a C, Go or Rust
 * service with fixed buffers), for processes that gave all device memory to
 * one pool at start-up, where a later cudaMalloc fails or fragments the pool,
 * and for latency-critical loops that must not run into the device-wide
 * synchronisation cudaMalloc and cudaFree imply.  Limits and rules:
 *  - n_bins <= 1048576 (MAXSIM_EUNSUPPORTED beyond, with a message);
 *  - the first call on a device looks up the array's device address; make it
 *    before any stream capture begins on that device;
 *  - every call uses the same array (it is cleared at the start of each call):
 *    two calls that overlap on the GPU, from different streams or threads,
 *    race on it -- issue them on one stream or serialise them yourself;
 *  - the group ends are not returned; the order feeds the *_ordered forward
 *    operators. */
MAXSIM_API int maxsim_b200_group_pairs_static(const int32_t* ids, int64_t n_pairs,
                                              int64_t n_bins, int32_t* order, void* stream);

/* ------------------------------------------------------------------------
 * Padded candidates.
 * queries [B*Lq_max, dim], query_lengths [B],
 * documents [B*C*Ld_max, dim], doc_lengths [B*C].
 * Pair p = b*C + c scores query b against document slab p.
 * ---------------------------------------------------------------------- */

/* Replaces maxsim_padded_forward (maxsim_cuda/maxsim.cu:924-1024).
 * scores [B*C]. */
MAXSIM_API int maxsim_padded_forward(const void* queries, const int32_t* query_lengths,
                          const void* documents, const int32_t* doc_lengths,
                          float* scores,
                          int64_t B, int64_t C, int64_t Lq_max, int64_t Ld_max,
                          int64_t dim, int dtype, void* stream);

/* Replaces maxsim_padded_forward_with_argmax (maxsim_cuda/maxsim.cu:1036-1116).
 * scores [B*C], argmax [B*C, Lq_max].  Unlike the reference this also accepts
 * MAXSIM_F32 and shapes that are not multiples of 16. */
MAXSIM_API int maxsim_padded_forward_with_argmax(
    const void* queries, const int32_t* query_lengths,
    const void* documents, const int32_t* doc_lengths,
    float* scores, int32_t* argmax,
    int64_t B, int64_t C, int64_t Lq_max, int64_t Ld_max,
    int64_t dim, int dtype, void* stream);

/* Replaces maxsim_padded_backward (maxsim_cuda/maxsim.cu:1124-1210).
 * dscore [B*C]; grad_queries [B*Lq_max, dim], grad_documents [B*C*Ld_max, dim]. */
MAXSIM_API int maxsim_padded_backward(
    const float* dscore,
    const void* queries, const void* documents,
    const int32_t* query_lengths, const int32_t* doc_lengths,
    const int32_t* argmax,
    float* grad_queries, float* grad_documents,
    int64_t B, int64_t C, int64_t Lq_max, int64_t Ld_max,
    int64_t dim, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * Contrastive all-pairs.
 * queries [Nq, Lq, dim] rectangular, documents [total_d_tokens, dim] packed,
 * document_offsets [Nb+1].  Pair p = q*Nb + d.
 * ---------------------------------------------------------------------- */

/* Replaces maxsim_contrastive_forward (maxsim_cuda/maxsim.cu:1718-1779).
 * scores [Nq, Nb]. */
MAXSIM_API int maxsim_contrastive_forward(const void* queries, const void* documents,
                               const int32_t* document_offsets,
                               float* scores,
                               int64_t Nq, int64_t Lq, int64_t Nb, int64_t dim,
                               int64_t total_d_tokens, int dtype, void* stream);

/* Replaces maxsim_contrastive_forward_with_argmax
 * (maxsim_cuda/maxsim.cu:1650-1716).  scores [Nq, Nb], argmax [Nq, Nb, Lq]. */
MAXSIM_API int maxsim_contrastive_forward_with_argmax(
    const void* queries, const void* documents,
    const int32_t* document_offsets,
    float* scores, int32_t* argmax,
    int64_t Nq, int64_t Lq, int64_t Nb, int64_t dim,
    int64_t total_d_tokens, int dtype, void* stream);

/* Column block of a score matrix (no reference counterpart: the reference has
 * no multi-device code; this is what the sharded training driver is built
 * from).  As maxsim_contrastive_forward_with_argmax for the Nb documents
 * described by document_offsets [Nb+1] (absolute token rows of `documents`,
 * which has total_d_tokens rows), except that pair (q, d) is written to slot
 * q * out_ld + out_col0 + d of scores [Nq, out_ld] / argmax [Nq, out_ld, Lq]:
 * launches over different document ranges, or different document tensors,
 * fill one matrix.  block_tokens: tokens in the block if known, else 0 (steers
 * the choice of tiling only).  reserve_sms: SMs the persistent kernel leaves
 * unused, for the kernels of a collective that is meant to run beside this
 * launch (0 = use all).  MAXSIM_EUNSUPPORTED, with nothing written, for
 * shapes outside the tcgen05 kernel (float16 / bfloat16, Lq <= 64, dim a
 * multiple of 16 up to 128, at least 2 * 128 / lanes-per-query queries). */
MAXSIM_API int maxsim_contrastive_forward_with_argmax_block(
    const void* queries, const void* documents, const int32_t* document_offsets,
    float* scores, int32_t* argmax,
    int64_t Nq, int64_t Lq, int64_t Nb, int64_t dim, int64_t total_d_tokens,
    int64_t block_tokens, int64_t out_ld, int64_t out_col0, int64_t reserve_sms,
    int dtype, void* stream);

/* Sharded training, owner exchange (no reference counterpart).
 * pack_owner_records regroups the pairs of a rank's queries by the rank that
 * owns the document: argmax [Nq, Nb, Lq] and dscore [Nq, Nb] become one int32
 * buffer `send` of Nq * Nb * (Lq + 1) words in which owner o's block
 * [Nq, n_o, Lq + 1] -- the Lq winning tokens of each pair, then the bits of
 * its score gradient -- starts at word col_start[o] * Nq * (Lq + 1);
 * col_start [n_owners + 1] (device) holds every owner's first column.
 * backward_documents_from_records computes grad_documents [total_d_tokens,
 * dim] of a rank's own documents from records [Nq, Nb, Lq + 1] (the blocks of
 * all ranks' queries, concatenated in rank order) and all queries
 * [Nq, Lq, dim]; native != 0 writes the gradient in the inputs' 16-bit type
 * (needs Nq * Lq <= 32768, dim <= 128), else float.  MAXSIM_EUNSUPPORTED for
 * shapes the routing kernel does not cover (dim % 8 != 0, misaligned). */
MAXSIM_API int maxsim_b200_pack_owner_records(const int32_t* argmax, const float* dscore,
                                              const int32_t* col_start, int64_t n_owners,
                                              int64_t Nq, int64_t Nb, int64_t Lq,
                                              int32_t* send, void* stream);
MAXSIM_API int maxsim_contrastive_backward_documents_from_records(
    const int32_t* records, const void* queries, const void* documents,
    const int32_t* document_offsets, void* grad_documents,
    int64_t Nq, int64_t Lq, int64_t Nb, int64_t dim, int64_t total_d_tokens,
    int dtype, int native, void* stream);

/* The same exchange over peer-mapped memory instead of a collective (no
 * reference counterpart; the GPUs of one node map each other's buffers).
 * pack_owner_records_to writes owner o's block straight to owner_blocks[o]
 * (device array of n_owners device pointers, each into that owner's memory as
 * mapped in this process, already advanced to where this rank's queries
 * belong): the kernel's stores are the transfer.
 * peer_barrier is the stream-ordered barrier that follows: flags (device
 * array of `world` pointers, flags[r] = rank r's `world` flag words, zero
 * before the first barrier) and `counter`, one device word of this rank, zero
 * before the first barrier, in which the kernel counts the barriers passed
 * (every rank must pass the same sequence of barriers; a barrier captured in a
 * CUDA graph keeps counting at every replay).  Stores made on `stream` before
 * the barrier are visible to a rank's kernels launched after its own barrier.
 * A rank waits at most `polls` polls (0: about ten seconds) for each peer; a
 * wait that runs out sets bit 4 of the word maxsim_b200_device_status reports. */
MAXSIM_API int maxsim_b200_pack_owner_records_to(const int32_t* argmax, const float* dscore,
                                                 const int32_t* col_start,
                                                 int32_t* const* owner_blocks, int64_t n_owners,
                                                 int64_t Nq, int64_t Nb, int64_t Lq, void* stream);
/* peer_gather copies n_segments small segments out of peer-mapped memory with
 * one launch: table (device, n_segments rows of four int64: source address,
 * destination selector 0 / 1, byte offset in that destination, bytes -- a
 * multiple of 4); max_bytes is the largest segment (sizes the grid). */
MAXSIM_API int maxsim_b200_peer_gather(const int64_t* table, int64_t n_segments, int64_t max_bytes,
                                       void* dst0, void* dst1, void* stream);
/* copy_many issues n device-to-device copies on `stream`, one asynchronous
 * copy each (dst, src, bytes: HOST arrays of device addresses and sizes): the
 * fetches of a step's shards out of peer-mapped memory through the copy
 * engines at the cost of one call into the library. */
MAXSIM_API int maxsim_b200_copy_many(void* const* dst, const void* const* src,
                                     const int64_t* bytes, int64_t n, void* stream);
MAXSIM_API int maxsim_b200_peer_barrier(uint32_t* const* flags, int64_t rank, int64_t world,
                                        uint32_t* counter, uint32_t polls, void* stream);

/* Replaces maxsim_contrastive_backward (maxsim_cuda/maxsim.cu:1856-1920).
 * dscore [Nq, Nb]; grad_queries [Nq, Lq, dim], grad_documents
 * [total_d_tokens, dim].  Extension: either gradient pointer may be NULL, in
 * which case that gradient is not computed (the multi-GPU driver computes
 * grad_queries on the rank that holds the queries and grad_documents on the
 * rank that owns the documents). */
MAXSIM_API int maxsim_contrastive_backward(
    const float* dscore,
    const void* queries, const void* documents,
    const int32_t* document_offsets, const int32_t* argmax,
    float* grad_queries, float* grad_documents,
    int64_t Nq, int64_t Lq, int64_t Nb, int64_t dim,
    int64_t total_d_tokens, int dtype, void* stream);

/* As maxsim_packed_backward_grouped with both gradients written once in the
 * inputs' float16 / bfloat16 type (what autograd's cast of the float gradients
 * gives, without the float tensors and the cast's pass over them; reference
 * behaviour replaced: torch-ext/maxsim/__init__.py:448-454 after
 * maxsim_cuda/maxsim.cu:2251-2252).  Needs the four grouping arrays, dim % 8 ==
 * 0, dim <= 128; MAXSIM_EUNSUPPORTED otherwise.  A document with more than 512
 * routed terms is summed in batches with one extra rounding per batch. */
MAXSIM_API int maxsim_packed_backward_grouped_native(
    const float* dscore, const void* queries, const int32_t* query_offsets,
    const void* documents, const int32_t* document_offsets,
    const int32_t* pair_query_ids, const int32_t* pair_document_ids,
    const int32_t* order_by_query, const int32_t* ends_by_query,
    const int32_t* order_by_document, const int32_t* ends_by_document,
    const int32_t* argmax, void* grad_queries, void* grad_documents,
    int64_t n_pairs, int64_t n_queries, int64_t n_documents,
    int64_t total_q_tokens, int64_t total_d_tokens,
    int64_t dim, int64_t max_q_len, int dtype, void* stream);

/* Gradients in the inputs' element type (no compiled reference counterpart:
 * the reference's operators return fp32 gradients, maxsim_cuda/maxsim.cu:
 * 1180-1181, 1896-1897, and its Python layer lets autograd cast them to the
 * leaf dtype, torch-ext/maxsim/__init__.py:771, 954).  Same arguments as
 * maxsim_padded_backward / maxsim_contrastive_backward, but grad_queries and
 * grad_documents are tensors of `dtype` (float16 or bfloat16): every gradient
 * row is summed in fp32 registers and rounded once when it is stored, which is
 * the value the cast of the fp32 result has, without the fp32 tensors and the
 * cast's pass over them.  Only for shapes whose rows are stored exactly once
 * (dim % 8 == 0, dim <= 128, 16-byte aligned tensors; padded: Lq_max <= 32,
 * Ld_max <= 1024; contrastive: Nq * Lq <= 32768); otherwise the status is
 * MAXSIM_EUNSUPPORTED, nothing is launched, and the caller uses the fp32
 * operator. */
MAXSIM_API int maxsim_padded_backward_native(
    const float* dscore, const void* queries, const void* documents,
    const int32_t* query_lengths, const int32_t* doc_lengths, const int32_t* argmax,
    void* grad_queries, void* grad_documents,
    int64_t B, int64_t C, int64_t Lq_max, int64_t Ld_max, int64_t dim,
    int dtype, void* stream);
MAXSIM_API int maxsim_contrastive_backward_native(
    const float* dscore, const void* queries, const void* documents,
    const int32_t* document_offsets, const int32_t* argmax,
    void* grad_queries, void* grad_documents,
    int64_t Nq, int64_t Lq, int64_t Nb, int64_t dim, int64_t total_d_tokens,
    int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MAXSIM_B200_H_ */
