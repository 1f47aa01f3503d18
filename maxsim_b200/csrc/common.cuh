// Shared device/host helpers for the MaxSim kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace maxsim {

// ---------------------------------------------------------------------------
// Layouts.  A "pair" is one (query, document) score.  The three operator
// families of the reference differ only in how a pair index maps to token
// rows (maxsim_cuda/maxsim.cu:157-160 padded, :1243-1247 contrastive,
// :70-126 packed).
// ---------------------------------------------------------------------------
enum Layout : int { kPadded = 0, kPacked = 1, kContrastive = 2 };

struct PairTable {
  // token matrices, row-major [rows, dim]
  const void* queries;
  const void* documents;
  // padded: ia = query_lengths[B], ib = doc_lengths[B*C]
  // packed: ia = query_offsets, ib = document_offsets, ic = pair_query_ids,
  //         id = pair_document_ids
  // contrastive: ib = document_offsets[Nb+1]
  const int32_t* ia;
  const int32_t* ib;
  const int32_t* ic;
  const int32_t* id;
  // packed only, may be null: processing order.  Position k of the grid works on
  // pair order[k] (a permutation of [0, n_pairs) that puts pairs of the same
  // document next to each other, see group.cuh); results still land in the
  // pair's own slot.
  const int32_t* order;
  // packed backward only, may be null: the pair list grouped by query and by
  // document.  Group b of a grouping is order_x[(b ? ends_x[b-1] : 0) .. ends_x[b]).
  const int32_t* order_q;
  const int32_t* ends_q;
  const int32_t* order_d;
  const int32_t* ends_d;
  int64_t n_pairs;
  int64_t q_rows;    // total query token rows
  int64_t d_rows;    // total document token rows
  int32_t dim;
  int32_t q_slots;   // argmax slots per pair: Lq_max / max_q_len / Lq
  int32_t Ld_max;    // padded only
  int32_t C;         // padded: candidates per query; contrastive: Nb
  // contrastive forward only: pair (q, d) is written to output slot
  // q * out_ld + out_col0 + d, so that launches over different document ranges
  // fill column blocks of one [Nq, out_ld] score matrix (out_ld = Nb, out_col0 =
  // 0 for the ordinary operator).  Only the tcgen05 kernel honours other values.
  int64_t out_ld;
  int64_t out_col0;
  int64_t block_rows;  // document rows this launch covers (d_rows unless a block of a larger tensor)
  int32_t reserve_sms; // SMs the persistent forward leaves free (for a collective running beside it)
};

struct PairGeom {
  int64_t q_row0;  // first query token row
  int64_t d_row0;  // first document token row
  int32_t Lq;
  int32_t Ld;
};

// Pair worked on at grid position `pos`.
template <int LAYOUT>
__device__ __forceinline__ int64_t pair_at(const PairTable& t, int64_t pos) {
  if constexpr (LAYOUT == kPacked) {
    if (t.order) return (int64_t)__ldg(t.order + pos);
  }
  return pos;
}

template <int LAYOUT>
__device__ __forceinline__ PairGeom pair_geom(const PairTable& t, int64_t p) {
  PairGeom g;
  if constexpr (LAYOUT == kPadded) {
    const int64_t b = p / t.C;
    g.q_row0 = b * (int64_t)t.q_slots;
    g.Lq = __ldg(t.ia + b);
    g.d_row0 = p * (int64_t)t.Ld_max;
    g.Ld = __ldg(t.ib + p);
  } else if constexpr (LAYOUT == kPacked) {
    const int32_t qi = __ldg(t.ic + p);
    const int32_t di = __ldg(t.id + p);
    const int32_t q0 = __ldg(t.ia + qi), q1 = __ldg(t.ia + qi + 1);
    const int32_t d0 = __ldg(t.ib + di), d1 = __ldg(t.ib + di + 1);
    g.q_row0 = q0;
    g.Lq = q1 - q0;
    g.d_row0 = d0;
    g.Ld = d1 - d0;
  } else {
    const int64_t qi = p / t.C;
    const int32_t di = (int32_t)(p - qi * t.C);
    const int32_t d0 = __ldg(t.ib + di), d1 = __ldg(t.ib + di + 1);
    g.q_row0 = qi * (int64_t)t.q_slots;
    g.Lq = t.q_slots;
    g.d_row0 = d0;
    g.Ld = d1 - d0;
  }
  // Defensive clamps: a length outside its slot count would index past the
  // argmax row.  Validated inputs never trigger them.
  if (g.Lq > t.q_slots) g.Lq = t.q_slots;
  if (g.Lq < 0) g.Lq = 0;
  if (g.Ld < 0) g.Ld = 0;
  return g;
}

// ---------------------------------------------------------------------------
// Element conversion
// ---------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }

// Device status word: kernels OR a code into it when a bounded wait gives up.
// The library is a single translation unit (abi.cu includes every kernel
// header), so one definition here serves all kernels.
__device__ int g_device_status = 0;

}  // namespace maxsim
