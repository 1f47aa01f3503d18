// Fused in-batch contrastive loss on top of the score matrix: temperature
// scaling, row-wise cross-entropy against one target column per query, and the
// gradient with respect to the scores, in one pass over [Nq, Nb].  This is the
// loss every caller of the contrastive operator in the reference builds out of
// separate softmax / nll kernels (tests/test_train_convergence.py:34-45,
// examples/03_contrastive_training.py:103-114); it has no counterpart among
// the reference's operators.
#pragma once

#include "common.cuh"

namespace maxsim {

constexpr int kLossThreads = 256;

// loss_rows[q] = logsumexp_d(s[q,d] / T) - s[q,target[q]] / T
// dscore[q,d]  = (softmax_d(s[q,:] / T)[d] - [d == target[q]]) * grad_scale / T
__global__ void __launch_bounds__(kLossThreads)
contrastive_ce_kernel(const float* __restrict__ scores, const int64_t* __restrict__ targets,
                      float* __restrict__ loss_rows, float* __restrict__ dscore, int Nb,
                      float inv_temperature, float grad_scale) {
  __shared__ float red[kLossThreads / 32];
  __shared__ float bcast;
  const int q = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = scores + (int64_t)q * Nb;
  float mx = neg_inf();
  for (int d = tid; d < Nb; d += kLossThreads) mx = fmaxf(mx, row[d] * inv_temperature);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = red[0];
    for (int w = 1; w < kLossThreads / 32; ++w) m = fmaxf(m, red[w]);
    bcast = m;
  }
  __syncthreads();
  mx = bcast;
  float sum = 0.f;
  for (int d = tid; d < Nb; d += kLossThreads) sum += expf(row[d] * inv_temperature - mx);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int w = 0; w < kLossThreads / 32; ++w) t += red[w];
    bcast = t;
  }
  __syncthreads();
  sum = bcast;
  const int64_t tgt = targets[q];
  const float inv_sum = 1.0f / sum;
  if (tid == 0) {
    const float st = (tgt >= 0 && tgt < Nb) ? row[tgt] * inv_temperature : neg_inf();
    loss_rows[q] = (mx + logf(sum)) - st;
  }
  if (dscore) {
    float* out = dscore + (int64_t)q * Nb;
    const float k = grad_scale * inv_temperature;
    for (int d = tid; d < Nb; d += kLossThreads) {
      const float p = expf(row[d] * inv_temperature - mx) * inv_sum;
      out[d] = (p - (d == tgt ? 1.0f : 0.0f)) * k;
    }
  }
}

}  // namespace maxsim
