// tcgen05 / TMEM contrastive forward.
#pragma once

#include "common.cuh"

namespace maxsim {

inline bool tc05_eligible(const PairTable&, int) { return false; }

template <bool ARGMAX>
int launch_tc05(const PairTable&, float*, int32_t*, int, cudaStream_t) { return -2; }

}  // namespace maxsim
