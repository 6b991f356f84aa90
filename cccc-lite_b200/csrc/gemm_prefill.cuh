// Prefill-side quantized-weight linear (M > 32 tokens): tcgen05 / TMEM BF16 GEMM.
#pragma once

#include "common.cuh"
#include "gemv_decode.cuh"

namespace b200
{

inline bool prefill_supported(int, unsigned int, unsigned int, unsigned int, unsigned int, unsigned int, unsigned int, unsigned int)
{
    return false;
}

inline int launch_prefill(int, const GemvParams&, int, int, cudaStream_t) { return -2; }

}    // namespace b200
