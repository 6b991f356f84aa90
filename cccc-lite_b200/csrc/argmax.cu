// Greedy token choice on the device: arg-max over each row of the BF16 logits.
// The reference copies V float logits to the host every token and samples there
// (cccc-llm/cccc-llm.cpp:181-343; with temperature 0 that is the first maximum).  One block per
// token row; ties resolve to the smallest index; NaN entries never win.
#include "common.cuh"
#include "../../include/cccc_cuda_b200.h"

namespace b200
{

__global__ void __launch_bounds__(1024) argmax_bf16_kernel(const uint16_t* __restrict__ x, unsigned int cols, unsigned long long ld,
    int* __restrict__ idx_out, float* __restrict__ val_out)
{
    __shared__ float sv[32];
    __shared__ unsigned int si[32];
    const uint16_t* row = x + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    unsigned int besti = 0xFFFFFFFFu;
    for (unsigned int i = threadIdx.x; i < cols; i += blockDim.x)
    {
        const float v = bf16_bits_to_float(row[i]);
        if (v > best || (v == best && i < besti))
        {
            best = v;
            besti = i;
        }
    }
    auto better = [](float v, unsigned int i, float bv, unsigned int bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const unsigned int oi = __shfl_xor_sync(0xFFFFFFFFu, besti, o);
        if (better(ov, oi, best, besti))
        {
            best = ov;
            besti = oi;
        }
    }
    if ((threadIdx.x & 31) == 0)
    {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = besti;
    }
    __syncthreads();
    if (threadIdx.x < 32)
    {
        const unsigned int nw = (blockDim.x + 31) >> 5;
        best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        besti = threadIdx.x < nw ? si[threadIdx.x] : 0xFFFFFFFFu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
        {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const unsigned int oi = __shfl_xor_sync(0xFFFFFFFFu, besti, o);
            if (better(ov, oi, best, besti))
            {
                best = ov;
                besti = oi;
            }
        }
        if (threadIdx.x == 0)
        {
            idx_out[blockIdx.x] = besti == 0xFFFFFFFFu ? -1 : (int)besti;
            if (val_out) { val_out[blockIdx.x] = best; }
        }
    }
}

}    // namespace b200

C_EXPORT int cuda_argmax_bf16(const void* logits, unsigned int rows, unsigned int cols, unsigned long long ld, void* idx_out,
    void* val_out, void* stream)
{
    if (rows == 0) { return 0; }
    if (!logits || !idx_out || cols == 0) { return -1; }
    b200::argmax_bf16_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>((const uint16_t*)logits, cols, ld, (int*)idx_out, (float*)val_out);
    b200::count_launch();
    return b200::report_launch("argmax_bf16");
}
