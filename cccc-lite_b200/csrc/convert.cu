// Standalone type conversions of the path: cuda_convert and the FP4 block-scale pair.
// Each result is bit-identical to the reference kernel for the same pair
// (cccc-cuda/cuda_functions.cu:53-126, :2415-2441, :2556-2600, :2727-2785, :2835-2960, :3066-3090);
// the hot ones (FP8 -> BF16, FP4 block-scale -> BF16) move 16 elements per thread with 128-bit
// loads and stores instead of one byte per thread.
#include "common.cuh"
#include "../../include/cccc_cuda_b200.h"

namespace b200
{

constexpr int kThreads = 256;

inline unsigned int grid_for(size_t units)
{
    size_t g = (units + kThreads - 1) / kThreads;
    return (unsigned int)(g ? g : 1);
}

// ---- one unit per thread, any alignment -----------------------------------------------------
template <class F>
__global__ void __launch_bounds__(kThreads) unit_kernel(F f, size_t units)
{
    const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < units) { f(i); }
}

template <class F>
static int run_units(const char* label, size_t units, F f)
{
    if (units)
    {
        unit_kernel<F><<<grid_for(units), kThreads>>>(f, units);
        count_launch();
    }
    return sync_and_report(label);
}

__device__ __forceinline__ uint32_t nibble_at(const uint8_t* src, size_t i)
{
    const uint32_t b = src[i >> 1];
    return (i & 1) ? (b >> 4) : (b & 0xFu);
}

// ---- 16 elements per thread: FP8 -> BF16 -----------------------------------------------------
template <int WT>
__global__ void __launch_bounds__(kThreads) fp8_to_bf16_x16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
    size_t packs, float inv_scale)
{
    const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= packs) { return; }
    const uint4 v = __ldg(src + i);
    const uint32_t w[4] = { v.x, v.y, v.z, v.w };
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; j++)
    {
        uint16_t h[4];
#pragma unroll
        for (int b = 0; b < 4; b++) { h[b] = float_to_bf16_bits_ref(decode_fp8<WT>((w[j] >> (8 * b)) & 0xFFu) * inv_scale); }
        o[2 * j] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
        o[2 * j + 1] = (uint32_t)h[2] | ((uint32_t)h[3] << 16);
    }
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// ---- 16 elements (= one scale block) per thread: FP4 block-scale -> BF16 -----------------------
__global__ void __launch_bounds__(kThreads) fp4bs16_to_bf16_kernel(const uint2* __restrict__ nib, const uint8_t* __restrict__ scales,
    uint4* __restrict__ dst, size_t blocks)
{
    const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= blocks) { return; }
    const uint2 v = __ldg(nib + i);
    const float sc = e4m3_to_float(__ldg(scales + i));
    const uint32_t w[2] = { v.x, v.y };
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
    {
        const uint32_t n0 = (w[j >> 2] >> (8 * (j & 3))) & 0xFu;
        const uint32_t n1 = (w[j >> 2] >> (8 * (j & 3) + 4)) & 0xFu;
        o[j] = (uint32_t)float_to_bf16_bits_ref(fp4_to_float(n0) * sc)
            | ((uint32_t)float_to_bf16_bits_ref(fp4_to_float(n1) * sc) << 16);
    }
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

template <int WT>
static int fp8_to_bf16(const void* src, void* dst, unsigned int n, float inv_scale, const char* label)
{
    size_t packs = 0;
    if (aligned16(src) && aligned16(dst)) { packs = n / 16; }
    if (packs)
    {
        fp8_to_bf16_x16_kernel<WT><<<grid_for(packs), kThreads>>>((const uint4*)src, (uint4*)dst, packs, inv_scale);
        count_launch();
    }
    const size_t done = packs * 16;
    const uint8_t* s = (const uint8_t*)src + done;
    uint16_t* d = (uint16_t*)dst + done;
    return run_units(label, (size_t)n - done,
        [=] __device__(size_t i) { d[i] = float_to_bf16_bits_ref(decode_fp8<WT>(s[i]) * inv_scale); });
}

// ---- the dispatch table of cuda_convert (cuda_functions.cu:3072-3089) ---------------------------
static int convert_dispatch(const void* src, int st, void* dst, int dt, unsigned int n, float scale)
{
    const size_t N = n;
    switch (st * 8 + dt)
    {
    case DT_FLOAT * 8 + DT_BF16:
    {
        auto s = (const float*)src;
        auto d = (__nv_bfloat16*)dst;
        return run_units("float_to_bf16", N, [=] __device__(size_t i) { d[i] = __float2bfloat16(s[i]); });
    }
    case DT_FLOAT * 8 + DT_E4M3:
    {
        auto s = (const float*)src;
        auto d = (uint8_t*)dst;
        return run_units("float_to_fp8e4m3", N, [=] __device__(size_t i) { d[i] = float_to_e4m3(s[i], scale); });
    }
    case DT_FLOAT * 8 + DT_E5M2:
    {
        auto s = (const float*)src;
        auto d = (uint8_t*)dst;
        return run_units("float_to_fp8e5m2", N, [=] __device__(size_t i) { d[i] = float_to_e5m2(s[i], scale); });
    }
    case DT_FLOAT * 8 + DT_FP4:
    {
        auto s = (const float*)src;
        auto d = (uint8_t*)dst;
        return run_units("float_to_fp4", (N + 1) / 2, [=] __device__(size_t i) {
            const size_t e0 = 2 * i;
            const uint32_t lo = float_to_fp4(s[e0] * scale);
            const uint32_t hi = (e0 + 1 < N) ? float_to_fp4(s[e0 + 1] * scale) : 0u;
            d[i] = (uint8_t)(lo | (hi << 4));
        });
    }
    case DT_HALF * 8 + DT_FLOAT:
    {
        auto s = (const __half*)src;
        auto d = (float*)dst;
        return run_units("half_to_float", N, [=] __device__(size_t i) { d[i] = __half2float(s[i]); });
    }
    case DT_HALF * 8 + DT_BF16:
    {
        auto s = (const __half*)src;
        auto d = (__nv_bfloat16*)dst;
        return run_units("half_to_bf16", N, [=] __device__(size_t i) { d[i] = __float2bfloat16(__half2float(s[i])); });
    }
    case DT_BF16 * 8 + DT_FLOAT:
    {
        auto s = (const __nv_bfloat16*)src;
        auto d = (float*)dst;
        return run_units("bf16_to_float", N, [=] __device__(size_t i) { d[i] = __bfloat162float(s[i]); });
    }
    case DT_BF16 * 8 + DT_HALF:
    {
        auto s = (const __nv_bfloat16*)src;
        auto d = (__half*)dst;
        return run_units("bf16_to_half", N, [=] __device__(size_t i) { d[i] = __float2half(__bfloat162float(s[i])); });
    }
    case DT_BF16 * 8 + DT_E4M3:
    {
        auto s = (const uint16_t*)src;
        auto d = (uint8_t*)dst;
        return run_units("bf16_to_fp8e4m3", N,
            [=] __device__(size_t i) { d[i] = float_to_e4m3(bf16_bits_to_float(s[i]), scale); });
    }
    case DT_E4M3 * 8 + DT_FLOAT:
    {
        auto s = (const uint8_t*)src;
        auto d = (float*)dst;
        return run_units("fp8e4m3_to_float", N, [=] __device__(size_t i) { d[i] = e4m3_to_float(s[i]) * scale; });
    }
    case DT_E4M3 * 8 + DT_HALF:
    {
        auto s = (const uint8_t*)src;
        auto d = (__half*)dst;
        return run_units("fp8e4m3_to_half", N,
            [=] __device__(size_t i) { d[i] = __float2half_rn(e4m3_to_float(s[i]) * scale); });
    }
    case DT_E4M3 * 8 + DT_BF16: return fp8_to_bf16<DT_E4M3>(src, dst, n, scale, "fp8e4m3_to_bf16");
    case DT_E5M2 * 8 + DT_FLOAT:
    {
        auto s = (const uint8_t*)src;
        auto d = (float*)dst;
        return run_units("fp8e5m2_to_float", N, [=] __device__(size_t i) { d[i] = e5m2_to_float(s[i]) * scale; });
    }
    case DT_E5M2 * 8 + DT_HALF:
    {
        auto s = (const uint8_t*)src;
        auto d = (__half*)dst;
        return run_units("fp8e5m2_to_half", N,
            [=] __device__(size_t i) { d[i] = __float2half_rn(e5m2_to_float(s[i]) * scale); });
    }
    case DT_E5M2 * 8 + DT_BF16: return fp8_to_bf16<DT_E5M2>(src, dst, n, scale, "fp8e5m2_to_bf16");
    case DT_FP4 * 8 + DT_FLOAT:
    {
        auto s = (const uint8_t*)src;
        auto d = (float*)dst;
        return run_units("fp4_to_float", N, [=] __device__(size_t i) { d[i] = fp4_to_float(nibble_at(s, i)) * scale; });
    }
    case DT_FP4 * 8 + DT_BF16:
    {
        auto s = (const uint8_t*)src;
        auto d = (uint16_t*)dst;
        return run_units("fp4_to_bf16", N,
            [=] __device__(size_t i) { d[i] = float_to_bf16_bits_ref(fp4_to_float(nibble_at(s, i)) * scale); });
    }
    default: return -1;
    }
}

}    // namespace b200

using namespace b200;

C_EXPORT int cuda_convert(const void* src, int src_type, void* dst, int dst_type, unsigned int n, float scale)
{
    if (src_type == dst_type && scale == 1.0f)
    {
        // The reference copies n BYTES here whatever the element size (cuda_functions.cu:3068-3071).
        cudaMemcpy(dst, src, (size_t)n, cudaMemcpyDeviceToDevice);
        return 0;
    }
    if ((unsigned)src_type >= 7 || (unsigned)dst_type >= 7) { return -1; }
    return convert_dispatch(src, src_type, dst, dst_type, n, scale);
}

C_EXPORT int cuda_fp4_blockscale_to_bf16(const void* src_nibbles, const void* src_scales, void* dst, unsigned int n_elems,
    unsigned int block_size)
{
    if (block_size == 0) { return -1; }
    const uint8_t* nib = (const uint8_t*)src_nibbles;
    const uint8_t* sc = (const uint8_t*)src_scales;
    uint16_t* d = (uint16_t*)dst;
    size_t blocks = 0;
    if (block_size == 16 && aligned16(dst) && ((uintptr_t)nib & 7u) == 0) { blocks = n_elems / 16; }
    if (blocks)
    {
        fp4bs16_to_bf16_kernel<<<grid_for(blocks), kThreads>>>((const uint2*)nib, sc, (uint4*)dst, blocks);
        count_launch();
    }
    const size_t done = blocks * 16;
    const size_t N = n_elems;
    return run_units("fp4_blockscale_to_bf16", N - done, [=] __device__(size_t j) {
        const size_t i = done + j;
        d[i] = float_to_bf16_bits_ref(fp4_to_float(nibble_at(nib, i)) * e4m3_to_float(sc[i / block_size]));
    });
}

C_EXPORT int cuda_float_to_fp4_blockscale(const void* src, void* dst_nibbles, void* dst_scales, unsigned int n_elems,
    unsigned int block_size)
{
    if (block_size == 0) { return -1; }
    const float* s = (const float*)src;
    uint8_t* nib = (uint8_t*)dst_nibbles;
    uint8_t* sc = (uint8_t*)dst_scales;
    const size_t N = n_elems;
    const size_t blocks = (N + block_size - 1) / block_size;
    // One thread per block, as the reference (cuda_functions.cu:2896-2923): absmax, the unrounded
    // forward scale for the nibbles, the truncated E4M3 byte of absmax/6 as the stored multiplier.
    return run_units("float_to_fp4_blockscale", blocks, [=] __device__(size_t b) {
        const size_t e0 = b * block_size;
        const size_t e1 = (e0 + block_size < N) ? e0 + block_size : N;
        float absmax = 0.0f;
        for (size_t i = e0; i < e1; i++) { absmax = fmaxf(absmax, fabsf(s[i])); }
        const float fwd = (absmax > 1e-10f) ? (6.0f / absmax) : 1.0f;
        const float dq = (absmax > 1e-10f) ? (absmax / 6.0f) : 1.0f;
        sc[b] = float_to_e4m3(dq, 1.0f);
        for (size_t i = e0; i < e1; i += 2)
        {
            const uint32_t lo = float_to_fp4(s[i] * fwd);
            const uint32_t hi = (i + 1 < N) ? float_to_fp4(s[i + 1] * fwd) : 0u;
            nib[i >> 1] = (uint8_t)(lo | (hi << 4));
        }
    });
}
