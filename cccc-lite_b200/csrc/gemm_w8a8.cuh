// W8A8: E4M3 weights times E4M3 ACTIVATIONS (one scale for the whole activation tensor) with FP32 accumulation, the mode
// the reference selects with act_data_type = FP8_E4M3 (cccc/cublas_real.h:619-666: quantise the BF16 activations, static
// scale or dynamic absmax, then a cublasLt FP8 x FP8 matmul with both scales).  Here the quantised activations are one
// E4M3 row per token of the native-operand FP8 kernel (gemm_native.cuh, PIECES = 1): both operands go into
// tcgen05.mma kind::f8f6f4 as they are.  More than 32 tokens run on CTA pairs (gemm_w8a8_pair.cuh).
#pragma once

#include "gemm_native.cuh"
#include "gemm_w8a8_pair.cuh"

namespace b200
{

constexpr int W8A8_MAX_TOKENS = 32;    // up to here the streaming kernel (all SMs share the k range); above, CTA pairs
// (the streaming kernel with 64 token columns measured slower than the pairs: 27.8 against 20 us for 4096 x 4096 at 64 tokens)

static inline int w8a8_launch_failed()
{
    report_launch("gemm_w8a8_bf16");
    return 1;
}

// Largest |x| over a [rows][cols] BF16 tensor (leading dimension ld) into *absmax (zero before), as the reference's
// absmax_bf16_kernel computes it (cccc-cuda/cuda_functions.cu:2611-2637): fmaxf over |x|, which skips NaN and keeps an
// infinity.  Non-negative floats order as their bits, so the device-wide step is an integer atomicMax.
static __global__ void __launch_bounds__(256) absmax_bf16_rows_kernel(const uint16_t* __restrict__ X, unsigned int ld, unsigned int cols,
    unsigned int rows, float* __restrict__ absmax)
{
    __shared__ unsigned int warp_max[8];
    const unsigned int tid = threadIdx.x;
    unsigned int m = 0;
    for (unsigned int r = blockIdx.y; r < rows; r += gridDim.y)
    {
        const uint16_t* x = X + (size_t)r * ld;
        for (unsigned int i = blockIdx.x * 256 + tid; i < cols; i += gridDim.x * 256)
        {
            const unsigned int b = x[i] & 0x7FFFu;
            if (b <= 0x7F80u) { m = max(m, b); }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o)); }
    if ((tid & 31u) == 0) { warp_max[tid >> 5] = m; }
    __syncthreads();
    if (tid == 0)
    {
#pragma unroll
        for (int w = 1; w < 8; w++) { m = max(m, warp_max[w]); }
        atomicMax(reinterpret_cast<unsigned int*>(absmax), m << 16);
    }
}

// BF16 -> E4M3 with the reference's encoder (float_to_e4m3, cuda_functions.cu:2551-2580).  Dynamic (fwd_static == 0):
// scale = 448 / absmax, multiplier back = absmax / 448 (1 and 1 for an all-zero tensor), cuda_functions.cu:2640-2657;
// static: fwd_static = 1 / act_scale, multiplier back = inv_static = act_scale (cublas_real.h:627-632).
// Grid (column chunks, rows + padding rows): rows past `rows` are written as zeros.  inv_out[r] receives the multiplier
// back for each of the first n_inv rows (the linear reads one per token); pass n_inv = 1 for a single word.
static __global__ void __launch_bounds__(256) quantise_activations_kernel(const uint16_t* __restrict__ X, unsigned int ld, unsigned int cols,
    unsigned int rows, uint8_t* __restrict__ Q, unsigned int ldq, const float* __restrict__ absmax, float fwd_static, float inv_static,
    float* __restrict__ inv_out, unsigned int n_inv, bool pdl, bool src_is_e4m3)
{
    if (pdl)
    {
        pdl_launch_dependents();
        pdl_wait();
    }
    if (src_is_e4m3)
    {
        // the activations are E4M3 already (ld in bytes): they are only moved into the padded rows the linear reads
        const unsigned int r = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
        if (blockIdx.x == 0 && threadIdx.x == 0 && r < n_inv) { inv_out[r] = inv_static; }
        if (i < cols) { Q[(size_t)r * ldq + i] = r < rows ? reinterpret_cast<const uint8_t*>(X)[(size_t)r * ld + i] : (uint8_t)0; }
        return;
    }
    float fwd = fwd_static, inv = inv_static;
    if (fwd_static == 0.f)
    {
        float a;
        if (absmax) { a = *absmax; }
        else
        {
            // a small tensor: every block that quantises finds the largest magnitude itself (eight values per load; the
            // maximum does not depend on the order), which saves the memset and the absmax launch
            __shared__ unsigned int warp_max[8];
            unsigned int m = 0;
            if (blockIdx.y < rows)
            {
                const unsigned int per_row = cols / 8;
                for (unsigned int j = threadIdx.x; j < rows * per_row; j += 256)
                {
                    const uint4 v = *reinterpret_cast<const uint4*>(X + (size_t)(j / per_row) * ld + (size_t)(j % per_row) * 8);
                    const unsigned int w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
                    for (int q = 0; q < 4; q++)
                    {
                        const unsigned int lo = w[q] & 0x7FFFu, hi = (w[q] >> 16) & 0x7FFFu;
                        if (lo <= 0x7F80u) { m = max(m, lo); }
                        if (hi <= 0x7F80u) { m = max(m, hi); }
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o)); }
            if ((threadIdx.x & 31u) == 0) { warp_max[threadIdx.x >> 5] = m; }
            __syncthreads();
#pragma unroll
            for (int w = 0; w < 8; w++) { m = max(m, warp_max[w]); }
            a = __uint_as_float(m << 16);
        }
        fwd = (a > 0.f) ? (448.0f / a) : 1.0f;
        inv = (a > 0.f) ? (a / 448.0f) : 1.0f;
    }
    const unsigned int r = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    if (blockIdx.x == 0 && threadIdx.x == 0 && r < n_inv) { inv_out[r] = inv; }
    if (i >= cols) { return; }
    Q[(size_t)r * ldq + i] = r < rows ? float_to_e4m3(bf16_bits_to_float(X[(size_t)r * ld + i]), fwd) : (uint8_t)0;
}

// The same two steps for many tokens, eight values per thread (16-byte loads, 8-byte stores; cols and ld multiples of 8,
// aligned bases), grid-stride over the [rows][cols / 8] groups.
static __global__ void __launch_bounds__(256) absmax_bf16_x8_kernel(const uint16_t* __restrict__ X, unsigned int ld, unsigned int cols, unsigned int rows,
    float* __restrict__ absmax)
{
    __shared__ unsigned int warp_max[8];
    const unsigned int per_row = cols / 8;
    const unsigned long long groups = (unsigned long long)rows * per_row;
    unsigned int m = 0;
    for (unsigned long long j = (unsigned long long)blockIdx.x * 256 + threadIdx.x; j < groups; j += (unsigned long long)gridDim.x * 256)
    {
        const uint4 v = *reinterpret_cast<const uint4*>(X + (size_t)(j / per_row) * ld + (size_t)(j % per_row) * 8);
        const unsigned int w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int q = 0; q < 4; q++)
        {
            const unsigned int lo = w[q] & 0x7FFFu, hi = (w[q] >> 16) & 0x7FFFu;
            if (lo <= 0x7F80u) { m = max(m, lo); }
            if (hi <= 0x7F80u) { m = max(m, hi); }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o)); }
    if ((threadIdx.x & 31u) == 0) { warp_max[threadIdx.x >> 5] = m; }
    __syncthreads();
    if (threadIdx.x == 0)
    {
#pragma unroll
        for (int w = 1; w < 8; w++) { m = max(m, warp_max[w]); }
        atomicMax(reinterpret_cast<unsigned int*>(absmax), m << 16);
    }
}

static __global__ void __launch_bounds__(256) quantise_activations_x8_kernel(const uint16_t* __restrict__ X, unsigned int ld, unsigned int cols,
    unsigned int rows, uint8_t* __restrict__ Q, const float* __restrict__ absmax, float fwd_static, float inv_static, float* __restrict__ inv_out)
{
    float fwd = fwd_static, inv = inv_static;
    if (fwd_static == 0.f)
    {
        const float a = *absmax;
        fwd = (a > 0.f) ? (448.0f / a) : 1.0f;
        inv = (a > 0.f) ? (a / 448.0f) : 1.0f;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) { *inv_out = inv; }
    const unsigned int per_row = cols / 8;
    const unsigned long long groups = (unsigned long long)rows * per_row;
    for (unsigned long long j = (unsigned long long)blockIdx.x * 256 + threadIdx.x; j < groups; j += (unsigned long long)gridDim.x * 256)
    {
        const size_t r = (size_t)(j / per_row), c = (size_t)(j % per_row) * 8;
        const uint4 v = *reinterpret_cast<const uint4*>(X + r * ld + c);
        const unsigned int w[4] = { v.x, v.y, v.z, v.w };
        unsigned int o[2] = { 0u, 0u };
#pragma unroll
        for (int q = 0; q < 4; q++)
        {
            const unsigned int lo = float_to_e4m3(bf16_bits_to_float((uint16_t)(w[q] & 0xFFFFu)), fwd);
            const unsigned int hi = float_to_e4m3(bf16_bits_to_float((uint16_t)(w[q] >> 16)), fwd);
            o[q >> 1] |= (lo | (hi << 8)) << (16 * (q & 1));
        }
        *reinterpret_cast<uint2*>(Q + r * cols + c) = make_uint2(o[0], o[1]);
    }
}

// The linear(s).  Returns the C-ABI code, -1 for what this path does not serve (K % 128 != 0, unaligned operands, more
// than three members, a workspace that is too small for the quantised activations).  pair_fh: tile shape of the launch
// for more than 32 tokens (0: chosen here).
// x_is_e4m3: X holds E4M3 bytes (ldx in bytes) whose multiplier back is act_scale (> 0); y_e4m3: Y receives E4M3 bytes.
static int launch_w8a8(const GemvScratch* ws, const W8A8Member* mem, unsigned int count, const void* X, float act_scale, unsigned int M,
    unsigned int K, unsigned int ldx, cudaStream_t stream, unsigned int flags, bool x_is_e4m3 = false, bool y_e4m3 = false, unsigned int pair_fh = 0)
{
    if (count == 0 || count > (unsigned int)PF_MAX_GROUP || M == 0 || M > 65535u || act_scale < 0.f) { return -1; }
    const bool big = M > (unsigned int)W8A8_MAX_TOKENS;
    if (x_is_e4m3 && !(act_scale > 0.f)) { return -1; }
    const unsigned int bnp = big ? M : (M <= 16 ? 16u : 32u);    // rows the quantiser writes
    NativeParams np;
    memset(&np, 0, sizeof(np));
    np.n_seg = count;
    np.status = ws->status;
    np.M = M;
    np.K = K;
    np.out_f32 = y_e4m3 ? 3u : ((flags & 4u) ? 1u : ((flags & 8u) ? 2u : 0u));
    np.counters = ws->counters;
    np.nkb = K / NK_BK;
    for (unsigned int j = 0; j < count; j++)
    {
        if (!mem[j].W || !mem[j].Y || !native_supported(DT_E4M3, mem[j].N_out, 1u, K, mem[j].ldw, x_is_e4m3 ? 8u : ldx) || !sk_al16(mem[j].W)) { return -1; }
        PrefillSeg& g = np.seg[j];
        g.W = (const uint8_t*)mem[j].W;
        g.Y = (uint16_t*)mem[j].Y;
        g.N = mem[j].N_out;
        g.ldw = mem[j].ldw;
        g.ldy_m = mem[j].ldy_m;
        g.ldy_n = mem[j].ldy_n;
        g.alpha = mem[j].alpha;
        g.beta = mem[j].beta;
        g.w_scale = 1.0f;
        g.post_scale = mem[j].w_inv_scale;    // both scales multiply the FP32 sums, as cublasLt's scale pointers do
        g.tile0 = np.tiles;
        np.tiles += (mem[j].N_out + NK_BM - 1) / NK_BM;
    }
    const unsigned int grid = big ? 0u : nk_grid(np.tiles, np.nkb, 2ull * (unsigned)ws->sm_count);
    // scratch: [0, 1024): the multipliers back (one per token) and, at float 255, the absmax word; then the E4M3 rows; then partial tiles
    unsigned char* sc = reinterpret_cast<unsigned char*>(ws->partials);
    const size_t q_bytes = (((size_t)bnp * K) + 1023) & ~(size_t)1023;
    const size_t part_bytes = (size_t)2 * grid * M * NK_BM * sizeof(float);
    if (!sc || NK_SCALE_BYTES + q_bytes + part_bytes > ws->partial_bytes || grid > ws->n_counters || ((uintptr_t)sc & 255u) != 0) { return -1; }
    float* inv = reinterpret_cast<float*>(sc);
    float* absmax = inv + 255;
    uint8_t* Q = sc + NK_SCALE_BYTES;
    np.inv_scale = inv;
    np.partials = reinterpret_cast<float*>(Q + q_bytes);
    CUtensorMap tmX;
    StreamWMaps tmW;
    memset(&tmW, 0, sizeof(tmW));
    bool ok = big || make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Q, K, bnp, K, NK_BK, bnp, true);
    for (unsigned int j = 0; j < (unsigned int)PF_MAX_GROUP && ok && !big; j++)
    {
        const W8A8Member& m = mem[j < count ? j : 0];
        ok = make_map_2d(&tmW.w[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, m.W, K, m.N_out, m.ldw, NK_BK, NK_BM, true);
    }
    if (!ok) { return -1; }
    const bool pdl = (flags & 1u) != 0;
    const bool dynamic = act_scale == 0.f && !x_is_e4m3;
    // dynamic scale of a small tensor: the quantiser finds the maximum itself (16-byte loads: K and ldx % 8, an aligned base)
    const bool self_absmax = dynamic && (size_t)M * K <= 16384 && (K % 8) == 0 && (ldx % 8) == 0 && sk_al16(X);
    if (big && x_is_e4m3 && (ldx % 16) == 0 && sk_al16(X))
    {
        // E4M3 activations that TMA can read where they lie: no copy, the multiplier back goes with the launch
        np.inv_scale = nullptr;
        np.act_inv = act_scale;
        return launch_w8a8_pair(np, mem, (const uint8_t*)X, ldx, ws->device, ws->sm_count, pair_fh, stream);
    }
    if (big && !x_is_e4m3 && (K % 8) == 0 && (ldx % 8) == 0 && sk_al16(X))
    {
        // many tokens: eight values per thread, a grid that fills the GPU a few times over
        const unsigned long long groups = (unsigned long long)M * (K / 8);
        unsigned long long blocks = (groups + 255) / 256;
        if (blocks > 16ull * (unsigned)ws->sm_count) { blocks = 16ull * (unsigned)ws->sm_count; }
        if (dynamic)
        {
            if (cudaMemsetAsync(absmax, 0, sizeof(float), stream) != cudaSuccess) { return w8a8_launch_failed(); }
            count_launch();
            absmax_bf16_x8_kernel<<<(unsigned int)blocks, 256, 0, stream>>>((const uint16_t*)X, ldx, K, M, absmax);
        }
        count_launch();
        quantise_activations_x8_kernel<<<(unsigned int)blocks, 256, 0, stream>>>((const uint16_t*)X, ldx, K, M, Q, absmax, dynamic ? 0.f : 1.0f / act_scale,
            dynamic ? 0.f : act_scale, inv);
        if (cudaPeekAtLastError() != cudaSuccess) { return w8a8_launch_failed(); }
        return launch_w8a8_pair(np, mem, Q, K, ws->device, ws->sm_count, pair_fh, stream);
    }
    if (dynamic && !self_absmax)
    {
        if (cudaMemsetAsync(absmax, 0, sizeof(float), stream) != cudaSuccess) { return w8a8_launch_failed(); }
        unsigned int gx = (K + 255) / 256;
        if (gx > 64) { gx = 64; }
        count_launch();
        absmax_bf16_rows_kernel<<<dim3(gx, M), 256, 0, stream>>>((const uint16_t*)X, ldx, K, M, absmax);
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.gridDim = dim3((K + 255) / 256, bnp);
    cfg.blockDim = dim3(256);
    const bool q_pdl = pdl && (!dynamic || self_absmax);    // behind the absmax kernel the quantiser is plainly ordered
    cfg.numAttrs = q_pdl ? 1 : 0;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, quantise_activations_kernel, (const uint16_t*)X, ldx, K, M, Q, K, self_absmax ? (const float*)nullptr : (const float*)absmax,
            dynamic ? 0.f : 1.0f / act_scale, dynamic ? 0.f : act_scale, inv, big ? 1u : M, q_pdl, x_is_e4m3)
        != cudaSuccess)
    {
        return w8a8_launch_failed();
    }
    if (big) { return launch_w8a8_pair(np, mem, Q, K, ws->device, ws->sm_count, pair_fh, stream); }
    auto launch_linear = [&](auto kernel, int smem) -> int {
        static std::atomic<bool> attr_set[2][64];
        const int which = bnp == 16 ? 0 : 1;
        if (!attr_set[which][ws->device].load(std::memory_order_acquire))
        {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) { return w8a8_launch_failed(); }
            attr_set[which][ws->device].store(true, std::memory_order_release);
        }
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(NK_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.numAttrs = 1;    // its weight prefetch does not depend on the quantiser before it
        count_launch();
        if (cudaLaunchKernelEx(&cfg, kernel, tmX, tmW, np) != cudaSuccess) { return w8a8_launch_failed(); }
        return 0;
    };
    return bnp == 16 ? launch_linear(gemm_wq_native_kernel<DT_E4M3, 16, false, 1>, nk_smem_bytes(16))
                     : launch_linear(gemm_wq_native_kernel<DT_E4M3, 32, false, 1>, nk_smem_bytes(32));
}

}    // namespace b200
