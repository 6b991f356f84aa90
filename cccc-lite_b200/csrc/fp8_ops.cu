// The elementwise ops of the reference's W8A8 mode on E4M3 tensors (cccc-cuda/cuda_functions.cu:2446-2544): every value
// is widened to float, combined, and narrowed with the hardware's round-to-nearest-even, saturating conversion
// (__nv_fp8_e4m3, as the reference does).  Same entry points and arguments; results bit for bit those of the reference's
// kernels (tests/test_gpu_w8a8.py runs both).  HBM-bound: one byte per operand per element; each thread takes sixteen
// consecutive elements as one 16-byte access where the operands allow it, the reference's one byte otherwise.
#include <cuda_fp8.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "../../include/cccc_cuda_b200.h"

namespace b200
{

__device__ __forceinline__ float e4m3_widen(unsigned char b)
{
    __nv_fp8_e4m3 v;
    v.__x = b;
    return (float)v;
}
__device__ __forceinline__ unsigned char e4m3_narrow(float f) { return __nv_fp8_e4m3(f).__x; }

// op(i, a, b, r) -> float for element i with the three operand bytes already widened
template <class Op>
__global__ void __launch_bounds__(256) fp8_elementwise_kernel(const unsigned char* __restrict__ A, const unsigned char* __restrict__ B, unsigned char* R,
    unsigned int n, bool wide, Op op)
{
    const unsigned int t = blockIdx.x * 256 + threadIdx.x;
    if (wide)
    {
        const size_t i0 = (size_t)t * 16;
        if (i0 >= n) { return; }
        const uint4 va = *reinterpret_cast<const uint4*>(A + i0);
        const uint4 vb = B ? *reinterpret_cast<const uint4*>(B + i0) : make_uint4(0, 0, 0, 0);
        const uint4 vr = *reinterpret_cast<const uint4*>(R + i0);
        const unsigned int wa[4] = { va.x, va.y, va.z, va.w }, wb[4] = { vb.x, vb.y, vb.z, vb.w }, wr[4] = { vr.x, vr.y, vr.z, vr.w };
        unsigned int out[4];
#pragma unroll
        for (int q = 0; q < 4; q++)
        {
            out[q] = 0;
#pragma unroll
            for (int e = 0; e < 4; e++)
            {
                const float v = op(e4m3_widen((wa[q] >> (8 * e)) & 0xFFu), e4m3_widen((wb[q] >> (8 * e)) & 0xFFu), e4m3_widen((wr[q] >> (8 * e)) & 0xFFu));
                out[q] |= (unsigned int)e4m3_narrow(v) << (8 * e);
            }
        }
        *reinterpret_cast<uint4*>(R + i0) = make_uint4(out[0], out[1], out[2], out[3]);
        return;
    }
    if (t < n) { R[t] = e4m3_narrow(op(e4m3_widen(A[t]), B ? e4m3_widen(B[t]) : 0.f, e4m3_widen(R[t]))); }
}

template <class Op>
static int launch_fp8_elementwise(const char* label, const void* A, const void* B, void* R, unsigned int n, Op op)
{
    if (n == 0) { return 0; }
    if (!A || !R) { return -1; }
    const bool wide = (n % 16u) == 0 && (((uintptr_t)A | (uintptr_t)B | (uintptr_t)R) & 15u) == 0;
    const unsigned int threads = wide ? n / 16u : n;
    count_launch();
    fp8_elementwise_kernel<<<(threads + 255u) / 256u, 256>>>((const unsigned char*)A, (const unsigned char*)B, (unsigned char*)R, n, wide, op);
    return report_launch(label);
}

// R[i] = a * bias[idx] + b * R[i], idx as MatrixEx::addBias walks it (cuda_functions.cu:2465-2477)
template <class Bias>
__global__ void __launch_bounds__(256) fp8_addbias_kernel(const Bias* __restrict__ bias, unsigned char* R, unsigned int n, unsigned int size_mc,
    unsigned int size_b, float a, float b)
{
    const unsigned int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) { return; }
    const unsigned int idx = (size_mc > 1) ? ((i % (size_mc * size_b)) / size_mc) : (i % size_b);
    float fbias;
    if constexpr (sizeof(Bias) == 1) { fbias = e4m3_widen(bias[idx]); }
    else { fbias = bf16_bits_to_float(bias[idx]); }
    const float fr = (b != 0.0f) ? e4m3_widen(R[i]) * b : 0.0f;
    R[i] = e4m3_narrow(a * fbias + fr);
}

// Embedding rows into an E4M3 activation tensor.  ids are FLOATS holding token numbers, as these two entry points of the
// reference take them ([B][T]); one thread per four consecutive dimensions of a row when D % 4 == 0, else per element.
// MODE 0: E4M3 table at inv_scale_w re-encoded at scale 1 with the hardware conversion (cuda_functions.cu:1615-1640);
// MODE 1: BF16 table encoded with the reference's truncating E4M3 encoder at scale 1 (cuda_functions.cu:1642-1667).
template <int MODE, int VEC>
__global__ void __launch_bounds__(256) embed_to_fp8_kernel(const float* __restrict__ ids, const void* __restrict__ W, unsigned char* __restrict__ Y,
    int D, long long total, float inv_scale_w)
{
    const long long idx = ((long long)blockIdx.x * 256 + threadIdx.x) * VEC;
    if (idx >= total) { return; }
    const int d = (int)(idx % D);
    const long long row = idx / D;    // = t + b * T
    const long long src = d + (long long)(int)ids[row] * D;
    unsigned int out = 0;
#pragma unroll
    for (int e = 0; e < VEC; e++)
    {
        unsigned char q;
        if (MODE == 0) { q = e4m3_narrow(e4m3_widen(reinterpret_cast<const unsigned char*>(W)[src + e]) * inv_scale_w); }
        else { q = float_to_e4m3(bf16_bits_to_float(reinterpret_cast<const uint16_t*>(W)[src + e]), 1.0f); }
        out |= (unsigned int)q << (8 * e);
    }
    if (VEC == 4) { *reinterpret_cast<unsigned int*>(Y + idx) = out; }
    else { Y[idx] = (unsigned char)out; }
}

template <int MODE>
static int launch_embed_to_fp8(const char* label, const void* ids, const void* W, void* Y, int D, int T, int B, float inv_scale_w)
{
    if (D <= 0 || T <= 0 || B <= 0) { return 0; }
    if (!ids || !W || !Y) { return -1; }
    const long long total = (long long)D * T * B;
    const bool vec = (D % 4) == 0 && ((uintptr_t)Y & 3u) == 0;
    const long long threads = vec ? total / 4 : total;
    count_launch();
    if (vec) { embed_to_fp8_kernel<MODE, 4><<<(unsigned int)((threads + 255) / 256), 256>>>((const float*)ids, W, (unsigned char*)Y, D, total, inv_scale_w); }
    else { embed_to_fp8_kernel<MODE, 1><<<(unsigned int)((threads + 255) / 256), 256>>>((const float*)ids, W, (unsigned char*)Y, D, total, inv_scale_w); }
    return report_launch(label);
}

}    // namespace b200

using namespace b200;

/* Replace cuda_embed_fwd_fp8_to_fp8 and cuda_embed_fwd_bf16_to_fp8 (cccc-cuda/cuda_functions.cu:1615-1667). */
C_EXPORT int cuda_embed_fwd_fp8_to_fp8(const void* ids, const void* W, void* Y, int D, int T, int B, float inv_scale_w)
{
    return launch_embed_to_fp8<0>("embed_fwd_fp8_to_fp8", ids, W, Y, D, T, B, inv_scale_w);
}
C_EXPORT int cuda_embed_fwd_bf16_to_fp8(const void* ids, const void* W, void* Y, int D, int T, int B)
{
    return launch_embed_to_fp8<1>("embed_fwd_bf16_to_fp8", ids, W, Y, D, T, B, 1.0f);
}

/* Replaces cuda_add_fp8e4m3 (cccc-cuda/cuda_functions.cu:2446-2463): R = a A + b B + r R on E4M3 tensors. */
C_EXPORT int cuda_add_fp8e4m3(const void* A, const void* B, void* R, unsigned int n, float a, float b, float r)
{
    if (n != 0 && !B) { return -1; }
    return launch_fp8_elementwise("add_fp8e4m3", A, B, R, n, [=] __device__(float fa, float fb, float fr0) {
        const float fr = (r != 0.f) ? fr0 * r : 0.f;
        return a * fa + b * fb + fr;
    });
}

/* Replaces cuda_silu_fp8e4m3 (cuda_functions.cu:2506-2520): R = x * sigmoid(x). */
C_EXPORT int cuda_silu_fp8e4m3(const void* A, void* R, unsigned int n)
{
    return launch_fp8_elementwise("silu_fp8e4m3", A, nullptr, R, n, [=] __device__(float x, float, float) { return x / (1.0f + expf(-x)); });
}

/* Replaces cuda_elementmul_fp8e4m3 (cuda_functions.cu:2522-2540): R = a A B + r R. */
C_EXPORT int cuda_elementmul_fp8e4m3(const void* A, const void* B, void* R, unsigned int n, float a, float r)
{
    if (n != 0 && !B) { return -1; }
    return launch_fp8_elementwise("elementmul_fp8e4m3", A, B, R, n, [=] __device__(float fa, float fb, float fr0) {
        const float fr = (r != 0.f) ? fr0 * r : 0.f;
        return a * fa * fb + fr;
    });
}

/* Replace cuda_addbias_fp8e4m3 and cuda_addbias_fp8e4m3_bf16bias (cuda_functions.cu:2465-2504): the caller has copied X
 * into R; R = a * bias[idx] + b * R. */
C_EXPORT int cuda_addbias_fp8e4m3(const void* X, const void* bias, void* R, unsigned int n, unsigned int size_mc, unsigned int size_b, float a,
    float b)
{
    (void)X;
    if (n == 0) { return 0; }
    if (!bias || !R || size_b == 0) { return -1; }
    count_launch();
    fp8_addbias_kernel<unsigned char><<<(n + 255u) / 256u, 256>>>((const unsigned char*)bias, (unsigned char*)R, n, size_mc, size_b, a, b);
    return report_launch("addbias_fp8e4m3");
}
C_EXPORT int cuda_addbias_fp8e4m3_bf16bias(const void* X, const void* bias, void* R, unsigned int n, unsigned int size_mc, unsigned int size_b,
    float a, float b)
{
    (void)X;
    if (n == 0) { return 0; }
    if (!bias || !R || size_b == 0) { return -1; }
    count_launch();
    fp8_addbias_kernel<uint16_t><<<(n + 255u) / 256u, 256>>>((const uint16_t*)bias, (unsigned char*)R, n, size_mc, size_b, a, b);
    return report_launch("addbias_fp8e4m3_bf16bias");
}
