/*
 * CPU oracle for cccc's quantized-weight linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic the reference performs on this path so
 * that the CUDA kernels can be checked against it.  It is never linked into, imported by
 * or called from the product library; only the tests, the smoke check and the CPU-baseline
 * leg of the benchmark load it.
 *
 * Each function names the reference code it follows (paths are relative to the
 * scarsty/cccc-lite tree).  The reference ships no golden vectors for this path, so the
 * restatement is pinned by (1) known-answer tables produced by compiling the reference's
 * own cccc/types.h (committed under tests/golden/) and (2) on a GPU, the reference's own
 * cccc-cuda/cuda_functions.cu compiled unmodified.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static inline float bits2f(uint32_t u)
{
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint32_t f2bits(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

/* ---- scalar codecs ------------------------------------------------------------------ */

/* cccc/types.h:72-90 and cccc-cuda/cuda_functions.cu:2366-2381: E4M3 byte -> float.
 * bias 7, 0x7F/0xFF are NaN, no Inf, subnormal = m * 2^-9. */
ORACLE_API float oracle_e4m3_to_float(uint8_t b)
{
    const uint32_t s = (b >> 7) & 1u;
    const int e = (b >> 3) & 0xF;
    const int m = b & 7;
    if (e == 15 && m == 7) { return bits2f(0x7FC00000u); }
    if (e == 0) { return (s ? -1.f : 1.f) * (float)m * (1.f / 512.f); }
    return bits2f((s << 31) | ((uint32_t)(e + 120) << 23) | ((uint32_t)m << 20));
}

/* cccc/types.h:139-166 and cuda_functions.cu:2674-2693: E5M2 byte -> float.
 * bias 15, e==31 is Inf (m==0) or NaN, subnormal = m * 2^-16. */
ORACLE_API float oracle_e5m2_to_float(uint8_t b)
{
    const uint32_t s = (b >> 7) & 1u;
    const int e = (b >> 2) & 0x1F;
    const int m = b & 3;
    if (e == 31) { return m == 0 ? bits2f((s << 31) | 0x7F800000u) : bits2f(0x7FC00000u); }
    if (e == 0) { return (s ? -1.f : 1.f) * (float)m * (1.f / 65536.f); }
    return bits2f((s << 31) | ((uint32_t)(e + 112) << 23) | ((uint32_t)m << 21));
}

/* cccc/types.h:92-126 and cuda_functions.cu:2382-2415: float*scale -> E4M3 by mantissa
 * TRUNCATION, saturating to 0x7E (448); NaN -> 0x7F. */
ORACLE_API uint8_t oracle_float_to_e4m3(float f, float scale)
{
    f *= scale;
    const uint32_t u = f2bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) { return 0x7Fu; }
    const uint32_t s = u >> 31;
    const int fe = (int)((u >> 23) & 0xFFu) - 127;
    const uint32_t fm = u & 0x7FFFFFu;
    if (fe > 8 || (fe == 8 && fm >= 0xC00000u)) { return (uint8_t)((s << 7) | 0x7Eu); }
    const int e8 = fe + 7;
    if (e8 <= 0)
    {
        const int shift = 14 - fe;
        if (shift >= 32) { return (uint8_t)(s << 7); }
        return (uint8_t)((s << 7) | (((fm | 0x800000u) >> shift) & 0x7u));
    }
    uint8_t m8 = (uint8_t)(fm >> 20);
    if (e8 == 15 && m8 == 7) { m8 = 6; }
    return (uint8_t)((s << 7) | ((uint8_t)(e8 & 0xF) << 3) | m8);
}

/* cccc/types.h:168-199 and cuda_functions.cu:2694-2725: float*scale -> E5M2 by mantissa
 * TRUNCATION, saturating to 0x7B (57344); NaN and Inf -> 0x7C with sign for Inf. */
ORACLE_API uint8_t oracle_float_to_e5m2(float f, float scale)
{
    f *= scale;
    const uint32_t u = f2bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) { return 0x7Cu; }
    const uint32_t s = u >> 31;
    if ((u & 0x7FFFFFFFu) == 0x7F800000u) { return (uint8_t)((s << 7) | 0x7Cu); }
    const int fe = (int)((u >> 23) & 0xFFu) - 127;
    const uint32_t fm = u & 0x7FFFFFu;
    if (fe > 15 || (fe == 15 && fm >= 0xE00000u)) { return (uint8_t)((s << 7) | 0x7Bu); }
    const int e8 = fe + 15;
    if (e8 <= 0)
    {
        const int shift = 7 - fe;
        if (shift >= 32) { return (uint8_t)(s << 7); }
        return (uint8_t)((s << 7) | (((fm | 0x800000u) >> shift) & 0x3u));
    }
    return (uint8_t)((s << 7) | ((uint8_t)(e8 & 0x1F) << 2) | (uint8_t)(fm >> 21));
}

/* cccc/types.h:210-211 and cuda_functions.cu:2791-2794: E2M1 nibble value table. */
static const float k_fp4_table[16] = { 0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
    0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f };

ORACLE_API float oracle_fp4_nibble_to_float(uint8_t nibble) { return k_fp4_table[nibble & 0xF]; }

/* cccc/types.h:218-255 and cuda_functions.cu:2796-2832: float -> E2M1 nibble by "<"
 * threshold compares (0.25 .75 1.25 1.75 2.5 3.5 5); the sign bit is set for f<0 only. */
ORACLE_API uint8_t oracle_float_to_fp4(float f)
{
    const uint8_t s = (f < 0.f) ? 8u : 0u;
    if (f < 0.f) { f = -f; }
    if (f < 0.25f) { return s; }
    if (f < 0.75f) { return s | 1u; }
    if (f < 1.25f) { return s | 2u; }
    if (f < 1.75f) { return s | 3u; }
    if (f < 2.5f) { return s | 4u; }
    if (f < 3.5f) { return s | 5u; }
    if (f < 5.0f) { return s | 6u; }
    return s | 7u;
}

/* cuda_functions.cu:2761-2764 (and :2571-2575, :2883-2886, :2935-2937): float -> BF16 by the
 * integer round-to-nearest-even trick.  The addition is allowed to wrap exactly as the
 * reference's does (a 0x7FFFFFFF NaN becomes 0x8000). */
ORACLE_API uint16_t oracle_float_to_bf16_rne(float f)
{
    uint32_t u = f2bits(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

ORACLE_API float oracle_bf16_to_float(uint16_t h) { return bits2f((uint32_t)h << 16); }

/* cccc/types.h:43-48: the HOST bfloat16(float) constructor truncates. */
ORACLE_API uint16_t oracle_float_to_bf16_trunc(float f) { return (uint16_t)(f2bits(f) >> 16); }

/* ---- array conversions (the device kernels of the path) ------------------------------ */

/* A device multiply of a NaN yields the canonical 0x7FFFFFFF on NVIDIA GPUs, whatever the
 * NaN operand's payload.  The reference's dequant kernels multiply before rounding, so the
 * oracle canonicalises the same way when asked to model the device result. */
static inline float dev_mul(float a, float b)
{
    const float r = a * b;
    return (r != r) ? bits2f(0x7FFFFFFFu) : r;
}

/* cuda_functions.cu:2756-2771 (type 5) and :2566-2582 (type 4):
 * dst[i] = RNE_bf16(decode(src[i]) * inv_scale). */
ORACLE_API void oracle_fp8_to_bf16(const uint8_t* src, int src_type, uint16_t* dst, size_t n, float inv_scale)
{
    for (size_t i = 0; i < n; i++)
    {
        const float v = (src_type == 5) ? oracle_e5m2_to_float(src[i]) : oracle_e4m3_to_float(src[i]);
        dst[i] = oracle_float_to_bf16_rne(dev_mul(v, inv_scale));
    }
}

/* cuda_functions.cu:2735-2753 / :2424-2431: fp8 -> float (no bf16 rounding). */
ORACLE_API void oracle_fp8_to_float(const uint8_t* src, int src_type, float* dst, size_t n, float inv_scale)
{
    for (size_t i = 0; i < n; i++)
    {
        const float v = (src_type == 5) ? oracle_e5m2_to_float(src[i]) : oracle_e4m3_to_float(src[i]);
        dst[i] = dev_mul(v, inv_scale);
    }
}

/* cuda_functions.cu:2727-2734 / :2415-2422: float -> fp8 with forward scale. */
ORACLE_API void oracle_float_to_fp8(const float* src, uint8_t* dst, int dst_type, size_t n, float scale)
{
    for (size_t i = 0; i < n; i++)
    {
        dst[i] = (dst_type == 5) ? oracle_float_to_e5m2(src[i], scale) : oracle_float_to_e4m3(src[i], scale);
    }
}

/* cuda_functions.cu:2872-2889: packed FP4 -> BF16 with one per-tensor multiplier;
 * low nibble = even element. */
ORACLE_API void oracle_fp4_to_bf16(const uint8_t* src, uint16_t* dst, size_t n, float inv_scale)
{
    for (size_t i = 0; i < n; i++)
    {
        const uint8_t nib = (i & 1) ? (src[i >> 1] >> 4) : (src[i >> 1] & 0xF);
        dst[i] = oracle_float_to_bf16_rne(k_fp4_table[nib] * inv_scale);
    }
}

/* cuda_functions.cu:2849-2858: packed FP4 -> float. */
ORACLE_API void oracle_fp4_packed_to_float(const uint8_t* src, float* dst, size_t n, float inv_scale)
{
    for (size_t i = 0; i < n; i++)
    {
        const uint8_t nib = (i & 1) ? (src[i >> 1] >> 4) : (src[i >> 1] & 0xF);
        dst[i] = k_fp4_table[nib] * inv_scale;
    }
}

/* cuda_functions.cu:2836-2847: float -> packed FP4 with forward scale. */
ORACLE_API void oracle_float_to_fp4_packed(const float* src, uint8_t* dst, size_t n, float scale)
{
    for (size_t e0 = 0; e0 < n; e0 += 2)
    {
        const uint8_t lo = oracle_float_to_fp4(src[e0] * scale);
        const uint8_t hi = (e0 + 1 < n) ? oracle_float_to_fp4(src[e0 + 1] * scale) : 0u;
        dst[e0 >> 1] = (uint8_t)(lo | (hi << 4));
    }
}

/* cuda_functions.cu:2926-2939: block-scale FP4 -> BF16.  Block = `block_size` consecutive
 * elements of the flat buffer; the scale is an E4M3 byte used as a dequant multiplier. */
ORACLE_API void oracle_fp4_blockscale_to_bf16(const uint8_t* nibbles, const uint8_t* scales, uint16_t* dst,
    size_t n, unsigned block_size)
{
    for (size_t i = 0; i < n; i++)
    {
        const float sc = oracle_e4m3_to_float(scales[i / block_size]);
        const uint8_t nib = (i & 1) ? (nibbles[i >> 1] >> 4) : (nibbles[i >> 1] & 0xF);
        dst[i] = oracle_float_to_bf16_rne(dev_mul(k_fp4_table[nib], sc));
    }
}

/* cuda_functions.cu:2896-2923: float -> block-scale FP4.  Per block: absmax; the forward
 * scale 6/absmax is used UNROUNDED for the nibbles while absmax/6 is stored as a
 * truncating E4M3 byte; blocks with absmax <= 1e-10 use 1.0 for both. */
ORACLE_API void oracle_float_to_fp4_blockscale(const float* src, uint8_t* nibbles, uint8_t* scales, size_t n,
    unsigned block_size)
{
    const size_t n_blocks = (n + block_size - 1) / block_size;
    for (size_t b = 0; b < n_blocks; b++)
    {
        const size_t s0 = b * block_size;
        const size_t s1 = (s0 + block_size < n) ? s0 + block_size : n;
        float absmax = 0.f;
        for (size_t i = s0; i < s1; i++) { absmax = fmaxf(absmax, fabsf(src[i])); }
        const float fwd = (absmax > 1e-10f) ? (6.0f / absmax) : 1.0f;
        const float dq = (absmax > 1e-10f) ? (absmax / 6.0f) : 1.0f;
        scales[b] = oracle_float_to_e4m3(dq, 1.0f);
        for (size_t i = s0; i < s1; i += 2)
        {
            const uint8_t lo = oracle_float_to_fp4(src[i] * fwd);
            const uint8_t hi = (i + 1 < n) ? oracle_float_to_fp4(src[i + 1] * fwd) : 0u;
            nibbles[i >> 1] = (uint8_t)(lo | (hi << 4));
        }
    }
}

/* cuda_functions.cu:76-93: float -> BF16 with __float2bfloat16 (RNE, NaN -> 0x7FFF). */
ORACLE_API void oracle_float_to_bf16(const float* src, uint16_t* dst, size_t n)
{
    for (size_t i = 0; i < n; i++)
    {
        const uint32_t u = f2bits(src[i]);
        dst[i] = ((u & 0x7FFFFFFFu) > 0x7F800000u) ? (uint16_t)0x7FFFu : oracle_float_to_bf16_rne(src[i]);
    }
}

/* ---- the linear itself --------------------------------------------------------------- */

/* Weight element (n,k) of a [N,K] row-major quantised weight, dequantised exactly as the
 * reference's GPU path does before its BF16 GEMM (cccc/cublas_real.h:943-956):
 *   types 4/5 : RNE_bf16(decode(byte) * inv_scale)
 *   type 6    : block scales given -> RNE_bf16(table[nib] * e4m3(scale[(n*ldw+k)/16]))
 *               else               -> RNE_bf16(table[nib] * inv_scale)
 * ldw is in ELEMENTS. */
static inline float dequant_w(int w_type, const uint8_t* W, const uint8_t* blk, float inv_scale, size_t idx)
{
    uint16_t h;
    if (w_type == 6)
    {
        const uint8_t nib = (idx & 1) ? (W[idx >> 1] >> 4) : (W[idx >> 1] & 0xF);
        const float sc = blk ? oracle_e4m3_to_float(blk[idx / 16]) : inv_scale;
        h = oracle_float_to_bf16_rne(dev_mul(k_fp4_table[nib], sc));
    }
    else
    {
        const float v = (w_type == 5) ? oracle_e5m2_to_float(W[idx]) : oracle_e4m3_to_float(W[idx]);
        h = oracle_float_to_bf16_rne(dev_mul(v, inv_scale));
    }
    return oracle_bf16_to_float(h);
}

/* The quantised-weight linear as the reference's GPU path defines it
 * (cccc/cublas_real.h:943-964: dequantise the whole weight to BF16, then
 * cublasGemmEx BF16 x BF16 -> BF16 with FP32 compute, C = alpha*op(A)*op(B) + beta*C):
 *   Y[m*ldy_m + n*ldy_n] = RNE_bf16( alpha * sum_k Wdq[n,k] * X[m*ldx+k] + beta * Y[...] )
 * The sum is accumulated in DOUBLE here so that the oracle is the mathematical value up to
 * one final rounding; the CUDA kernels accumulate in FP32 in a different order, and the
 * tests bound the difference (max relative error 1e-2, cosine >= 0.9999).
 * y32 (optional) receives the unrounded value. */
ORACLE_API void oracle_linear_wq_bf16(int w_type, const uint8_t* W, const uint8_t* blk, float inv_scale,
    const uint16_t* X, uint16_t* Y, float* y32, size_t N, size_t M, size_t K, size_t ldw, size_t ldx,
    size_t ldy_m, size_t ldy_n, float alpha, float beta)
{
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < (long long)N; n++)
    {
        float* wrow = (float*)malloc(K * sizeof(float));
        for (size_t k = 0; k < K; k++) { wrow[k] = dequant_w(w_type, W, blk, inv_scale, (size_t)n * ldw + k); }
        for (size_t m = 0; m < M; m++)
        {
            double acc = 0.0;
            const uint16_t* x = X + m * ldx;
            for (size_t k = 0; k < K; k++) { acc += (double)wrow[k] * (double)oracle_bf16_to_float(x[k]); }
            const size_t yi = m * ldy_m + (size_t)n * ldy_n;
            float r = alpha * (float)acc;
            if (beta != 0.f) { r += beta * oracle_bf16_to_float(Y[yi]); }
            if (y32) { y32[m * N + (size_t)n] = r; }
            Y[yi] = oracle_float_to_bf16_rne(r);
        }
        free(wrow);
    }
}

/* ---- the reference's CPU path, as a timed baseline ------------------------------------ */

#if defined(__x86_64__) && defined(__GNUC__)
#define ORACLE_CLONES __attribute__((target_clones("default", "avx2", "avx512f")))
#else
#define ORACLE_CLONES
#endif

ORACLE_CLONES
static float dot_f32(const float* a, const float* b, size_t n)
{
    float acc[16] = { 0 };
    size_t i = 0;
    for (; i + 16 <= n; i += 16)
    {
        for (int j = 0; j < 16; j++) { acc[j] += a[i + j] * b[i + j]; }
    }
    float s = 0.f;
    for (int j = 0; j < 16; j++) { s += acc[j]; }
    for (; i < n; i++) { s += a[i] * b[i]; }
    return s;
}

/* "Dequantise to float, then sgemm": the CPU form of the path, assembled from the
 * reference's two CPU primitives - per-element decode (cccc/types.h:139-166, :72-90,
 * :257-261; cccc/MatrixData.h:61-77) into a float buffer times the dequant multiplier, then
 * the column-major sgemm of cccc/cblas_real.h:332-335 as called from cccc/Matrix.cpp:1155
 * (C[N,M] = W^T[N,K] * X[K,M]).  Float weights (no BF16 rounding), float activations,
 * float output.  wf is caller-provided scratch of N*K floats.  Returns the dequant time
 * fraction through *t_dequant (seconds) and the GEMM time through *t_gemm. */
ORACLE_API void oracle_cpu_path_dequant_sgemm(int w_type, const uint8_t* W, const uint8_t* blk, float inv_scale,
    const float* Xf, float* Yf, float* wf, size_t N, size_t M, size_t K, double* t_dequant, double* t_gemm)
{
    double t0 = 0, t1 = 0, t2 = 0;
#if defined(_OPENMP)
    t0 = omp_get_wtime();
#endif
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < (long long)N; n++)
    {
        for (size_t k = 0; k < K; k++)
        {
            const size_t idx = (size_t)n * K + k;
            float v;
            if (w_type == 6)
            {
                const uint8_t nib = (idx & 1) ? (W[idx >> 1] >> 4) : (W[idx >> 1] & 0xF);
                v = k_fp4_table[nib] * (blk ? oracle_e4m3_to_float(blk[idx / 16]) : inv_scale);
            }
            else
            {
                v = ((w_type == 5) ? oracle_e5m2_to_float(W[idx]) : oracle_e4m3_to_float(W[idx])) * inv_scale;
            }
            wf[idx] = v;
        }
    }
#if defined(_OPENMP)
    t1 = omp_get_wtime();
#endif
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < (long long)N; n++)
    {
        for (size_t m = 0; m < M; m++) { Yf[m * N + (size_t)n] = dot_f32(wf + (size_t)n * K, Xf + m * K, K); }
    }
#if defined(_OPENMP)
    t2 = omp_get_wtime();
#endif
    if (t_dequant) { *t_dequant = t1 - t0; }
    if (t_gemm) { *t_gemm = t2 - t1; }
}

ORACLE_API int oracle_num_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
