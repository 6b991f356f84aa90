// Shared device helpers: the scalar codecs of the path (bit-exact with the reference's
// device functions) and the host-side error/launch bookkeeping.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

namespace b200
{

// cccc::DataType (cccc/types.h:24-34)
enum : int
{
    DT_FLOAT = 0,
    DT_DOUBLE = 1,
    DT_HALF = 2,
    DT_BF16 = 3,
    DT_E4M3 = 4,
    DT_E5M2 = 5,
    DT_FP4 = 6
};

// ---- host bookkeeping (defined in api.cu) ---------------------------------------------------
void count_launch();
// Device sync + error report in the reference's format (cuda_functions.cu:26-40).
int sync_and_report(const char* label);
// Launch-only check (no sync) for the asynchronous entry points.
int report_launch(const char* label);
// The current device's status word (allocating the workspace if need be); nullptr on failure.
unsigned int* cuda_b200_status_word();

// ---- scalar codecs ----------------------------------------------------------------------------

// E4M3 byte -> float (cuda_functions.cu:2366-2381): bias 7, 0x7F/0xFF NaN, subnormal m*2^-9.
__device__ __forceinline__ float e4m3_to_float(uint32_t b)
{
    const uint32_t s = (b >> 7) & 1u;
    const uint32_t e = (b >> 3) & 0xFu;
    const uint32_t m = b & 7u;
    if (e == 15u && m == 7u) { return __uint_as_float(0x7FC00000u); }
    if (e == 0u) { return (s ? -1.f : 1.f) * (float)m * (1.f / 512.f); }
    return __uint_as_float((s << 31) | ((e + 120u) << 23) | (m << 20));
}

// E5M2 byte -> float (cuda_functions.cu:2674-2693): bias 15, e==31 Inf/NaN, subnormal m*2^-16.
__device__ __forceinline__ float e5m2_to_float(uint32_t b)
{
    const uint32_t s = (b >> 7) & 1u;
    const uint32_t e = (b >> 2) & 0x1Fu;
    const uint32_t m = b & 3u;
    if (e == 31u) { return m == 0u ? __uint_as_float((s << 31) | 0x7F800000u) : __uint_as_float(0x7FC00000u); }
    if (e == 0u) { return (s ? -1.f : 1.f) * (float)m * (1.f / 65536.f); }
    return __uint_as_float((s << 31) | ((e + 112u) << 23) | (m << 21));
}

// float*scale -> E4M3, truncating, saturating to 0x7E (cuda_functions.cu:2382-2415), without branches: from 2^-6 up the
// code is the float's exponent and top three mantissa bits rebased ((bits >> 20) - 120 * 8, the magnitude clamped to 448
// first, which also maps 448..inf to 0x7E); below, the subnormal code is the magnitude in units of 2^-9, truncated.
__device__ __forceinline__ uint8_t float_to_e4m3(float f, float scale)
{
    f *= scale;
    const uint32_t u = __float_as_uint(f);
    const uint32_t a = u & 0x7FFFFFFFu;
    const uint32_t normal = (min(a, 0x43E00000u) >> 20) - 960u;
    const uint32_t subnormal = (uint32_t)__float2int_rz(__uint_as_float(a) * 512.0f);
    const uint32_t code = (a >= 0x3C800000u ? normal : subnormal) | ((u >> 24) & 0x80u);
    return (uint8_t)(a > 0x7F800000u ? 0x7Fu : code);
}

// float*scale -> E5M2, truncating, saturating to 0x7B (cuda_functions.cu:2694-2725).
__device__ __forceinline__ uint8_t float_to_e5m2(float f, float scale)
{
    f *= scale;
    const uint32_t u = __float_as_uint(f);
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
    return (uint8_t)((s << 7) | ((uint32_t)(e8 & 0x1F) << 2) | (fm >> 21));
}

// E2M1 nibble -> float (table of cuda_functions.cu:2791-2794), computed from the bits:
// magnitude code c: 0 -> 0, 1 -> 0.5, else 2^((c>>1)-1) * (1 + (c&1)/2).  Code 8 ("-0") is
// +0 in the reference's table, so the sign is only applied to non-zero magnitudes.
__device__ __forceinline__ float fp4_to_float(uint32_t nib)
{
    const uint32_t c = nib & 7u;
    if (c == 0u) { return 0.f; }
    const uint32_t bits = (c == 1u) ? 0x3F000000u : (((c >> 1) + 126u) << 23) | ((c & 1u) << 22);
    return __uint_as_float(bits | ((nib & 8u) << 28));
}

// float -> E2M1 nibble by "<" thresholds (cuda_functions.cu:2796-2832).
__device__ __forceinline__ uint32_t float_to_fp4(float f)
{
    const uint32_t s = (f < 0.f) ? 8u : 0u;
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

// float -> BF16 bits by the reference's integer round-to-nearest-even
// (cuda_functions.cu:2761-2764); the add wraps exactly as the reference's does.
__device__ __forceinline__ uint16_t float_to_bf16_bits_ref(float f)
{
    uint32_t u = __float_as_uint(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t h) { return __uint_as_float(h << 16); }

// The dequantised BF16 weight of the path, as a float, for one element (used by the plain
// kernel and the standalone conversions).
template <int WT>
__device__ __forceinline__ float decode_fp8(uint32_t b)
{
    return WT == DT_E5M2 ? e5m2_to_float(b) : e4m3_to_float(b);
}

}    // namespace b200
