// Host side of the prefill path: which tile shape and which kernel (one CTA per tile, or a CTA pair)
// a shape gets, and the launch.
#pragma once

#include "gemm_prefill.cuh"
#include "gemm_prefill_pair.cuh"

#include <cstdlib>

namespace b200
{

// 256-token tiles halve the weight conversions per flop; 128-token tiles are taken when the larger
// tile would leave more than half of the 2-per-SM CTA slots empty (few output features, few tokens).
static int pf_pick_bn(unsigned int N, unsigned int M, unsigned int K, int sm_count)
{
    const unsigned long long ftiles = (N + PF_BM - 1) / PF_BM;
    const unsigned long long tiles256 = (unsigned long long)((M + 255) / 256) * ftiles;
    const unsigned long long tiles512 = (unsigned long long)((M + 511) / 512) * ftiles;
    if (M <= 128 || tiles256 * 2 <= (unsigned long long)sm_count) { return 128; }
    // 256 features x 256 tokens per CTA (one CTA per SM, the activation tile shared by two weight
    // tiles) when that still fills most of the SMs; -256 encodes it
    (void)tiles512;
    const unsigned long long tiles_wide = (unsigned long long)((M + 255) / 256) * ((N + 2 * PF_BM - 1) / (2 * PF_BM));
    // Measured at M=2048: K=12288 1107 vs 1066 TFLOP/s for it, K=4096 861 vs 964 against it (its
    // prologue and epilogue are not hidden by a second CTA), so it is taken for long K only.
    if (K >= 8192 && tiles_wide * 10 >= (unsigned long long)sm_count * 8) { return -256; }
    return 256;
}

template <int WT, bool SCALED>
static int launch_prefill_t(const void* X, unsigned int ldx, const PrefillParams& pp_in, int device, int sm_count, cudaStream_t stream)
{
    int bn = pf_pick_bn(pp_in.N, pp_in.M, pp_in.K, sm_count);
    CUtensorMap tmX, tmY;
    memset(&tmY, 0, sizeof(tmY));
    PrefillParams pp = pp_in;
    // BF16 output with contiguous features, no accumulate: the epilogue writes whole tiles with TMA stores
    pp.y_tma = 0;
    if (!pp.out_f32 && pp.beta == 0.f && pp.ldy_n == 1 && (pp.ldy_m % 8) == 0 && pp.ldy_m >= (long long)pp.N
        && (reinterpret_cast<uintptr_t>(pp.Y) & 15u) == 0 && !(getenv("B200_PF_NOTMAY")))
    {
        const char* f0 = getenv("B200_PF_MODE");
        const int m0 = f0 ? atoi(f0) : 0;
        const unsigned box_rows = (m0 == 2 || m0 == 3) ? (unsigned)PP_TOKENS : (unsigned)(bn == 128 ? 128 : 256);
        if (make_map_2d(&tmY, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pp.Y, pp.N, pp.M, (unsigned long long)pp.ldy_m * 2, PF_BM, box_rows,
                false))
        {
            pp.y_tma = 1;
        }
    }
    const char* force = getenv("B200_PF_MODE");    // development switch
    const int mode = force ? atoi(force) : 0;
    if (mode == 2 || mode == 3)
    {
        if (!make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, pp.K, pp.M, (unsigned long long)ldx * 2, PF_BK, PP_HALF, true))
        {
            return -2;
        }
        return mode == 2 ? launch_prefill_pair<WT, SCALED, 1>(tmX, tmY, pp, device, stream)
                         : launch_prefill_pair<WT, SCALED, 2>(tmX, tmY, pp, device, stream);
    }
    if (mode == 1 && bn == -256) { bn = 256; }
    if (!make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, pp.K, pp.M, (unsigned long long)ldx * 2, PF_BK,
            (unsigned)(bn == 128 ? 128 : 256), true))
    {
        return -2;
    }
    if (bn == -256) { return launch_prefill_bn<WT, SCALED, 256, 2>(tmX, tmY, pp, device, stream); }
    return bn == 128 ? launch_prefill_bn<WT, SCALED, 128, 1>(tmX, tmY, pp, device, stream)
                     : launch_prefill_bn<WT, SCALED, 256, 1>(tmX, tmY, pp, device, stream);
}

// Returns -2 when the shape has to go elsewhere.
static int launch_prefill(int w_type, const GemvParams& p, int device, int sm_count, cudaStream_t stream)
{
    if (w_type == DT_FP4 && p.blk == nullptr) { return -2; }
    PrefillParams pp;
    memset(&pp, 0, sizeof(pp));
    pp.W = p.W;
    pp.blk = p.blk;
    pp.Y = p.Y;
    pp.status = p.status;
    pp.N = p.N;
    pp.M = p.M;
    pp.K = p.K;
    pp.ldw = p.ldw;
    pp.ldy_m = p.ldy_m;
    pp.ldy_n = p.ldy_n;
    pp.w_scale = p.w_scale;
    pp.alpha = p.alpha;
    pp.beta = p.beta;
    pp.post_scale = 1.0f;
    pp.out_f32 = p.out_f32;
    { const char* d = getenv("B200_PF_DBG"); pp.dbg = d ? (unsigned)atoi(d) : 0u; }
    if (w_type == DT_FP4) { return launch_prefill_t<DT_FP4, false>(p.X, p.ldx, pp, device, sm_count, stream); }
    int e = 0;
    const bool pow2 = p.w_scale > 0.f && !std::isinf(p.w_scale) && std::frexp(p.w_scale, &e) == 0.5f && e >= -39 && e <= 41;
    if (pow2)
    {
        pp.post_scale = p.w_scale;
        pp.w_scale = 1.0f;
        return w_type == DT_E5M2 ? launch_prefill_t<DT_E5M2, false>(p.X, p.ldx, pp, device, sm_count, stream)
                                 : launch_prefill_t<DT_E4M3, false>(p.X, p.ldx, pp, device, sm_count, stream);
    }
    return w_type == DT_E5M2 ? launch_prefill_t<DT_E5M2, true>(p.X, p.ldx, pp, device, sm_count, stream)
                             : launch_prefill_t<DT_E4M3, true>(p.X, p.ldx, pp, device, sm_count, stream);
}

}    // namespace b200
