// Host side of the prefill path: which tile shape and which kernel (one CTA per tile, or a CTA pair)
// a shape gets, and the launch.
#pragma once

#include "gemm_prefill.cuh"
#include "gemm_prefill_pair.cuh"


namespace b200
{


// Tile shapes of the prefill path.  One CTA per tile: 128 features x 128 or 256 tokens (two CTAs per
// SM), or 256 features x 256 tokens (one CTA per SM).  CTA pairs (cta_group::2): 256 x 256, 512
// features x 256 tokens, or 256 features x 512 tokens per pair.
enum PrefillVariant : int
{
    PFV_AUTO = 0,
    PFV_CTA_T128 = 1,
    PFV_CTA_T256 = 2,
    PFV_CTA_F256 = 3,
    PFV_PAIR = 4,
    PFV_PAIR_F512 = 5,
    PFV_PAIR_T512 = 6,
    PFV_COUNT = 7
};

// Measured on B200 (M = 64 ... 8192, N x K of 1024..12288 x 4096..12288, all three weight types): the
// pair tile of 512 tokens is the fastest shape whenever its pairs cover about two thirds of the SMs
// (each weight is converted once per 512 tokens, each CTA stages half of the activations, five and
// four stages deep); with fewer tiles the 256 x 256 pair tile (two CTAs per SM) wins, and when even
// that leaves most SMs idle the 128 x 128 one-CTA tile gives the most CTAs.  The k loop of a CTA
// costs about 0.55 us per 64-wide k block whatever the tile, so small problems are bound by K alone.
static int pf_pick_variant(int w_type, unsigned int N, unsigned int M, unsigned int K, int sm_count)
{
    (void)w_type;
    (void)K;
    const unsigned long long f256 = (N + 2 * PF_BM - 1) / (2 * PF_BM);
    const unsigned long long pairs_t512 = (unsigned long long)((M + 511) / 512) * f256;
    const unsigned long long pairs_256 = (unsigned long long)((M + 255) / 256) * f256;
    const unsigned long long want = (unsigned long long)sm_count / 3;    // pairs: two thirds of the SMs
    if (pairs_t512 >= want)
    {
        // Both pair tiles are possible: count waves.  One 256 x 512 tile occupies a pair of SMs for two
        // units of time; 256 x 256 tiles run two per SM pair, so a full wave of them also takes two
        // units and a last wave that fits one CTA per SM takes one.  The smaller tile converts each
        // weight twice as often and measured 8-12 % slower at equal occupancy, so it is only taken when
        // it saves a clear part of a wave (q+k+v at 2048 tokens: 96 large tiles on 74 SM pairs).
        const unsigned long long slots = (unsigned long long)sm_count / 2;    // SM pairs
        const double cost_t512 = 2.0 * (double)((pairs_t512 + slots - 1) / slots);
        const unsigned long long rem = pairs_256 % (2 * slots);
        const double cost_256 = (2.0 * (double)(pairs_256 / (2 * slots)) + (rem == 0 ? 0.0 : (rem <= slots ? 1.0 : 2.0))) / 0.88;
        return cost_256 < 0.9 * cost_t512 ? PFV_PAIR : PFV_PAIR_T512;
    }
    if (M > 128 && pairs_256 >= want) { return PFV_PAIR; }
    return PFV_CTA_T128;
}

// Features per blockIdx.y of a tile shape.
static unsigned int pf_variant_tile_features(int variant)
{
    switch (variant)
    {
    case PFV_CTA_F256: return 2 * PF_BM;
    case PFV_PAIR: return 2 * PF_BM;
    case PFV_PAIR_F512: return 4 * PF_BM;
    case PFV_PAIR_T512: return 2 * PF_BM;
    default: return PF_BM;
    }
}

template <int WT, bool SCALED>
static int launch_prefill_t(const void* X, unsigned int ldx, const PrefillParams& pp_in, int device, int sm_count, int variant,
    cudaStream_t stream)
{
    PrefillParams pp = pp_in;
    unsigned int n_total = 0;
    for (unsigned int j = 0; j < pp.n_seg; j++) { n_total += pp.seg[j].N; }
    if (variant <= PFV_AUTO || variant >= PFV_COUNT) { variant = pf_pick_variant(WT, n_total, pp.M, pp.K, sm_count); }
    const bool pair = variant >= PFV_PAIR;
    const unsigned x_box_rows = pair ? (unsigned)PP_HALF : (variant == PFV_CTA_T128 ? 128u : 256u);
    const unsigned y_box_rows = pair ? (unsigned)PP_TOKENS : x_box_rows;
    const unsigned int tile_features = pf_variant_tile_features(variant);
    CUtensorMap tmX;
    PrefillYMaps tmY;
    memset(&tmY, 0, sizeof(tmY));
    unsigned int feature_tiles = 0;
    for (unsigned int j = 0; j < pp.n_seg; j++)
    {
        PrefillSeg& g = pp.seg[j];
        g.tile0 = feature_tiles;
        feature_tiles += (g.N + tile_features - 1) / tile_features;
        // BF16 output with contiguous features and no accumulate: the epilogue writes whole tiles with TMA stores
        g.y_tma = 0;
        if (pp.out_f32 != 1u && g.beta == 0.f && g.ldy_n == 1 && (g.ldy_m % 8) == 0 && g.ldy_m >= (long long)g.N
            && (reinterpret_cast<uintptr_t>(g.Y) & 15u) == 0
            && make_map_2d(&tmY.m[j], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.Y, g.N, pp.M, (unsigned long long)g.ldy_m * 2, PF_BM, y_box_rows,
                false))
        {
            g.y_tma = 1;
        }
    }
    if (feature_tiles == 0 || feature_tiles > 65535u) { return -2; }    // grid.y
    if (!make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, pp.K, pp.M, (unsigned long long)ldx * 2, PF_BK, x_box_rows, true))
    {
        return -2;
    }
    switch (variant)
    {
    case PFV_CTA_T128: return launch_prefill_bn<WT, SCALED, 128, 1>(tmX, tmY, pp, feature_tiles, device, stream);
    case PFV_CTA_F256: return launch_prefill_bn<WT, SCALED, 256, 2>(tmX, tmY, pp, feature_tiles, device, stream);
    case PFV_PAIR: return launch_prefill_pair<WT, SCALED, 1, 1, 16>(tmX, tmY, pp, feature_tiles, device, stream);
    case PFV_PAIR_F512: return launch_prefill_pair<WT, SCALED, 2, 1, 16>(tmX, tmY, pp, feature_tiles, device, stream);
    case PFV_PAIR_T512: return launch_prefill_pair<WT, SCALED, 1, 2, 16>(tmX, tmY, pp, feature_tiles, device, stream);
    default: return launch_prefill_bn<WT, SCALED, 256, 1>(tmX, tmY, pp, feature_tiles, device, stream);
    }
}

static bool pf_is_pow2_scale(float s)
{
    int e = 0;
    return s > 0.f && !std::isinf(s) && std::frexp(s, &e) == 0.5f && e >= -39 && e <= 41;
}

// One launch for up to PF_MAX_GROUP linears that share X (count = 1: a single linear).  `items`
// carry W, blk, Y, N, ldw, ldy_m, ldy_n, w_scale, alpha, beta; the rest comes from items[0].
// Returns -2 when the shapes have to go elsewhere.
static int launch_prefill(int w_type, const GemvParams* items, unsigned int count, int device, int sm_count, int variant,
    cudaStream_t stream)
{
    if (count == 0 || count > (unsigned)PF_MAX_GROUP) { return -2; }
    PrefillParams pp;
    memset(&pp, 0, sizeof(pp));
    pp.n_seg = count;
    pp.status = items[0].status;
    pp.M = items[0].M;
    pp.K = items[0].K;
    pp.out_f32 = items[0].out_f32;
    bool all_pow2 = true;
    for (unsigned int j = 0; j < count; j++)
    {
        if (w_type == DT_FP4 && items[j].blk == nullptr) { return -2; }
        all_pow2 = all_pow2 && pf_is_pow2_scale(items[j].w_scale);
    }
    // a power-of-two scale commutes exactly with the BF16 rounding and the FP32 sums: it moves to the epilogue
    const bool scaled = w_type != DT_FP4 && !all_pow2;
    for (unsigned int j = 0; j < count; j++)
    {
        PrefillSeg& g = pp.seg[j];
        g.W = items[j].W;
        g.blk = items[j].blk;
        g.Y = items[j].Y;
        g.N = items[j].N;
        g.ldw = items[j].ldw;
        g.ldy_m = items[j].ldy_m;
        g.ldy_n = items[j].ldy_n;
        g.alpha = items[j].alpha;
        g.beta = items[j].beta;
        g.w_scale = scaled ? items[j].w_scale : 1.0f;
        g.post_scale = (w_type == DT_FP4 || scaled) ? 1.0f : items[j].w_scale;
    }
    const void* X = items[0].X;
    const unsigned int ldx = items[0].ldx;
    if (w_type == DT_FP4) { return launch_prefill_t<DT_FP4, false>(X, ldx, pp, device, sm_count, variant, stream); }
    if (!scaled)
    {
        return w_type == DT_E5M2 ? launch_prefill_t<DT_E5M2, false>(X, ldx, pp, device, sm_count, variant, stream)
                                 : launch_prefill_t<DT_E4M3, false>(X, ldx, pp, device, sm_count, variant, stream);
    }
    return w_type == DT_E5M2 ? launch_prefill_t<DT_E5M2, true>(X, ldx, pp, device, sm_count, variant, stream)
                             : launch_prefill_t<DT_E4M3, true>(X, ldx, pp, device, sm_count, variant, stream);
}

}    // namespace b200
