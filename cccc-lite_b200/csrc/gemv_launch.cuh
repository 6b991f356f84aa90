// Host-side launch logic of the quantized-weight linear: kernel choice, tensor maps, schedule.
// Shared by every translation unit that launches these kernels; what differs between them is
// only where the scratch memory (FP32 partial tiles, arrival counters, status word) lives.
#pragma once

#include "common.cuh"
#include "gemv_decode.cuh"
#include "tensor_map.cuh"
#include "prefill_launch.cuh"
#include "gemm_stream.cuh"
#include "gemm_native.cuh"
#include "gemm_native_fp4.cuh"

#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace b200
{

constexpr int kMaxDevices = 64;

// Where a launch finds its scratch memory, and the device facts the launch logic needs.
struct GemvScratch
{
    float* partials = nullptr;           // FP32 partial tiles of the split-k schedule
    size_t partial_bytes = 0;
    unsigned int* counters = nullptr;    // arrival counters, zero between launches
    unsigned int n_counters = 0;
    unsigned int* status = nullptr;      // error word, 0 = clean
    int device = 0;
    int sm_count = 0;
    int max_smem = 0;       // largest dynamic shared memory one CTA may ask for
    int smem_per_sm = 0;    // shared memory of one SM
};

// ---- launch helpers ---------------------------------------------------------------------------------
static bool is_pow2_scale(float s)
{
    if (!(s > 0.f) || std::isinf(s)) { return false; }
    int e = 0;
    const float m = std::frexp(s, &e);
    return m == 0.5f && e >= -39 && e <= 41;    // 2^-40 .. 2^40
}


template <class Cfg, bool SCALED>
static int launch_gemv_cfg(GemvParams p, const GemvScratch* ws, cudaStream_t stream, bool pdl)
{
    constexpr int WT = Cfg::WT;
    // two CTAs per SM share the SM's shared memory (each also reserves 1 KB for the system)
    const int budget = (Cfg::OCC == 2) ? (ws->smem_per_sm / 2 - 1024) : ws->max_smem;
    int ns = (budget - Cfg::HEADER_BYTES - Cfg::RED_BYTES) / Cfg::STAGE_BYTES;
    if (ns > Cfg::kMaxStages) { ns = Cfg::kMaxStages; }
    if (ns < 2) { return -2; }
    if (p.n_seg == 0)
    {
        // a single linear: describe it as a group of one
        p.n_seg = 1;
        p.seg[0].W = p.W;
        p.seg[0].blk = p.blk;
        p.seg[0].Y = p.Y;
        p.seg[0].N = p.N;
        p.seg[0].ldw = p.ldw;
        p.seg[0].ldy_m = p.ldy_m;
        p.seg[0].ldy_n = p.ldy_n;
        p.seg[0].w_scale = p.w_scale;
        p.seg[0].alpha = p.alpha;
        p.seg[0].beta = p.beta;
        p.seg[0].post_scale = p.post_scale;
    }
    p.n_row_blocks = 0;
    for (int j = 0; j < kMaxGroup; j++)
    {
        if ((unsigned)j < p.n_seg)
        {
            p.seg[j].rb_begin = p.n_row_blocks;
            p.n_row_blocks += (p.seg[j].N + Cfg::R - 1) / Cfg::R;
        }
        else { p.seg[j].rb_begin = 0xFFFFFFFFu; }
    }
    p.n_kstages = (p.K + Cfg::SKE - 1) / Cfg::SKE;
    const unsigned long long total = (unsigned long long)p.n_row_blocks * p.n_kstages;
    if (total == 0 || total > 0x7FFFFFFFull) { return -2; }
    p.total_items = (unsigned int)total;
    p.n_stages = (unsigned int)ns;
    // With at least one row block per SM, whole row blocks are dealt out: no CTA shares a row block,
    // so nothing is exchanged between CTAs.  With fewer, the k range is split as well (stream-K).
    // Measured on B200: the exchange costs about 5 us of serial latency, one SM alone streams about
    // 45 GB/s; so the k range is only split when whole row blocks would leave most SMs idle for long.
    bool whole_blocks = true;
    {
        const double block_bytes = (double)Cfg::R * (double)((WT == DT_FP4) ? p.K / 2 + p.K / 16 : p.K);
        const double sms = (double)ws->sm_count;
        const double rounds = (double)((p.n_row_blocks + ws->sm_count - 1) / ws->sm_count);
        const double t_whole = rounds * block_bytes / 45e9;
        const double t_split = 5e-6 + (double)p.n_row_blocks * block_bytes / (sms * 40e9);
        whole_blocks = t_whole <= t_split || Cfg::MT > 1;    // large partial tiles make the exchange far dearer
    }
    p.gran = whole_blocks ? p.n_kstages : 1u;
    const unsigned long long groups = total / p.gran;
    const unsigned int grid = (unsigned int)(groups < (unsigned long long)ws->sm_count ? groups : ws->sm_count);
    if ((size_t)grid * 2 * Cfg::R * 8 * Cfg::MT * sizeof(float) > ws->partial_bytes || grid > ws->n_counters) { return -2; }

    CUtensorMap tmW[kMaxGroup], tmS[kMaxGroup], tmX;
    const unsigned long long kbytes = (WT == DT_FP4) ? p.K / 2 : p.K;
    bool ok = true;
    for (int j = 0; j < kMaxGroup; j++)
    {
        if ((unsigned)j >= p.n_seg)
        {
            tmW[j] = tmW[0];
            tmS[j] = tmS[0];
            continue;
        }
        const GemvSeg& g = p.seg[j];
        const unsigned long long ldw_bytes = (WT == DT_FP4) ? g.ldw / 2 : g.ldw;
        ok = ok && make_map(&tmW[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.W, 64, g.N, kbytes / 64, ldw_bytes, Cfg::R, Cfg::SKS, false);
        if (ok && WT == DT_FP4)
        {
            ok = make_map(&tmS[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.blk, 16, g.N, p.K / 256, g.ldw / 16, Cfg::R, Cfg::SKS / 2, false);
        }
        else { tmS[j] = tmW[j]; }
    }
    ok = ok && make_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.X, 64, p.M, p.K / 64, (unsigned long long)p.ldx * 2, Cfg::XB,
                   Cfg::XSLABS, Cfg::XSWZ);
    if (!ok)
    {
        static std::atomic<bool> told{ false };
        if (!told.exchange(true))
        {
            fprintf(stderr, "gemm_wq_bf16: tensor map encoding failed; using the plain kernel\n");
        }
        return -2;
    }

    const size_t smem = (size_t)Cfg::HEADER_BYTES + (size_t)ns * Cfg::STAGE_BYTES + Cfg::RED_BYTES;
    auto kernel = gemv_wq_kernel<Cfg, SCALED>;
    static std::atomic<bool> attr_set[kMaxDevices];    // per instantiation, per device (zero-initialised)
    if (!attr_set[ws->device].load(std::memory_order_acquire))
    {
        // setting the same attribute twice from two threads is harmless; the flag only saves the call
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16");
            return 1;
        }
        attr_set[ws->device].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, kernel, tmW[0], tmS[0], tmW[1], tmS[1], tmW[2], tmS[2], tmX, p) != cudaSuccess)
    {
        report_launch("gemm_wq_bf16");
        return 1;
    }
    return 0;
}

template <int WT, bool SCALED>
static int launch_gemv(const GemvParams& p, const GemvScratch* ws, cudaStream_t stream, bool pdl)
{
    // More tokens: more rows per CTA, so that the activation slice (re-read from L2 by every CTA) stays
    // at or below the weight bytes it is multiplied with.
    //                                              WT MT RT WR WK SKS XB OCC
    if (p.M <= 2) { return launch_gemv_cfg<GemvCfg<WT, 1, 2, 1, 8, 32, 2, 1>, SCALED>(p, ws, stream, pdl); }
    if (p.M <= 8) { return launch_gemv_cfg<GemvCfg<WT, 1, 2, 1, 8, 16, 8, 1>, SCALED>(p, ws, stream, pdl); }
    // (FP4 stages hold twice the elements per weight byte, so twice the activations: half the k steps)
    constexpr int S16 = (WT == DT_FP4) ? 8 : 16, S32 = (WT == DT_FP4) ? 4 : 8;
    if (p.M <= 16) { return launch_gemv_cfg<GemvCfg<WT, 2, 4, 1, 8, S16, 16, 1>, SCALED>(p, ws, stream, pdl); }
    return launch_gemv_cfg<GemvCfg<WT, 4, 2, 2, 4, S32, 32, 1>, SCALED>(p, ws, stream, pdl);
}

template <int WT>
static int launch_plain(const GemvParams& p, cudaStream_t stream)
{
    const unsigned int grid = (p.N + 7) / 8;
    linear_wq_plain_kernel<WT><<<grid, 256, 0, stream>>>(p);
    count_launch();
    return report_launch("gemm_wq_bf16");
}

enum
{
    PLAN_PLAIN = 0,
    PLAN_DECODE = 1,
    PLAN_PREFILL = 2,
    PLAN_STREAM = 3,
    PLAN_NATIVE = 4
};

// flags bits 8-10 == 7: take the streaming tensor-core kernel whenever it accepts the shape (tests, tuning)
constexpr unsigned int kVariantStream = 7u;
// flags bit 11: never take the streaming kernel (the decode kernel up to 32 tokens, the prefill kernel above)
constexpr unsigned int kFlagNoStream = 0x800u;

// flags bit 12: take the native-operand tensor-core kernel (FP8 weights straight into the UMMA) whenever it accepts
// the shape; bit 13: never take it
constexpr unsigned int kFlagNative = 0x1000u;
constexpr unsigned int kFlagNoNative = 0x2000u;
// flags bit 14: the native-operand FP8 kernel splits the activations itself (up to 8 tokens) instead of a kernel of its
// own doing it: the shortest path from activations to outputs for one linear alone
constexpr unsigned int kFlagNativeFused = 0x4000u;

static inline bool al16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

// Where the native-operand kernels are the default.  Measured on B200 against the kernels that dequantise in registers
// (one linear in a CUDA graph of distinct weight copies, PDL):
//   * streaming, they reach 0.93-0.86 (FP8, 1-32 tokens, 151936 x 4096) and 0.81-0.84 (FP4, 128256 x 4096) of the
//     measured copy bandwidth, where the decode / streaming kernels reach 0.90 / 0.78 / 0.69 (FP8 at 1 / 4 / 32) and
//     0.45 (FP4: the dequantising arithmetic is the bound);
//   * one launch costs them more besides streaming (the activations' split, and the exchange of partial tiles when a
//     128-feature tile has to be cut across CTAs): 4096 x 4096 FP8 at one token 8.0 us against 5.4 us;
//   * no tile is cut when the launch has between one and two feature tiles per SM (every CTA takes one whole tile):
//     24576 x 4096 FP8 at 1 / 4 / 16 / 32 tokens 20.8 / 20.9 / 22.0 / 25.5 us against 22.1 / 24.5 / 26.1 / 28.3 us,
//     28672 x 4096 FP4 at 1 / 8 tokens 16.9 / 17.9 us against 26.8 / 28.5 us.
// Hence: launches of whole tiles (gate+up as a group) and lm_head-sized ones; FP4 always, FP8 from 3 tokens (at 1-2 the
// decode kernel is as fast on lm_head, and inside a whole decode step the two launches of the native form cost a
// batch-1 step 50 us where the chain of linears alone gains 12 us).
constexpr unsigned long long kNativeFp8MinBytes = 256ull << 20, kNativeFp4MinBytes = 48ull << 20;
constexpr unsigned int kNativeFp8MinTokens = 3;

static inline bool native_by_default(int w_type, unsigned int M, unsigned long long weight_elems, unsigned int feature_tiles, int sm_count)
{
    if (M > (unsigned int)(w_type == DT_FP4 ? NF_MAX_TOKENS : NK_MAX_TOKENS)) { return false; }
    if (w_type != DT_FP4 && M < kNativeFp8MinTokens) { return false; }
    const bool wide_fp4 = w_type == DT_FP4 && M > (unsigned int)NF_NARROW_TOKENS;    // one CTA per SM
    if (!wide_fp4 && feature_tiles > (unsigned int)sm_count && feature_tiles <= 2u * (unsigned int)sm_count) { return true; }
    return w_type == DT_FP4 ? weight_elems / 2 >= kNativeFp4MinBytes : weight_elems >= kNativeFp8MinBytes;
}

static inline bool want_native(unsigned int flags, int w_type, unsigned int M, unsigned long long weight_elems, unsigned int feature_tiles,
    int sm_count)
{
    if ((flags & kFlagNoNative) != 0 || M > (unsigned int)(w_type == DT_FP4 ? NF_MAX_TOKENS : NK_MAX_TOKENS)) { return false; }
    const unsigned int variant = (flags >> 8) & 7u;
    if (variant != 0 || (flags & kFlagNoStream) != 0) { return false; }    // a particular older kernel was asked for
    return (flags & kFlagNative) != 0 || native_by_default(w_type, M, weight_elems, feature_tiles, sm_count);
}

static int plan_base(int w_type, const void* W, const void* blk, const void* X, unsigned int N, unsigned int M, unsigned int K, unsigned int ldw,
    unsigned int ldx, unsigned int ldy_m, unsigned int ldy_n)
{
    if (N == 0 || M == 0 || K == 0) { return PLAN_PLAIN; }
    if (!al16(W) || !al16(X) || (ldx % 8) != 0) { return PLAN_PLAIN; }
    if (M > 32)
    {
        if (w_type == DT_FP4 && !blk) { return PLAN_PLAIN; }
        return prefill_supported(w_type, N, M, K, ldw, ldx, ldy_m, ldy_n) ? PLAN_PREFILL : PLAN_PLAIN;
    }
    if (w_type == DT_FP4)
    {
        if (!blk || !al16(blk) || (K % 256) != 0 || (ldw % 256) != 0) { return PLAN_PLAIN; }
    }
    else
    {
        if ((K % 64) != 0 || (ldw % 16) != 0) { return PLAN_PLAIN; }
    }
    return PLAN_DECODE;
}

// Measured on B200 (4096 x 4096, 12288 x 4096, 4096 x 12288; FP8 and FP4): up to 8 tokens the decode kernel's
// dot products keep up with the weight stream and its persistent CTAs waste nothing between tiles; from 9
// tokens on the streaming tensor-core kernel is faster (1.1x at 16 tokens, 1.4-2x at 32, 2-7x at 64-128, where
// the alternative is the prefill kernel's compute-shaped tiles).
constexpr unsigned int kStreamMinTokens = 9, kStreamMaxTokens = 128;

static int plan_for(int w_type, const void* W, const void* blk, const void* X, const void* Y, unsigned int N, unsigned int M,
    unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m, unsigned int ldy_n)
{
    (void)Y;
    const int base = plan_base(w_type, W, blk, X, N, M, K, ldw, ldx, ldy_m, ldy_n);
    if (base != PLAN_PLAIN && M >= kStreamMinTokens && M <= kStreamMaxTokens && stream_supported(w_type, blk, N, M, K, ldw, ldx))
    {
        return PLAN_STREAM;
    }
    return base;
}


// The whole entry: argument checks done by the caller; picks the kernel and launches it on
// `st`.  Returns the C-ABI code (0 ok, 1 CUDA error, -1 bad argument).
static int run_linear_wq(const GemvScratch* ws, int w_type, const void* W, const void* blk_scales, float inv_scale, const void* X,
    void* Y, unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m,
    unsigned int ldy_n, float alpha, float beta, cudaStream_t st, unsigned int flags, bool decode_only = false,
    const GemvAllReduce* ar = nullptr)
{
    GemvParams p;
    memset(&p, 0, sizeof(p));
    if (ar != nullptr && ar->world > 1)
    {
        // the exchange lives in the decode kernel's epilogue: nothing else takes it
        if (beta != 0.f || N_out > 16u * (unsigned)kArMaxRowBlocks || (unsigned long long)M_tokens * N_out > ar->n_max) { return -1; }
        p.ar = *ar;
        decode_only = true;
    }
    p.W = (const uint8_t*)W;
    p.blk = (w_type == DT_FP4) ? (const uint8_t*)blk_scales : nullptr;
    p.X = (const uint16_t*)X;
    p.Y = (uint16_t*)Y;
    p.partials = ws->partials;
    p.counters = ws->counters;
    p.status = ws->status;
    p.N = N_out;
    p.M = M_tokens;
    p.K = K;
    p.ldw = ldw;
    p.ldx = ldx;
    p.ldy_m = ldy_m;
    p.ldy_n = ldy_n;
    p.w_scale = inv_scale;
    p.alpha = alpha;
    p.beta = beta;
    p.post_scale = 1.0f;
    p.out_f32 = (flags & 4u) ? 1u : ((flags & 8u) ? 2u : 0u);
    const bool pdl = (flags & 1u) != 0;

    if (!decode_only && want_native(flags, w_type, M_tokens, (unsigned long long)N_out * K, (N_out + NK_BM - 1) / NK_BM, ws->sm_count))
    {
        const int r = w_type == DT_FP4
            ? launch_native_fp4(&p, 1, ws->partials, ws->partial_bytes, ws->counters, ws->n_counters, ws->device, ws->sm_count, st, pdl)
            : launch_native(w_type, &p, 1, ws->partials, ws->partial_bytes, ws->counters, ws->n_counters, ws->device, ws->sm_count, st, pdl,
                  (flags & kFlagNativeFused) == 0);
        if (r != -2) { return r; }
    }
    int plan = plan_for(w_type, W, blk_scales, X, Y, N_out, M_tokens, K, ldw, ldx, ldy_m, ldy_n);
    // the exchange lives in the decode kernel; flags bit 11 asks for the kernels that were there before the streaming one
    const unsigned int variant = (flags >> 8) & 7u;
    const bool no_stream = (flags & kFlagNoStream) != 0 || (variant >= 1 && variant <= 6);    // a prefill tile shape was asked for
    if (plan == PLAN_STREAM && (decode_only || no_stream)) { plan = M_tokens <= 32 ? PLAN_DECODE : PLAN_PREFILL; }
    if (decode_only && plan != PLAN_DECODE) { return -1; }
    if (!decode_only && (plan == PLAN_STREAM || (variant == kVariantStream && plan != PLAN_PLAIN)))
    {
        const int r = launch_stream(w_type, &p, 1, ws->device, ws->sm_count, st, pdl);
        if (r != -2) { return r; }
        if (plan == PLAN_STREAM) { plan = M_tokens <= 32 ? PLAN_DECODE : PLAN_PREFILL; }
    }
    if (plan == PLAN_DECODE)
    {
        int r;
        if (w_type == DT_FP4)
        {
            p.post_scale = 65536.0f;    // the FP4 dequantiser leaves 2^-16 in every weight
            r = launch_gemv<DT_FP4, false>(p, ws, st, pdl);
        }
        else if (is_pow2_scale(inv_scale))
        {
            // A power-of-two multiplier commutes exactly with the BF16 rounding and the FP32 sums.
            p.post_scale = inv_scale;
            p.w_scale = 1.0f;
            r = (w_type == DT_E5M2) ? launch_gemv<DT_E5M2, false>(p, ws, st, pdl) : launch_gemv<DT_E4M3, false>(p, ws, st, pdl);
        }
        else { r = (w_type == DT_E5M2) ? launch_gemv<DT_E5M2, true>(p, ws, st, pdl) : launch_gemv<DT_E4M3, true>(p, ws, st, pdl); }
        if (r != -2) { return r; }
        if (decode_only) { return -1; }
        p.post_scale = 1.0f;
        p.w_scale = inv_scale;
        plan = PLAN_PLAIN;
    }
    if (plan == PLAN_PREFILL)
    {
        const int r = launch_prefill(w_type, &p, 1, ws->device, ws->sm_count, (int)((flags >> 8) & 7u), st);
        if (r != -2) { return r; }
        plan = PLAN_PLAIN;
    }
    switch (w_type)
    {
    case DT_E4M3: return launch_plain<DT_E4M3>(p, st);
    case DT_E5M2: return launch_plain<DT_E5M2>(p, st);
    default: return launch_plain<DT_FP4>(p, st);
    }
}


// One linear of a group, as the C-ABI passes it (mirrors cuda_wq_linear of the public header).
struct GroupItem
{
    const void* W;
    const void* blk_scales;
    void* Y;
    float inv_scale, alpha, beta;
    unsigned int N_out, ldw, ldy_m, ldy_n;
};

// Several linears that read the same activations (q/k/v, gate/up) as ONE launch of the decode
// kernel: their row blocks are dealt out together.  Anything the decode kernel does not take
// (unaligned operands, more than kMaxGroup linears) runs one linear at a time; more than 32 tokens
// go to the tensor-core kernel, again as one launch when every member qualifies.
static int run_linear_wq_group(const GemvScratch* ws, int w_type, unsigned int count, const GroupItem* items, const void* X,
    unsigned int M_tokens, unsigned int K, unsigned int ldx, cudaStream_t st, unsigned int flags)
{
    unsigned long long group_elems = 0;
    unsigned int group_tiles = 0;
    for (unsigned int j = 0; j < count; j++)
    {
        group_elems += (unsigned long long)items[j].N_out * K;
        group_tiles += (items[j].N_out + NK_BM - 1) / NK_BM;
    }
    if (count >= 1 && count <= (unsigned)PF_MAX_GROUP && want_native(flags, w_type, M_tokens, group_elems, group_tiles, ws->sm_count))
    {
        GemvParams ps[PF_MAX_GROUP];
        memset(ps, 0, sizeof(ps));
        bool all = true;
        for (unsigned int j = 0; j < count; j++)
        {
            GemvParams& q = ps[j];
            q.W = (const uint8_t*)items[j].W;
            q.blk = (w_type == DT_FP4) ? (const uint8_t*)items[j].blk_scales : nullptr;
            q.X = (const uint16_t*)X;
            q.Y = (uint16_t*)items[j].Y;
            q.status = ws->status;
            q.N = items[j].N_out;
            q.M = M_tokens;
            q.K = K;
            q.ldw = items[j].ldw;
            q.ldx = ldx;
            q.ldy_m = items[j].ldy_m;
            q.ldy_n = items[j].ldy_n;
            q.w_scale = items[j].inv_scale;
            q.alpha = items[j].alpha;
            q.beta = items[j].beta;
            q.out_f32 = (flags & 4u) ? 1u : ((flags & 8u) ? 2u : 0u);
            all = all && items[j].N_out != 0;
        }
        if (all)
        {
            const bool pdl = (flags & 1u) != 0;
            const int r = w_type == DT_FP4
                ? launch_native_fp4(ps, count, ws->partials, ws->partial_bytes, ws->counters, ws->n_counters, ws->device, ws->sm_count, st, pdl)
                : launch_native(w_type, ps, count, ws->partials, ws->partial_bytes, ws->counters, ws->n_counters, ws->device, ws->sm_count, st, pdl,
                      (flags & kFlagNativeFused) == 0);
            if (r != -2) { return r; }
        }
    }
    // the streaming tensor-core kernel takes up to three members as one grid
    bool one_stream = count >= 1 && count <= (unsigned)PF_MAX_GROUP;
    bool want_stream = ((flags >> 8) & 7u) == kVariantStream;
    if ((flags & kFlagNoStream) != 0 || (((flags >> 8) & 7u) >= 1 && ((flags >> 8) & 7u) <= 6)) { one_stream = false; }
    for (unsigned int j = 0; j < count && one_stream; j++)
    {
        const int plan = items[j].N_out == 0 ? PLAN_PLAIN
                                             : plan_for(w_type, items[j].W, items[j].blk_scales, X, items[j].Y, items[j].N_out, M_tokens, K,
                                                   items[j].ldw, ldx, items[j].ldy_m, items[j].ldy_n);
        one_stream = plan != PLAN_PLAIN;
        want_stream = want_stream || plan == PLAN_STREAM;
    }
    if (one_stream && want_stream)
    {
        GemvParams ps[PF_MAX_GROUP];
        memset(ps, 0, sizeof(ps));
        for (unsigned int j = 0; j < count; j++)
        {
            GemvParams& q = ps[j];
            q.W = (const uint8_t*)items[j].W;
            q.blk = (w_type == DT_FP4) ? (const uint8_t*)items[j].blk_scales : nullptr;
            q.X = (const uint16_t*)X;
            q.Y = (uint16_t*)items[j].Y;
            q.status = ws->status;
            q.N = items[j].N_out;
            q.M = M_tokens;
            q.K = K;
            q.ldw = items[j].ldw;
            q.ldx = ldx;
            q.ldy_m = items[j].ldy_m;
            q.ldy_n = items[j].ldy_n;
            q.w_scale = items[j].inv_scale;
            q.alpha = items[j].alpha;
            q.beta = items[j].beta;
            q.out_f32 = (flags & 4u) ? 1u : ((flags & 8u) ? 2u : 0u);
        }
        const int r = launch_stream(w_type, ps, count, ws->device, ws->sm_count, st, (flags & 1u) != 0);
        if (r != -2) { return r; }
    }
    bool one_launch = count >= 1 && count <= (unsigned)kMaxGroup && M_tokens <= 32;
    for (unsigned int j = 0; j < count && one_launch; j++)
    {
        one_launch = items[j].N_out != 0
            && plan_for(w_type, items[j].W, items[j].blk_scales, X, items[j].Y, items[j].N_out, M_tokens, K, items[j].ldw, ldx,
                   items[j].ldy_m, items[j].ldy_n)
                != PLAN_PLAIN;
    }
    if (one_launch)
    {
        GemvParams p;
        memset(&p, 0, sizeof(p));
        p.X = (const uint16_t*)X;
        p.partials = ws->partials;
        p.counters = ws->counters;
        p.status = ws->status;
        p.M = M_tokens;
        p.K = K;
        p.ldx = ldx;
        p.out_f32 = (flags & 4u) ? 1u : ((flags & 8u) ? 2u : 0u);
        p.n_seg = count;
        bool all_pow2 = true;
        for (unsigned int j = 0; j < count; j++) { all_pow2 = all_pow2 && is_pow2_scale(items[j].inv_scale); }
        const bool scaled = w_type != DT_FP4 && !all_pow2;
        for (unsigned int j = 0; j < count; j++)
        {
            GemvSeg& g = p.seg[j];
            g.W = (const uint8_t*)items[j].W;
            g.blk = (w_type == DT_FP4) ? (const uint8_t*)items[j].blk_scales : nullptr;
            g.Y = (uint16_t*)items[j].Y;
            g.N = items[j].N_out;
            g.ldw = items[j].ldw;
            g.ldy_m = items[j].ldy_m;
            g.ldy_n = items[j].ldy_n;
            g.alpha = items[j].alpha;
            g.beta = items[j].beta;
            g.w_scale = scaled ? items[j].inv_scale : 1.0f;
            g.post_scale = (w_type == DT_FP4) ? 65536.0f : (scaled ? 1.0f : items[j].inv_scale);
        }
        p.W = p.seg[0].W;
        p.blk = p.seg[0].blk;
        p.Y = p.seg[0].Y;
        p.N = p.seg[0].N;
        p.ldw = p.seg[0].ldw;
        const bool pdl = (flags & 1u) != 0;
        int r;
        if (w_type == DT_FP4) { r = launch_gemv<DT_FP4, false>(p, ws, st, pdl); }
        else if (scaled) { r = (w_type == DT_E5M2) ? launch_gemv<DT_E5M2, true>(p, ws, st, pdl) : launch_gemv<DT_E4M3, true>(p, ws, st, pdl); }
        else { r = (w_type == DT_E5M2) ? launch_gemv<DT_E5M2, false>(p, ws, st, pdl) : launch_gemv<DT_E4M3, false>(p, ws, st, pdl); }
        if (r != -2) { return r; }
    }
    // More than 32 tokens: the members' feature tiles form one grid of the tensor-core kernel.
    bool one_prefill = count >= 2 && count <= (unsigned)PF_MAX_GROUP && M_tokens > 32;
    for (unsigned int j = 0; j < count && one_prefill; j++)
    {
        one_prefill = items[j].N_out != 0
            && plan_for(w_type, items[j].W, items[j].blk_scales, X, items[j].Y, items[j].N_out, M_tokens, K, items[j].ldw, ldx,
                   items[j].ldy_m, items[j].ldy_n)
                != PLAN_PLAIN;
    }
    if (one_prefill)
    {
        GemvParams ps[PF_MAX_GROUP];
        memset(ps, 0, sizeof(ps));
        for (unsigned int j = 0; j < count; j++)
        {
            GemvParams& q = ps[j];
            q.W = (const uint8_t*)items[j].W;
            q.blk = (w_type == DT_FP4) ? (const uint8_t*)items[j].blk_scales : nullptr;
            q.X = (const uint16_t*)X;
            q.Y = (uint16_t*)items[j].Y;
            q.status = ws->status;
            q.N = items[j].N_out;
            q.M = M_tokens;
            q.K = K;
            q.ldw = items[j].ldw;
            q.ldx = ldx;
            q.ldy_m = items[j].ldy_m;
            q.ldy_n = items[j].ldy_n;
            q.w_scale = items[j].inv_scale;
            q.alpha = items[j].alpha;
            q.beta = items[j].beta;
            q.out_f32 = (flags & 4u) ? 1u : ((flags & 8u) ? 2u : 0u);
        }
        const int r = launch_prefill(w_type, ps, count, ws->device, ws->sm_count, (int)((flags >> 8) & 7u), st);
        if (r != -2) { return r; }
    }
    for (unsigned int j = 0; j < count; j++)
    {
        if (items[j].N_out == 0) { continue; }
        const int r = run_linear_wq(ws, w_type, items[j].W, items[j].blk_scales, items[j].inv_scale, X, items[j].Y, items[j].N_out,
            M_tokens, K, items[j].ldw, ldx, items[j].ldy_m, items[j].ldy_n, items[j].alpha, items[j].beta, st, flags);
        if (r != 0) { return r; }
    }
    return 0;
}

}    // namespace b200
