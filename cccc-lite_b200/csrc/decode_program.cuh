// A whole decode step (or any chain of dependent quantized-weight linears and the ops between them)
// as ONE persistent kernel: one CTA per SM walks a device-side list of phases.
//
// Why.  A decode token at batch 1 is a chain of ~150 dependent GEMVs of 4-100 MB.  As separate
// launches each of them pays for the launch, for the first bytes' DRAM latency and for the drain of
// the last CTA: HBM idles about 2.5 us per launch, 30 % of the step.  Weights, however, depend on
// nothing.  Here the producer lane of every CTA keeps streaming weights through the shared-memory ring
// ACROSS phase boundaries: while the consumers wait for the other CTAs to finish a linear (its output is
// the next linear's input) the ring is already filling with the next linear's rows.
//
// Phases.  LINEAR: up to three linears that share their input; the 256 consumer threads first build the
// input in shared memory (copy | RMSNorm with the reference's summation order | SwiGLU of two inputs),
// then the (row block, k stage) items of the CTA's run are consumed exactly as in the decode GEMV kernel
// (same k-step code, same stream-K fix-up).  ATTN_SCORES / ATTN_PV: split-KV attention of one new token
// per sequence; the two halves are separate phases because the softmax normaliser is a grid-wide value.
// Between consecutive phases every CTA arrives on one global counter and waits until all have arrived
// (the launch is cooperative, so all CTAs are resident); every wait is bounded and raises the status
// word instead of hanging.
#pragma once

#include "decode_ops.cuh"

namespace b200
{

enum : unsigned int
{
    PH_LINEAR = 0,
    PH_ATTN_SCORES = 1,
    PH_ATTN_PV = 2
};
enum : unsigned int
{
    XM_COPY = 0,       // X = x_src
    XM_RMSNORM = 1,    // X = rmsnorm(x_src) * norm_w
    XM_SWIGLU = 2      // X = swiglu(x_src, x_src2)
};

// Tile configuration of the chain: up to 2 tokens, 32 rows x 2048 k per stage (32 k steps of 64 bytes; measured
// better than twice as many stages of half the size: four k steps per warp and stage keep more loads in flight).
template <int WT>
using ChainCfg = GemvCfg<WT, 1, 2, 1, 8, 32, 2, 1>;
constexpr int kChainMaxTokens = 2;
constexpr int kChainThreads = 32 * 9;

struct ProgPhase
{
    unsigned int kind;
    // ---- LINEAR ----
    unsigned int n_seg, K, n_kstages, n_row_blocks, total_items, gran;
    unsigned int x_mode, out_mode;    // out_mode: 0 BF16, 1 float32, 2 BF16 with the product rounded before beta * Y is added
    unsigned int map_base;            // index of the phase's tensor maps: W0, S0, W1, S1, W2, S2
    unsigned int paired;              // 1: seg[0] = gate, seg[1] = up with equal N; a row block is 16 rows of each, and the
                                      // epilogue writes swiglu(gate, up) to seg[0].Y (nothing else is stored)
    unsigned int ldx, ldx2;
    float eps;
    const uint16_t* x_src;
    const uint16_t* x_src2;
    const uint16_t* norm_w;
    GemvSeg seg[kMaxGroup];
    // ---- ATTN_* ----
    AttnDecodeParams attn;
    unsigned int attn_S, attn_ts_cap;
    float* attn_stats;          // [items][G][2]
    float* attn_partial;        // [items][G * HD]
    unsigned int* attn_counters;    // [B * Hkv], zero between launches
};

struct ProgHeader
{
    const ProgPhase* phases;
    const CUtensorMap* maps;
    float* partials;            // stream-K scratch: [grid][2][tile]
    unsigned int* counters;     // [grid], zero between launches
    unsigned int* status;       // the library's status word
    unsigned int* sync;         // [0]: phase arrivals of all launches so far
    unsigned int n_phases, M, n_stages;
    unsigned int epoch;         // launches of this program so far: the arrival counter is never reset, targets move on
    unsigned int xbuf_bytes;    // bytes of the input buffer (2 token rows of the largest K), a multiple of 1024
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// The input of a LINEAR phase, built by the team in the [64-element slab][token][128 B] layout the k-step
// code reads (the layout a TMA box of two token rows would have).  Rows beyond M are zero.  All global
// loads are 16-byte loads issued before anything waits on them: what another CTA wrote a moment ago
// comes from L2, about a microsecond away, and one round trip is all this should cost.
__device__ __forceinline__ void chain_build_x(const ProgPhase& P, unsigned int M, unsigned char* xb, float* part, unsigned int tid)
{
    constexpr unsigned int XB = kChainMaxTokens;
    constexpr unsigned int kVec = 4;    // 16-byte pieces in flight per thread and pass (a pass covers 8192 elements)
    const unsigned int K = P.K, nvec = K / 8;
    auto slot = [&](unsigned int m, unsigned int k) { return xb + (((size_t)(k >> 6) * XB + m) << 7) + ((k & 63u) << 1); };
    for (unsigned int m = M; m < XB; m++)
    {
        for (unsigned int i = tid; i < nvec; i += kTeam) { *reinterpret_cast<uint4*>(slot(m, i * 8)) = make_uint4(0, 0, 0, 0); }
    }
    if (P.x_mode == XM_SWIGLU)
    {
        for (unsigned int m = 0; m < M; m++)
        {
            const uint4* g = reinterpret_cast<const uint4*>(P.x_src + (size_t)m * P.ldx);
            const uint4* u = reinterpret_cast<const uint4*>(P.x_src2 + (size_t)m * P.ldx2);
            for (unsigned int base = 0; base < nvec; base += kVec * kTeam)
            {
                uint4 gv[kVec], uv[kVec];
#pragma unroll
                for (unsigned int q = 0; q < kVec; q++)
                {
                    const unsigned int i = base + tid + q * kTeam;
                    gv[q] = i < nvec ? __ldcg(g + i) : make_uint4(0, 0, 0, 0);
                    uv[q] = i < nvec ? __ldcg(u + i) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (unsigned int q = 0; q < kVec; q++)
                {
                    const unsigned int i = base + tid + q * kTeam;
                    if (i < nvec)
                    {
                        float gf[8], uf[8];
                        unpack8(gv[q], gf);
                        unpack8(uv[q], uf);
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; e++)
                        {
                            o[e] = (uint32_t)bf16_bits(swiglu_one(gf[2 * e], uf[2 * e])) | ((uint32_t)bf16_bits(swiglu_one(gf[2 * e + 1], uf[2 * e + 1])) << 16);
                        }
                        *reinterpret_cast<uint4*>(slot(m, i * 8)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
            }
        }
        return;
    }
    // COPY, and the first half of RMSNORM: the raw rows go into their slots
    const bool norm = P.x_mode == XM_RMSNORM;
    for (unsigned int m = 0; m < M; m++)
    {
        const uint4* src = reinterpret_cast<const uint4*>(P.x_src + (size_t)m * P.ldx);
        for (unsigned int base = 0; base < nvec; base += kVec * kTeam)
        {
            uint4 v[kVec];
#pragma unroll
            for (unsigned int q = 0; q < kVec; q++)
            {
                const unsigned int i = base + tid + q * kTeam;
                v[q] = i < nvec ? __ldcg(src + i) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (unsigned int q = 0; q < kVec; q++)
            {
                const unsigned int i = base + tid + q * kTeam;
                if (i < nvec) { *reinterpret_cast<uint4*>(slot(m, i * 8)) = v[q]; }
            }
        }
    }
    if (!norm) { return; }
    // cccc-cuda/cuda_functions.cu:904-933: thread t sums x[t], x[t + 256], ... with a fused multiply-add each, then
    // a halving tree; y = bf16((x * invstd) * scale).  The sums read the rows back from shared memory in that
    // order.  The norm weights of the first pass are fetched before the sums so that their latency hides there.
    const uint4* wsrc = reinterpret_cast<const uint4*>(P.norm_w);
    uint4 wv[kVec];
#pragma unroll
    for (unsigned int q = 0; q < kVec; q++)
    {
        const unsigned int i = tid + q * kTeam;
        wv[q] = (wsrc != nullptr && i < nvec) ? __ldg(wsrc + i) : make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
    }
    team_sync();
    for (unsigned int m = 0; m < M; m++)
    {
        float s = 0.f;
#pragma unroll 8
        for (unsigned int i = tid; i < K; i += kTeam)
        {
            const float xv = bf16_bits_to_float(*reinterpret_cast<const uint16_t*>(slot(m, i)));
            s = __fmaf_rn(xv, xv, s);
        }
        part[m * kTeam + tid] = s;
    }
    team_tree_sum(part, M, tid);
    for (unsigned int m = 0; m < M; m++)
    {
        const float invstd = rms_invstd(part[m * kTeam], K, P.eps);
        for (unsigned int base = 0; base < nvec; base += kVec * kTeam)
        {
#pragma unroll
            for (unsigned int q = 0; q < kVec; q++)
            {
                const unsigned int i = base + tid + q * kTeam;
                if (i < nvec)
                {
                    uint4* px = reinterpret_cast<uint4*>(slot(m, i * 8));
                    const uint4 w4 = base == 0 ? wv[q] : (wsrc != nullptr ? __ldg(wsrc + i) : wv[q]);
                    float xf[8], wf[8];
                    unpack8(*px, xf);
                    unpack8(w4, wf);
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; e++)
                    {
                        o[e] = (uint32_t)bf16_bits(rms_apply(xf[2 * e], invstd, wf[2 * e]))
                            | ((uint32_t)bf16_bits(rms_apply(xf[2 * e + 1], invstd, wf[2 * e + 1])) << 16);
                    }
                    *px = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        }
    }
}

// One segment (consecutive k stages of one row block) of this CTA's run: wait for each stage, run the k
// steps of this warp, hand the stage back, and leave this warp's partial sums in red[wk][token][row].
// MODE 0: tensor-core k step (any scale); MODE 1 / 2: CUDA-core k step for one / two tokens.
template <class Cfg, bool SCALED, int MODE>
__device__ __forceinline__ bool chain_consume_segment(const unsigned int seg, const unsigned int ks0, const unsigned int K, unsigned int& it,
    const unsigned int NS, unsigned char* stages, const unsigned int stage_bytes, uint64_t* full_bar, uint64_t* empty_bar,
    volatile unsigned int* sh_flags, unsigned int* status, const uint32_t xbuf_addr, float* red, const float w_scale, bool ok,
    const unsigned int wr, const unsigned int wk, const unsigned int lane, const bool paired, const float w_scale_second)
{
    constexpr int RT = Cfg::RT, MT = Cfg::MT, WK = Cfg::WK, R = Cfg::R;
    constexpr unsigned int TILE = R * 8 * MT;
    constexpr int NT = MODE == 2 ? 2 : 1;
    constexpr int SPW = (Cfg::SKS + WK - 1) / WK;
    const unsigned int g = lane >> 2, t = lane & 3;
    float acc[RT][MT][2][4];
    float facc[RT][2][NT];
    if (MODE == 0)
    {
#pragma unroll
        for (int a = 0; a < RT; a++)
#pragma unroll
            for (int b = 0; b < MT; b++)
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int d = 0; d < 4; d++) { acc[a][b][c][d] = 0.f; }
    }
    else
    {
#pragma unroll
        for (int a = 0; a < RT; a++)
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int c = 0; c < NT; c++) { facc[a][b][c] = 0.f; }
    }
    for (unsigned int j = 0; j < seg; j++, it++)
    {
        const unsigned int s = it % NS;
        if (ok && (sh_flags[0] != 0 || !mbar_wait_bounded(full_bar + s, (it / NS) & 1u)))
        {
            ok = false;
            if (sh_flags[0] == 0)
            {
                atomicMax(status, (unsigned int)ST_TIMEOUT_FULL);
                sh_flags[0] = 1;
            }
        }
        if (!ok) { continue; }
        const unsigned int ks = ks0 + j;
        const unsigned int kval = min((unsigned int)Cfg::SKE, K - ks * Cfg::SKE);
        const unsigned int nsteps = kval / Cfg::KSTEP;    // beyond K the TMA fills zeros; skip them
        const uint32_t st = smem_u32(stages + (size_t)s * stage_bytes);
        const uint32_t xt = xbuf_addr + ks * (Cfg::XSLABS * Cfg::XB * 128);
        if (nsteps == (unsigned int)Cfg::SKS)
        {
#pragma unroll
            for (int u = 0; u < SPW; u++)
            {
                if (MODE == 0) { gemv_k_step<Cfg, SCALED>(acc, st, xt, wk + u * WK, wr, g, t, w_scale, paired, w_scale_second); }
                else { gemv_k_step_fma<Cfg, NT>(facc, st, xt, wk + u * WK, wr, g, t, paired); }
            }
        }
        else
        {
            for (unsigned int step = wk; step < nsteps; step += WK)
            {
                if (MODE == 0) { gemv_k_step<Cfg, SCALED>(acc, st, xt, step, wr, g, t, w_scale, paired, w_scale_second); }
                else { gemv_k_step_fma<Cfg, NT>(facc, st, xt, step, wr, g, t, paired); }
            }
        }
        __syncwarp();
        if (lane == 0) { mbar_arrive(empty_bar + s); }
    }
    float* myred = red + wk * TILE;
    if (MODE == 0)
    {
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
        {
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
            {
                const unsigned int row = (wr * RT + rt) * 16 + g;
                const unsigned int tok = mt * 8 + 2 * t;
                myred[tok * R + row] = acc[rt][mt][0][0] + acc[rt][mt][1][0];
                myred[(tok + 1) * R + row] = acc[rt][mt][0][1] + acc[rt][mt][1][1];
                myred[tok * R + row + 8] = acc[rt][mt][0][2] + acc[rt][mt][1][2];
                myred[(tok + 1) * R + row + 8] = acc[rt][mt][0][3] + acc[rt][mt][1][3];
            }
        }
    }
    else
    {
        // the four lanes of a row hold the four quarters of each 64-byte k step: add them in a fixed order
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int m = 0; m < NT; m++)
                {
                    float v = facc[rt][h][m];
                    v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                    v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
                    if (t == 0) { myred[m * R + (wr * RT + rt) * 16 + h * 8 + g] = v; }
                }
    }
    return ok;
}

template <int WT, bool SCALED, int G, bool FMA>
__global__ void __launch_bounds__(kChainThreads, 1) decode_program_kernel(const ProgHeader hd)
{
    using Cfg = ChainCfg<WT>;
    constexpr int MT = Cfg::MT, WK = Cfg::WK, R = Cfg::R, HD = 128;
    constexpr int kConsumerWarps = Cfg::NCW;
    constexpr unsigned int STAGE = ((Cfg::W_BYTES + Cfg::S_BYTES + 1023) / 1024) * 1024;
    constexpr unsigned int TILE = R * 8 * MT;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = full_bar + Cfg::kMaxStages;
    // sh_flags[0] = abort, [1] = "this CTA reduces the row block" / "last split", [2] = scratch
    volatile unsigned int* sh_flags = reinterpret_cast<volatile unsigned int*>(smem + 2 * Cfg::kMaxStages * 8);
    unsigned char* stages = smem + Cfg::HEADER_BYTES;
    const unsigned int NS = hd.n_stages;
    unsigned char* ubase = stages + (size_t)NS * STAGE;             // the region phases share
    unsigned char* xbuf = ubase;
    float* red = reinterpret_cast<float*>(ubase + hd.xbuf_bytes);   // [WK][TILE] floats; also the norms' partial sums
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned int cta = blockIdx.x, grid = gridDim.x;

    if (threadIdx.x == 0)
    {
        for (unsigned int s = 0; s < NS; s++)
        {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, kConsumerWarps);
        }
        sh_flags[0] = 0;
        sh_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps)
    {
        // =========================== producer: one elected lane ===========================
        // Streams the weights of every LINEAR phase, in phase order, as far ahead as the ring allows.
        // It never waits for another CTA: weights depend on nothing.
        if (lane != 0) { return; }
        const uint64_t pol_stream = l2_policy_evict_first();
        unsigned int it = 0;
        bool ok = true;
        for (unsigned int ph = 0; ph < hd.n_phases && ok; ph++)
        {
            const ProgPhase& P = hd.phases[ph];
            if (P.kind != PH_LINEAR) { continue; }
            const ItemRange items = cta_items(cta, grid, P.total_items, P.gran);
            if (items.end == items.beg) { continue; }
            // the tensor maps were written by the host before the launch: no proxy fence is needed to use them
            const CUtensorMap* maps = hd.maps + P.map_base;
            const unsigned int rb1 = P.seg[1].rb_begin, rb2 = P.seg[2].rb_begin, nk = P.n_kstages;
            for (unsigned int item = items.beg; item < items.end; item++, it++)
            {
                const unsigned int s = it % NS;
                if (it >= NS && (sh_flags[0] != 0 || !mbar_wait_bounded(empty_bar + s, ((it / NS) - 1) & 1u)))
                {
                    ok = false;
                    if (sh_flags[0] == 0) { atomicMax(hd.status, (unsigned int)ST_TIMEOUT_EMPTY); }
                    sh_flags[0] = 1;
                    break;
                }
                const unsigned int rb = item / nk, ks = item % nk;
                unsigned char* st = stages + (size_t)s * STAGE;
                mbar_expect_tx(full_bar + s, Cfg::W_BYTES + Cfg::S_BYTES);
                if (P.paired)
                {
                    // 16 rows of the gate matrix, then the same 16 rows of the up matrix
                    const int row0 = (int)(rb * 16);
                    tma_load_3d_hint(st, maps, 0, row0, (int)(ks * Cfg::SKS), full_bar + s, pol_stream);
                    tma_load_3d_hint(st + Cfg::W_BYTES / 2, maps + 2, 0, row0, (int)(ks * Cfg::SKS), full_bar + s, pol_stream);
                    if (WT == DT_FP4)
                    {
                        tma_load_3d_hint(st + Cfg::W_BYTES, maps + 1, 0, row0, (int)(ks * (Cfg::SKS / 2)), full_bar + s, pol_stream);
                        tma_load_3d_hint(st + Cfg::W_BYTES + Cfg::S_BYTES / 2, maps + 3, 0, row0, (int)(ks * (Cfg::SKS / 2)), full_bar + s,
                            pol_stream);
                    }
                }
                else
                {
                    const unsigned int j = (rb >= rb1 ? 1u : 0u) + (rb >= rb2 ? 1u : 0u);
                    const unsigned int rbb = j == 0 ? 0u : (j == 1 ? rb1 : rb2);
                    const int row0 = (int)((rb - rbb) * R);
                    tma_load_3d_hint(st, maps + 2 * j, 0, row0, (int)(ks * Cfg::SKS), full_bar + s, pol_stream);
                    if (WT == DT_FP4)
                    {
                        tma_load_3d_hint(st + Cfg::W_BYTES, maps + 2 * j + 1, 0, row0, (int)(ks * (Cfg::SKS / 2)), full_bar + s, pol_stream);
                    }
                }
                mbar_arrive(full_bar + s);
            }
        }
        // Do not leave while copies are in flight: the consumers' "empty" arrivals prove that a stage has
        // landed and been read; after an abort wait (bounded) for the outstanding stages to land instead.
        const unsigned int first = it > NS ? it - NS : 0;
        for (unsigned int i = first; i < it; i++)
        {
            uint64_t* bar = ok ? empty_bar + (i % NS) : full_bar + (i % NS);
            if (!mbar_wait_bounded(bar, (i / NS) & 1u))
            {
                if (ok && sh_flags[0] == 0) { atomicMax(hd.status, (unsigned int)ST_TIMEOUT_EMPTY); }
                ok = false;
            }
        }
        return;
    }

    // =========================== consumer team ===========================
    const unsigned int wr = warp / WK, wk = warp % WK;
    const unsigned int ctid = threadIdx.x;
    bool ok = true;
    unsigned int it = 0;
    for (unsigned int ph = 0; ph < hd.n_phases; ph++)
    {
        const ProgPhase& P = hd.phases[ph];
        if (ph > 0)
        {
            // every CTA has finished the previous phase: its outputs are this phase's inputs
            if (ctid == 0 && ok)
            {
                const unsigned int target = (hd.epoch * hd.n_phases + ph) * grid;    // wraps with the counter
                const unsigned long long t0 = global_timer_ns();
                unsigned int spins = 0;
                while ((int)(ld_acquire_gpu(hd.sync) - target) < 0)
                {
                    if ((++spins & 0x3Fu) == 0
                        && (sh_flags[0] != 0 || *reinterpret_cast<volatile unsigned int*>(hd.status) != 0 || global_timer_ns() - t0 > kWaitLimitNs))
                    {
                        if (*reinterpret_cast<volatile unsigned int*>(hd.status) == 0) { atomicMax(hd.status, (unsigned int)ST_TIMEOUT_PEER); }
                        sh_flags[0] = 1;
                        break;
                    }
                }
            }
            team_sync();
            if (sh_flags[0] != 0) { ok = false; }
        }

        if (P.kind == PH_LINEAR)
        {
            const ItemRange items = cta_items(cta, grid, P.total_items, P.gran);
            const unsigned int n_items = items.end - items.beg;
            if (n_items > 0 && ok)
            {
                chain_build_x(P, hd.M, xbuf, red, ctid);
                team_sync();
            }
            unsigned int done = 0;
            while (done < n_items)
            {
                const unsigned int item0 = items.beg + done;
                const unsigned int rb = item0 / P.n_kstages;
                const unsigned int ks0 = item0 % P.n_kstages;
                const unsigned int seg = min(P.n_kstages - ks0, n_items - done);
                const bool first_segment = (done == 0);
                const unsigned int lj = P.paired ? 0u : (rb >= P.seg[1].rb_begin ? 1u : 0u) + (rb >= P.seg[2].rb_begin ? 1u : 0u);
                const GemvSeg& L = P.seg[lj];
                const float w_scale = L.w_scale;
                if (FMA)
                {
                    ok = hd.M == 1 ? chain_consume_segment<Cfg, SCALED, 1>(seg, ks0, P.K, it, NS, stages, STAGE, full_bar, empty_bar, sh_flags,
                                         hd.status, smem_u32(xbuf), red, w_scale, ok, wr, wk, lane, P.paired != 0, P.seg[1].w_scale)
                                   : chain_consume_segment<Cfg, SCALED, 2>(seg, ks0, P.K, it, NS, stages, STAGE, full_bar, empty_bar, sh_flags,
                                         hd.status, smem_u32(xbuf), red, w_scale, ok, wr, wk, lane, P.paired != 0, P.seg[1].w_scale);
                }
                else
                {
                    ok = chain_consume_segment<Cfg, SCALED, 0>(seg, ks0, P.K, it, NS, stages, STAGE, full_bar, empty_bar, sh_flags, hd.status,
                        smem_u32(xbuf), red, w_scale, ok, wr, wk, lane, P.paired != 0, P.seg[1].w_scale);
                }
                done += seg;
                team_sync();
                const unsigned int n_out = P.paired ? hd.M * 16u : hd.M * R;
                const bool full = (ks0 == 0 && seg == P.n_kstages);
                const unsigned int n0 = P.paired ? rb * 16u : (rb - L.rb_begin) * R;
                // paired: entry e = (token m, row r < 16) -> gate sum at [m][r], up sum at [m][r + 16] of the tile
                auto tile_index = [&](unsigned int e) { return P.paired ? (e >> 4) * R + (e & 15u) : e; };
                auto store_pair = [&](unsigned int e, float gsum, float usum) {
                    const unsigned int m = e >> 4, n = n0 + (e & 15u);
                    if (n < L.N)
                    {
                        const GemvSeg& U = P.seg[1];
                        const float gv = bf16_round(L.alpha * (gsum * L.post_scale));
                        const float uv = bf16_round(U.alpha * (usum * U.post_scale));
                        L.Y[(long long)m * L.ldy_m + (long long)n * L.ldy_n] = bf16_bits(swiglu_one(gv, uv));
                    }
                };
                auto store_out = [&](unsigned int e, float v) {
                    const unsigned int m = e / R, r = e - m * R;
                    const unsigned int n = n0 + r;
                    if (n < L.N)
                    {
                        const long long yi = (long long)m * L.ldy_m + (long long)n * L.ldy_n;
                        float o = L.alpha * (v * L.post_scale);
                        if (P.out_mode == 1u)
                        {
                            float* y = reinterpret_cast<float*>(L.Y) + yi;
                            if (L.beta != 0.f) { o += L.beta * __ldcg(y); }
                            *y = o;
                        }
                        else
                        {
                            uint16_t* y = L.Y + yi;
                            if (L.beta != 0.f) { o = (P.out_mode == 2u ? bf16_round(o) : o) + L.beta * ld_bf16_cg(y); }
                            *y = bf16_bits(o);
                        }
                    }
                };
                if (full)
                {
                    if (ok)
                    {
                        for (unsigned int e = ctid; e < n_out; e += kTeam)
                        {
                            const unsigned int ti = tile_index(e);
                            float v = 0.f, v2 = 0.f;
#pragma unroll
                            for (int w = 0; w < WK; w++) { v += red[w * TILE + ti]; }
                            if (P.paired)
                            {
#pragma unroll
                                for (int w = 0; w < WK; w++) { v2 += red[w * TILE + ti + 16]; }
                                store_pair(e, v, v2);
                            }
                            else { store_out(e, v); }
                        }
                    }
                }
                else
                {
                    float* mine = hd.partials + ((size_t)cta * 2 + (first_segment ? 0 : 1)) * TILE;
                    if (ok)
                    {
                        for (unsigned int e = ctid; e < hd.M * R; e += kTeam)
                        {
                            float v = 0.f;
#pragma unroll
                            for (int w = 0; w < WK; w++) { v += red[w * TILE + e]; }
                            __stcg(mine + e, v);
                        }
                    }
                    team_sync();
                    const unsigned int c_first = cta_of_item(rb * P.n_kstages, grid, P.total_items, P.gran);
                    const unsigned int c_last = cta_of_item(rb * P.n_kstages + P.n_kstages - 1, grid, P.total_items, P.gran);
                    if (ctid == 0)
                    {
                        unsigned int last = 0;
                        if (ok && sh_flags[0] == 0)
                        {
                            __threadfence();
                            const unsigned int old = atomicAdd(hd.counters + c_first, 1u);
                            last = (old == c_last - c_first) ? 1u : 0u;
                            __threadfence();
                        }
                        sh_flags[1] = last;
                    }
                    team_sync();
                    if (sh_flags[1] != 0)
                    {
                        for (unsigned int e = ctid; e < n_out; e += kTeam)
                        {
                            const unsigned int ti = tile_index(e);
                            float v = 0.f, v2 = 0.f;
                            for (unsigned int c = c_first; c <= c_last; c++)
                            {
                                const unsigned int slot = (cta_items(c, grid, P.total_items, P.gran).beg / P.n_kstages == rb) ? 0u : 1u;
                                const float* part = hd.partials + ((size_t)c * 2 + slot) * TILE;
                                v += __ldcg(part + ti);
                                if (P.paired) { v2 += __ldcg(part + ti + 16); }
                            }
                            if (P.paired) { store_pair(e, v, v2); }
                            else { store_out(e, v); }
                        }
                        if (ctid == 0) { hd.counters[c_first] = 0; }
                    }
                }
                team_sync();    // `red` and sh_flags[1] are reused by the next segment
            }
        }
        else
        {
            // ---- attention: item = (sequence, kv head, split), one per CTA ----
            const AttnDecodeParams& A = P.attn;
            const unsigned int S = P.attn_S, ts_cap = P.attn_ts_cap;
            const unsigned int n_att = A.B * A.Hkv * S;
            if (cta < n_att && ok)
            {
                AttnSmem<G, HD> sm(reinterpret_cast<float*>(ubase), ts_cap);
                const unsigned int rank = cta % S, bh = cta / S, kvh = bh % A.Hkv, b = bh / A.Hkv;
                const int pos_i = __ldcg(A.pos + b);
                const unsigned int pos = pos_i < 0 ? 0u : (unsigned int)pos_i;
                const unsigned int T = min(pos + 1u, A.T_max);
                unsigned int ts = (T + S - 1) / S;
                ts = (ts + 31u) & ~31u;
                const unsigned int t0 = min(rank * ts, T), t1 = min(t0 + ts, T);
                const bool owner = pos >= t0 && pos < t1;
                if (P.kind == PH_ATTN_SCORES)
                {
                    attn_scores<G, HD, 4>(A, sm, b, kvh, t0, t1, ts_cap, pos, owner, ctid);    // (runs the prologue too; 4 passes in flight: 168 registers)
                    if (ctid < 2 * G) { __stcg(P.attn_stats + (size_t)cta * 2 * G + ctid, sm.ml[ctid]); }
                }
                else
                {
                    attn_pv<G, HD>(A, sm, b, kvh, t0, t1, ts_cap, owner ? pos : 0xFFFFFFFFu, ctid, [&]() {
                        if (ctid < G)
                        {
                            const float* st = P.attn_stats + (size_t)bh * S * 2 * G;
                            float gmax = -INFINITY;
                            for (unsigned int r = 0; r < S; r++) { gmax = fmaxf(gmax, __ldcg(st + r * 2 * G + 2 * ctid)); }
                            float Lsum = 0.f;
                            for (unsigned int r = 0; r < S; r++)
                            {
                                const float l = __ldcg(st + r * 2 * G + 2 * ctid + 1);
                                if (l > 0.f) { Lsum += l * __expf(__ldcg(st + r * 2 * G + 2 * ctid) - gmax); }
                            }
                            sm.gl[2 * ctid] = gmax;
                            sm.gl[2 * ctid + 1] = 1.0f / Lsum;
                        }
                    });
                    float* mine = P.attn_partial + (size_t)cta * G * HD;
                    for (unsigned int i = ctid; i < G * HD; i += kTeam) { __stcg(mine + i, sm.opart[i]); }
                    team_sync();
                    if (ctid == 0)
                    {
                        __threadfence();
                        const unsigned int old = atomicAdd(P.attn_counters + bh, 1u);
                        __threadfence();
                        sh_flags[1] = (old == S - 1) ? 1u : 0u;
                    }
                    team_sync();
                    if (sh_flags[1] != 0)
                    {
                        // the last split of this (sequence, kv head) adds the splits in order and rounds once
                        const float* parts = P.attn_partial + (size_t)bh * S * G * HD;
                        uint16_t* o = A.out + (size_t)b * A.ldo + (size_t)kvh * G * HD;
                        for (unsigned int i = ctid; i < G * HD; i += kTeam)
                        {
                            float sacc = 0.f;
                            for (unsigned int r = 0; r < S; r++) { sacc += __ldcg(parts + (size_t)r * G * HD + i); }
                            o[i] = bf16_bits(sacc);
                        }
                        if (ctid == 0) { P.attn_counters[bh] = 0; }
                    }
                }
            }
        }

        // ---- this CTA has finished the phase ----
        team_sync();
        // (the barrier above orders the team's writes before thread 0's release, which is cumulative over them)
        if (ctid == 0) { asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(hd.sync) : "memory"); }
    }
}

}    // namespace b200
