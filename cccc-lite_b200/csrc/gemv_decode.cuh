// Decode-side quantized-weight linear (M <= 32 tokens): an HBM-bound GEMV.
//
// One persistent CTA per SM.  A producer warp streams the weight bytes (and FP4 block scales)
// from HBM into a shared-memory ring with bulk asynchronous copies (cp.async.bulk + mbarrier),
// one copy per weight row segment, and stages the matching slice of the BF16 activations.
// Eight consumer warps dequantise to BF16 in registers and feed m16n8k16 BF16 MMAs with FP32
// accumulators: the weight tile is the A operand (16 output features x 16 k), the tokens are
// the 8 columns of B.  The k order inside a fragment is permuted so that every lane converts
// the 16 bytes it loaded itself; the activation slice is staged in the same permutation.
//
// Work is cut stream-K style: the (row block, k stage) items of the whole matrix are dealt to
// the CTAs in equal contiguous runs, so every SM streams the same number of bytes whatever the
// shape.  A run that covers only part of a row block's k range writes an FP32 partial tile to
// the workspace; the last CTA to arrive for that row block adds the partials in CTA order
// (a fixed order, so results are reproducible) and writes the BF16 output.
//
// Every wait is bounded: a wait that runs out raises the status word and the CTA drains without
// touching the barrier again.
#pragma once

#include "common.cuh"

namespace b200
{

struct GemvParams
{
    const uint8_t* W;      // [N, ldw] quantised weight
    const uint8_t* blk;    // FP4 block scales (E4M3 bytes), one per 16 elements of the flat buffer
    const uint16_t* X;     // [M, ldx] bf16
    uint16_t* Y;           // bf16, element (m, n) at m*ldy_m + n*ldy_n
    float* partials;       // workspace: [grid][2][R * 8*MT] fp32
    unsigned int* counters;    // workspace: [grid] arrival counters, zero between launches
    unsigned int* status;      // workspace: error word (0 = clean)
    unsigned int N, M, K;
    unsigned int ldw, ldx;      // elements
    long long ldy_m, ldy_n;     // elements
    float w_scale;              // multiplier applied to each decoded weight before BF16 rounding
    float alpha, beta;
    float post_scale;           // exact power of two folded out of the weights (applied with alpha)
    unsigned int n_row_blocks, n_kstages, total_items;
    unsigned int n_stages;      // ring depth
};

constexpr int kConsumerWarps = 8;
constexpr int kGemvThreads = 32 * (kConsumerWarps + 1);
constexpr unsigned long long kWaitLimitNs = 2000000000ull;    // 2 s

enum : unsigned int
{
    ST_OK = 0,
    ST_TIMEOUT_FULL = 1,
    ST_TIMEOUT_EMPTY = 2,
    ST_TIMEOUT_FIXUP = 3
};

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cta.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false when the limit ran out (the caller raises the status word).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) { return true; }
    const unsigned long long t0 = global_timer_ns();
    unsigned int spins = 0;
    while (!mbar_try_wait(bar, parity))
    {
        if ((++spins & 0x3FFu) == 0 && global_timer_ns() - t0 > kWaitLimitNs) { return false; }
    }
    return true;
}
// 1-D bulk copy global -> shared, completion counted on an mbarrier.  Both addresses and the
// size are multiples of 16 bytes (checked on the host before this kernel is chosen).
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void consumer_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr)
{
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
    uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- in-register dequantisation ----------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t h)
{
    __half2 v;
    *reinterpret_cast<uint32_t*>(&v) = h;
    return __half22float2(v);
}
// Four FP8 bytes (k, k+1, k+2, k+3) -> two bf16x2 registers (k,k+1) and (k+2,k+3), each value
// rne_bf16(decode * scale).  E5M2 is the top byte of an FP16, so a byte permute widens it;
// E4M3 uses the hardware e4m3x2 -> f16x2 conversion.  SCALED = false skips the multiply (the
// decoded value is exactly representable in BF16, so no rounding happens at all).
template <int WT, bool SCALED>
__device__ __forceinline__ void dequant_fp8x4(uint32_t w, float scale, uint32_t& r01, uint32_t& r23)
{
    uint32_t h01, h23;
    if (WT == DT_E5M2)
    {
        h01 = prmt(w, 0u, 0x1404u);
        h23 = prmt(w, 0u, 0x3424u);
    }
    else
    {
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"((uint16_t)(w & 0xFFFFu)));
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"((uint16_t)(w >> 16)));
    }
    float2 f01 = half2_bits_to_float2(h01);
    float2 f23 = half2_bits_to_float2(h23);
    if (SCALED)
    {
        f01.x *= scale;
        f01.y *= scale;
        f23.x *= scale;
        f23.y *= scale;
    }
    r01 = pack_bf16x2(f01.x, f01.y);
    r23 = pack_bf16x2(f23.x, f23.y);
}

__device__ __forceinline__ uint32_t hmul2_bf16(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// Eight E2M1 nibbles (one 32-bit word, elements e0..e7, e0 in the low nibble) -> four bf16x2
// registers holding the element pairs (e0,e4) (e1,e5) (e2,e6) (e3,e7), each value
// table[nibble] * s * 2^-16, where mult = bf16x2(s * 2^110, s * 2^110).
// The three magnitude bits are dropped into the low exponent bits and the top mantissa bit of a
// BF16 (value = table * 2^-126, the 0.5 code being a BF16 subnormal) and one multiply both
// rescales and applies the block scale; the product table * s has at most 6 significant bits, so
// it is exact.  The 2^-16 left in is taken out after accumulation.
__device__ __forceinline__ void dequant_fp4x8(uint32_t w, uint32_t mult, uint32_t (&r)[4])
{
    const uint32_t magmask = 0x01C001C0u, sgnmask = 0x80008000u;
    r[0] = hmul2_bf16(((w << 6) & magmask) | ((w << 12) & sgnmask), mult);
    r[1] = hmul2_bf16(((w << 2) & magmask) | ((w << 8) & sgnmask), mult);
    r[2] = hmul2_bf16(((w >> 2) & magmask) | ((w << 4) & sgnmask), mult);
    r[3] = hmul2_bf16(((w >> 6) & magmask) | (w & sgnmask), mult);
}
// Two E4M3 block-scale bytes (low 16 bits of `two`) -> bf16x2 multipliers (s0*2^110 in both
// halves) and (s1*2^110 in both halves).  byte << 4 is the BF16 whose exponent field is the
// E4M3 exponent and whose top mantissa bits are the E4M3 mantissa: value = s * 2^-120, with
// E4M3 subnormals landing on BF16 subnormals; one exact multiply by 2^230 is not representable,
// so the factor is split: * 2^115 twice.
__device__ __forceinline__ void fp4_block_multipliers(uint32_t two, uint32_t& m0, uint32_t& m1)
{
    // magnitude bits of each byte to bits 4..10 of its half, sign bit to bit 15
    const uint32_t both = ((two & 0x7Fu) << 4) | ((two & 0x80u) << 8) | ((two & 0x7F00u) << 12) | ((two & 0x8000u) << 16);
    const uint32_t c115 = 0x79007900u;                                        // bf16 2^115 twice
    uint32_t v = hmul2_bf16(hmul2_bf16(both, c115), c115);                    // (s0, s1) * 2^110
    m0 = prmt(v, v, 0x1010u);
    m1 = prmt(v, v, 0x3232u);
}

// ---- geometry ------------------------------------------------------------------------------------
// MT  : token groups of 8 (tokens <= 8*MT)
// RT  : 16-row MMA tiles per warp along N
// WR  : consumer warps along N (the other kConsumerWarps/WR warps split the k steps of a stage)
// SKS : k steps per stage; one k step is 64 bytes of every weight row
template <int WT_, int MT_, int RT_, int WR_, int SKS_>
struct GemvCfg
{
    static constexpr int WT = WT_, MT = MT_, RT = RT_, WR = WR_, SKS = SKS_;
    static constexpr int WK = kConsumerWarps / WR;
    static constexpr int R = 16 * RT * WR;                        // rows per row block
    static constexpr int KSTEP = (WT == DT_FP4) ? 128 : 64;       // elements per k step
    static constexpr int SKB = 64 * SKS;                          // weight bytes per row per stage
    static constexpr int SKE = KSTEP * SKS;                       // elements per stage along k
    static constexpr int WPITCH = SKB + 64;                       // pitch % 128 == 64: conflict-free 128-bit reads
    static constexpr int SPITCH = (WT == DT_FP4) ? (SKE / 16 + 16) : 0;
    static constexpr int XPITCH = SKE * 2 + 16;
    static constexpr int W_BYTES = R * WPITCH;
    static constexpr int S_BYTES = R * SPITCH;
    static constexpr int RED_BYTES = WK * R * 8 * MT * 4;
    __host__ __device__ static constexpr int x_bytes(int m) { return ((m * XPITCH + 127) / 128) * 128; }
    __host__ __device__ static constexpr int stage_bytes(int m) { return W_BYTES + S_BYTES + x_bytes(m); }
    // barriers (2 * 16 * 8 B) + flags, padded to 512 B
    static constexpr int HEADER_BYTES = 512;
    static constexpr int kMaxStages = 16;
};

struct ItemRange
{
    unsigned int beg, end;
};
__host__ __device__ inline ItemRange cta_items(unsigned int cta, unsigned int grid, unsigned int total)
{
    ItemRange r;
    r.beg = (unsigned int)(((unsigned long long)cta * total) / grid);
    r.end = (unsigned int)(((unsigned long long)(cta + 1) * total) / grid);
    return r;
}
// The CTA whose run contains item i: the largest c with floor(c*total/grid) <= i.
__host__ __device__ inline unsigned int cta_of_item(unsigned int i, unsigned int grid, unsigned int total)
{
    return (unsigned int)((((unsigned long long)i + 1) * grid - 1) / total);
}

// ---- the kernel ------------------------------------------------------------------------------------
template <class Cfg, bool SCALED>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_wq_kernel(const GemvParams p)
{
    constexpr int WT = Cfg::WT, MT = Cfg::MT, RT = Cfg::RT, WK = Cfg::WK, R = Cfg::R;
    constexpr int AREGS = (WT == DT_FP4) ? 16 : 8;    // bf16x2 registers per weight row per k step
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = full_bar + Cfg::kMaxStages;
    // sh_flags[0] = abort, sh_flags[1] = "this CTA reduces the row block"
    volatile unsigned int* sh_flags = reinterpret_cast<volatile unsigned int*>(smem + 2 * Cfg::kMaxStages * 8);
    float* red = reinterpret_cast<float*>(smem + Cfg::HEADER_BYTES);
    unsigned char* stages = smem + Cfg::HEADER_BYTES + Cfg::RED_BYTES;
    const unsigned int stage_bytes = (unsigned int)Cfg::stage_bytes((int)p.M);
    const unsigned int NS = p.n_stages;

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const ItemRange items = cta_items(blockIdx.x, gridDim.x, p.total_items);
    const unsigned int n_items = items.end - items.beg;

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
    pdl_launch_dependents();

    if (warp == kConsumerWarps)
    {
        // =========================== producer warp ===========================
        auto issue_weights = [&](unsigned int it) {
            const unsigned int item = items.beg + it;
            const unsigned int rb = item / p.n_kstages, ks = item % p.n_kstages;
            const unsigned int s = it % NS;
            unsigned char* st = stages + (size_t)s * stage_bytes;
            const unsigned int k0 = ks * Cfg::SKE;
            const unsigned int kval = min((unsigned int)Cfg::SKE, p.K - k0);    // valid elements along k
            const unsigned int wbytes = (WT == DT_FP4) ? kval / 2 : kval;
            const unsigned int sbytes = (WT == DT_FP4) ? kval / 16 : 0;
            const unsigned int n0 = rb * R;
            const unsigned int rows = min((unsigned int)R, p.N - n0);
            if (lane == 0) { mbar_expect_tx(full_bar + s, rows * (wbytes + sbytes)); }
            __syncwarp();
            for (unsigned int r = lane; r < rows; r += 32)
            {
                const size_t e = (size_t)(n0 + r) * p.ldw + k0;    // element index of the row segment
                bulk_g2s(st + r * Cfg::WPITCH, p.W + ((WT == DT_FP4) ? e / 2 : e), wbytes, full_bar + s);
                if (WT == DT_FP4) { bulk_g2s(st + Cfg::W_BYTES + r * Cfg::SPITCH, p.blk + e / 16, sbytes, full_bar + s); }
            }
        };
        auto stage_x = [&](unsigned int it) {
            const unsigned int item = items.beg + it;
            const unsigned int ks = item % p.n_kstages;
            const unsigned int s = it % NS;
            unsigned char* xt = stages + (size_t)s * stage_bytes + Cfg::W_BYTES + Cfg::S_BYTES;
            const unsigned int k0 = ks * Cfg::SKE;
            const unsigned int kval = min((unsigned int)Cfg::SKE, p.K - k0);
            const unsigned int chunks = kval / 8;    // 16-byte chunks per token row
            const unsigned int total = chunks * p.M;
            for (unsigned int base = 0; base < total; base += 32 * 4)
            {
                uint4 v[4];
                unsigned int cidx[4], midx[4];
#pragma unroll
                for (int u = 0; u < 4; u++)
                {
                    const unsigned int q = base + u * 32 + lane;
                    midx[u] = q / chunks;
                    cidx[u] = q - midx[u] * chunks;
                    v[u] = make_uint4(0, 0, 0, 0);
                    if (q < total)
                    {
                        v[u] = *reinterpret_cast<const uint4*>(p.X + (size_t)midx[u] * p.ldx + k0 + cidx[u] * 8);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++)
                {
                    const unsigned int q = base + u * 32 + lane;
                    if (q < total)
                    {
                        uint4 o = v[u];
                        unsigned int c = cidx[u];
                        if (WT == DT_FP4)
                        {
                            // (x0..x7) -> (x0,x4)(x1,x5)(x2,x6)(x3,x7); chunks swizzled so that the four
                            // 16-byte reads of a lane (64 bytes apart across lanes) hit distinct banks
                            o.x = prmt(v[u].x, v[u].z, 0x5410u);
                            o.y = prmt(v[u].x, v[u].z, 0x7632u);
                            o.z = prmt(v[u].y, v[u].w, 0x5410u);
                            o.w = prmt(v[u].y, v[u].w, 0x7632u);
                            c ^= ((c >> 3) & 1u) << 1;
                        }
                        *reinterpret_cast<uint4*>(xt + midx[u] * Cfg::XPITCH + c * 16) = o;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) { mbar_arrive(full_bar + s); }
        };

        // Weights do not depend on the previous kernel of the stream: prefetch the first ring of
        // stages before waiting for it; activations only after.
        const unsigned int pre = min(NS, n_items);
        for (unsigned int it = 0; it < pre; it++) { issue_weights(it); }
        pdl_wait();
        for (unsigned int it = 0; it < pre; it++) { stage_x(it); }
        bool ok = true;
        unsigned int issued = pre;
        for (unsigned int it = pre; it < n_items; it++)
        {
            const unsigned int s = it % NS;
            if (sh_flags[0] != 0 || !mbar_wait_bounded(empty_bar + s, ((it / NS) - 1) & 1u))
            {
                ok = false;
                if (lane == 0)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    sh_flags[0] = 1;
                }
                break;
            }
            issue_weights(it);
            stage_x(it);
            issued = it + 1;
        }
        // Do not leave while copies are in flight.  Normally the consumers' last "empty" arrivals
        // prove that every stage has landed and been read; after an abort, wait (bounded) for the
        // outstanding stages to land instead.
        const unsigned int first = issued > NS ? issued - NS : 0;
        for (unsigned int it = first; it < issued; it++)
        {
            uint64_t* bar = ok ? empty_bar + (it % NS) : full_bar + (it % NS);
            if (!mbar_wait_bounded(bar, (it / NS) & 1u))
            {
                if (ok && sh_flags[0] == 0 && lane == 0) { atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY); }
                ok = false;
            }
        }
        return;
    }

    // =========================== consumer warps ===========================
    pdl_wait();
    const unsigned int g = lane >> 2, t = lane & 3;
    const unsigned int wr = warp / WK, wk = warp % WK;
    const unsigned int ctid = threadIdx.x;    // 0 .. 255: the consumer threads come first
    constexpr unsigned int TILE = R * 8 * MT;  // floats in one [token][row] tile
    bool ok = true;

    unsigned int it = 0;
    while (it < n_items)
    {
        const unsigned int item0 = items.beg + it;
        const unsigned int rb = item0 / p.n_kstages;
        const unsigned int ks0 = item0 % p.n_kstages;
        const unsigned int seg = min(p.n_kstages - ks0, n_items - it);    // items of this row block in my run
        const bool first_segment = (it == 0);

        float acc[RT][MT][2][4];
#pragma unroll
        for (int a = 0; a < RT; a++)
#pragma unroll
            for (int b = 0; b < MT; b++)
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int d = 0; d < 4; d++) { acc[a][b][c][d] = 0.f; }

        for (unsigned int j = 0; j < seg; j++, it++)
        {
            const unsigned int s = it % NS;
            if (ok && (sh_flags[0] != 0 || !mbar_wait_bounded(full_bar + s, (it / NS) & 1u)))
            {
                ok = false;
                if (sh_flags[0] == 0)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    sh_flags[0] = 1;
                }
            }
            if (!ok) { continue; }
            const unsigned int ks = ks0 + j;
            const unsigned int kval = min((unsigned int)Cfg::SKE, p.K - ks * Cfg::SKE);
            const unsigned int nsteps = kval / Cfg::KSTEP;
            const uint32_t st = smem_u32(stages + (size_t)s * stage_bytes);
            const uint32_t xt = st + Cfg::W_BYTES + Cfg::S_BYTES;
            for (unsigned int step = wk; step < nsteps; step += WK)
            {
                // ---- weights: rows (g, g+8) of each of my RT tiles, 16 bytes per row ----
                uint32_t A[RT][2][AREGS];
#pragma unroll
                for (int rt = 0; rt < RT; rt++)
                {
#pragma unroll
                    for (int h = 0; h < 2; h++)
                    {
                        const unsigned int row = (wr * RT + rt) * 16 + h * 8 + g;
                        const uint4 wv = lds128(st + row * Cfg::WPITCH + step * 64 + t * 16);
                        const uint32_t w[4] = { wv.x, wv.y, wv.z, wv.w };
                        if (WT == DT_FP4)
                        {
                            uint32_t m01[2];
                            fp4_block_multipliers(lds_u16(st + Cfg::W_BYTES + row * Cfg::SPITCH + step * 8 + t * 2), m01[0], m01[1]);
#pragma unroll
                            for (int i = 0; i < 4; i++)
                            {
                                uint32_t r4[4];
                                dequant_fp4x8(w[i], m01[i >> 1], r4);
#pragma unroll
                                for (int q = 0; q < 4; q++) { A[rt][h][(4 * i + q) % AREGS] = r4[q]; }
                            }
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 4; i++)
                            {
                                dequant_fp8x4<WT, SCALED>(w[i], p.w_scale, A[rt][h][(2 * i) % AREGS], A[rt][h][(2 * i + 1) % AREGS]);
                            }
                        }
                    }
                }
                // ---- activations of my token column and the MMAs ----
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
                {
                    const unsigned int token = mt * 8 + g;
                    const bool live = token < p.M;
                    if (WT == DT_FP4)
                    {
                        uint4 XB[4];
#pragma unroll
                        for (int i = 0; i < 4; i++)
                        {
                            unsigned int c = step * 16 + t * 4 + i;
                            c ^= ((c >> 3) & 1u) << 1;
                            XB[i] = live ? lds128(xt + token * Cfg::XPITCH + c * 16) : make_uint4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int rt = 0; rt < RT; rt++)
                        {
#pragma unroll
                            for (int i = 0; i < 4; i++)
                            {
                                mma_bf16_16816(acc[rt][mt][0], A[rt][0][(4 * i) % AREGS], A[rt][1][(4 * i) % AREGS],
                                    A[rt][0][(4 * i + 1) % AREGS], A[rt][1][(4 * i + 1) % AREGS], XB[i].x, XB[i].y);
                                mma_bf16_16816(acc[rt][mt][1], A[rt][0][(4 * i + 2) % AREGS], A[rt][1][(4 * i + 2) % AREGS],
                                    A[rt][0][(4 * i + 3) % AREGS], A[rt][1][(4 * i + 3) % AREGS], XB[i].z, XB[i].w);
                            }
                        }
                    }
                    else
                    {
                        const uint32_t xa = xt + token * Cfg::XPITCH + (step * 64 + t * 16) * 2;
                        const uint4 x0 = live ? lds128(xa) : make_uint4(0, 0, 0, 0);
                        const uint4 x1 = live ? lds128(xa + 16) : make_uint4(0, 0, 0, 0);
                        const uint32_t B[8] = { x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w };
#pragma unroll
                        for (int rt = 0; rt < RT; rt++)
                        {
#pragma unroll
                            for (int q = 0; q < 4; q++)
                            {
                                mma_bf16_16816(acc[rt][mt][q & 1], A[rt][0][2 * q], A[rt][1][2 * q], A[rt][0][2 * q + 1],
                                    A[rt][1][2 * q + 1], B[2 * q], B[2 * q + 1]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) { mbar_arrive(empty_bar + s); }
        }

        // ---- end of the segment: combine the k-split warps, then write or hand over ----
        float* myred = red + wk * TILE;
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
        consumer_bar_sync();
        const unsigned int n_out = p.M * R;    // live [token][row] entries
        const bool full = (ks0 == 0 && seg == p.n_kstages);
        const unsigned int n0 = rb * R;
        auto store_out = [&](unsigned int e, float v) {
            const unsigned int m = e / R, r = e - m * R;
            const unsigned int n = n0 + r;
            if (n < p.N)
            {
                uint16_t* y = p.Y + (long long)m * p.ldy_m + (long long)n * p.ldy_n;
                float o = p.alpha * (v * p.post_scale);
                if (p.beta != 0.f) { o += p.beta * bf16_bits_to_float(*y); }
                *y = __bfloat16_as_ushort(__float2bfloat16_rn(o));
            }
        };
        if (full)
        {
            if (ok)
            {
                for (unsigned int e = ctid; e < n_out; e += kConsumerWarps * 32)
                {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < WK; w++) { v += red[w * TILE + e]; }
                    store_out(e, v);
                }
            }
        }
        else
        {
            float* mine = p.partials + ((size_t)blockIdx.x * 2 + (first_segment ? 0 : 1)) * TILE;
            if (ok)
            {
                for (unsigned int e = ctid; e < n_out; e += kConsumerWarps * 32)
                {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < WK; w++) { v += red[w * TILE + e]; }
                    __stcg(mine + e, v);
                }
            }
            __threadfence();
            consumer_bar_sync();
            const unsigned int c_first = cta_of_item(rb * p.n_kstages, gridDim.x, p.total_items);
            const unsigned int c_last = cta_of_item(rb * p.n_kstages + p.n_kstages - 1, gridDim.x, p.total_items);
            if (ctid == 0)
            {
                unsigned int last = 0;
                if (ok && sh_flags[0] == 0)
                {
                    const unsigned int old = atomicAdd(p.counters + c_first, 1u);
                    last = (old == c_last - c_first) ? 1u : 0u;
                }
                sh_flags[1] = last;
            }
            consumer_bar_sync();
            if (sh_flags[1] != 0)
            {
                __threadfence();
                for (unsigned int e = ctid; e < n_out; e += kConsumerWarps * 32)
                {
                    float v = 0.f;
                    for (unsigned int c = c_first; c <= c_last; c++)
                    {
                        const unsigned int slot = (cta_items(c, gridDim.x, p.total_items).beg / p.n_kstages == rb) ? 0u : 1u;
                        v += __ldcg(p.partials + ((size_t)c * 2 + slot) * TILE + e);
                    }
                    store_out(e, v);
                }
                if (ctid == 0) { p.counters[c_first] = 0; }
            }
        }
        consumer_bar_sync();    // `red` and sh_flags[1] are reused by the next segment
    }
}

// ---- plain kernel: any shape, stride or alignment ----------------------------------------------------
// One warp per output feature, eight tokens at a time, one element per lane per step; every
// weight is dequantised exactly as the reference's conversion kernels do it.
template <int WT>
__global__ void __launch_bounds__(256) linear_wq_plain_kernel(const GemvParams p)
{
    const unsigned int lane = threadIdx.x & 31;
    const unsigned long long n = (unsigned long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= p.N) { return; }
    for (unsigned int m0 = 0; m0 < p.M; m0 += 8)
    {
        float acc[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
        const unsigned int mcount = min(8u, p.M - m0);
        for (unsigned int k = lane; k < p.K; k += 32)
        {
            const size_t e = (size_t)n * p.ldw + k;
            float wf;
            if (WT == DT_FP4)
            {
                const uint32_t b = p.W[e >> 1];
                const uint32_t nib = (e & 1) ? (b >> 4) : (b & 0xFu);
                const float sc = p.blk ? e4m3_to_float(p.blk[e / 16]) : p.w_scale;
                wf = fp4_to_float(nib) * sc;
            }
            else { wf = decode_fp8<WT>(p.W[e]) * p.w_scale; }
            wf = bf16_bits_to_float(float_to_bf16_bits_ref(wf));
            for (unsigned int mm = 0; mm < mcount; mm++) { acc[mm] += wf * bf16_bits_to_float(p.X[(size_t)(m0 + mm) * p.ldx + k]); }
        }
        for (unsigned int mm = 0; mm < mcount; mm++)
        {
            float v = acc[mm];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { v += __shfl_xor_sync(0xFFFFFFFFu, v, o); }
            if (lane == 0)
            {
                uint16_t* y = p.Y + (long long)(m0 + mm) * p.ldy_m + (long long)n * p.ldy_n;
                float o = p.alpha * v;
                if (p.beta != 0.f) { o += p.beta * bf16_bits_to_float(*y); }
                *y = __bfloat16_as_ushort(__float2bfloat16_rn(o));
            }
        }
    }
}

}    // namespace b200
