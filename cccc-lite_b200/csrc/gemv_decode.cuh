// Decode-side quantized-weight linear (M <= 32 tokens): an HBM-bound GEMV.
//
// One persistent CTA per SM.  A producer lane streams the weight bytes (and FP4 block scales)
// and the matching slice of the BF16 activations from HBM/L2 into a shared-memory ring with
// tiled TMA copies (cp.async.bulk.tensor + mbarrier): one copy per operand per stage, because
// the copy engine takes on the order of a hundred cycles per instruction whatever its size.
// Eight consumer warps dequantise to BF16 in registers and feed m16n8k16 BF16 MMAs with FP32
// accumulators: the weight tile is the A operand (16 output features x 16 k), the tokens are
// the 8 columns of B.  The k order inside a fragment is permuted so that every lane converts
// the 16 bytes it loaded itself; the activation fragment is loaded in the same order.
// Under programmatic dependent launch the weight prefetch of a linear is issued before it waits
// for the previous kernel of the stream; activations, outputs and scratch are touched only after.
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

#include <cuda.h>

namespace b200
{

constexpr int kMaxGroup = 3;    // linears that may share one launch (same activations, same K)

// One linear of a grouped launch.  Its row blocks are [rb_begin, next segment's rb_begin).
struct GemvSeg
{
    const uint8_t* W;
    const uint8_t* blk;
    uint16_t* Y;
    unsigned int N, ldw;
    unsigned int rb_begin;
    long long ldy_m, ldy_n;
    float w_scale, alpha, beta, post_scale;
};

// The exchange of a row-parallel (K-split) shard fused into the kernel's epilogue: every rank's
// receive area [2 sets][world sources][n_max floats] and flag area [2 sets][kArMaxRowBlocks][world]
// as mapped into this process (symmetric memory), and this rank's call counters.
// One counter per exchange area numbers the calls: seq[0] = fused calls completed on this area,
// seq[1] = CTAs of the running call that have finished (the last one to finish resets it and
// advances seq[0]).  The call number c = seq[0] + 1 is the value published in the flags and its
// low bit picks the slot set, so the two sets alternate call by call whatever the calls' shapes
// are: a rank can only reach call c + 1 after every peer has published flags of call c, that is
// after every peer has finished reading the slots of call c - 1, which are the ones call c + 1
// overwrites.
constexpr int kArMaxWorld = 8;
constexpr int kArMaxRowBlocks = 2048;
struct GemvAllReduce
{
    float* peer_recv[kArMaxWorld];
    unsigned int* peer_flag[kArMaxWorld];
    unsigned int* seq;        // local: [0] completed calls, [1] finished CTAs of the running call
    unsigned int n_max;
    int rank, world;          // world <= 1: no exchange
};

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
    unsigned int out_f32;       // 0: Y is BF16; 1: Y holds float32 (partial sums of a row-parallel shard); 2: Y is BF16 and
                                // alpha * product is rounded to BF16 before beta * Y is added (the reference's linear
                                // followed by its residual add, two BF16 tensors)
    unsigned int n_row_blocks, n_kstages, total_items;
    unsigned int gran;          // items are dealt to CTAs in groups of `gran`: 1 = stream-K, n_kstages = whole row blocks
    unsigned int n_stages;      // ring depth
    unsigned int n_seg;         // linears in this launch (1 unless grouped); the fields above describe the
    GemvSeg seg[kMaxGroup];     // first one, seg[] all of them (unused entries have rb_begin = 0xFFFFFFFF)
    GemvAllReduce ar;           // fused all-reduce of a row-parallel shard (single linear, beta = 0)
};

constexpr unsigned long long kWaitLimitNs = 2000000000ull;    // 2 s

enum : unsigned int
{
    ST_OK = 0,
    ST_TIMEOUT_FULL = 1,
    ST_TIMEOUT_EMPTY = 2,
    ST_TIMEOUT_FIXUP = 3,
    ST_TIMEOUT_PEER = 4
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
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
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
// L2 eviction policy of the streamed weights: each byte is read once, so it should be the first to go.
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <int THREADS>
__device__ __forceinline__ void consumer_bar_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}

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
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
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
// WR  : consumer warps along N
// WK  : consumer warps along k (they split the k steps of a stage)
// SKS : k steps per stage; one k step is 64 bytes of every weight row
// XB  : token rows in the activation box (2: M <= 2, plain layout; else 8*MT, 128-byte swizzle)
// OCC : CTAs that may share an SM (2 lets the next kernel of the stream prefetch its weights
//       while this one finishes)
//
// Shared-memory layout of a stage, each part written by ONE tiled TMA copy:
//   weights  [k step][row][64 B]            rows 2q and 2q+1 are adjacent 64-byte runs, so the eight
//                                           lanes of a 128-bit read phase cover 128 contiguous bytes
//   scales   [k step pair][row][16 B]       FP4 only: 8 E4M3 bytes per row per k step
//   acts     [128-byte slab][token][128 B]  64 BF16 per slab row, 16-byte chunks XOR-swizzled by
//                                           (token & 7) when XB is a multiple of 8
template <int WT_, int MT_, int RT_, int WR_, int WK_, int SKS_, int XB_, int OCC_>
struct GemvCfg
{
    static constexpr int WT = WT_, MT = MT_, RT = RT_, WR = WR_, WK = WK_, SKS = SKS_, XB = XB_, OCC = OCC_;
    static constexpr int NCW = WR * WK;                           // consumer warps
    static constexpr int THREADS = 32 * (NCW + 1);                // + the producer warp
    static constexpr int R = 16 * RT * WR;                        // rows per row block
    static constexpr int KSTEP = (WT == DT_FP4) ? 128 : 64;       // elements per k step
    static constexpr int SKE = KSTEP * SKS;                       // elements per stage along k
    static constexpr int XSLABS = SKE / 64;                       // 128-byte activation slabs per stage
    static constexpr bool XSWZ = (XB % 8) == 0;
    static constexpr int W_BYTES = SKS * R * 64;
    static constexpr int S_BYTES = (WT == DT_FP4) ? (SKS / 2) * R * 16 : 0;
    static constexpr int X_BYTES = XSLABS * XB * 128;
    static constexpr int STAGE_BYTES = ((W_BYTES + S_BYTES + X_BYTES + 1023) / 1024) * 1024;
    static constexpr int X_OFFSET = ((W_BYTES + S_BYTES + 1023) / 1024) * 1024;    // swizzle needs 1 KB alignment
    static constexpr int RED_BYTES = WK * R * 8 * MT * 4;
    static constexpr int HEADER_BYTES = 1024;                     // barriers and flags
    static constexpr int kMaxStages = 16;
    static_assert(WT != DT_FP4 || (SKS % 2) == 0, "FP4 stages hold whole scale chunks");
    static_assert(X_OFFSET + X_BYTES <= STAGE_BYTES + 1024, "layout");
};

struct ItemRange
{
    unsigned int beg, end;
};
// CTA c owns the item groups [floor(c*G/grid), floor((c+1)*G/grid)), G = total/gran groups.
__host__ __device__ inline ItemRange cta_items(unsigned int cta, unsigned int grid, unsigned int total, unsigned int gran)
{
    const unsigned long long groups = total / gran;
    ItemRange r;
    r.beg = (unsigned int)(((unsigned long long)cta * groups) / grid) * gran;
    r.end = (unsigned int)(((unsigned long long)(cta + 1) * groups) / grid) * gran;
    return r;
}
// The CTA whose run contains item i: the largest c with floor(c*G/grid) <= i/gran.
__host__ __device__ inline unsigned int cta_of_item(unsigned int i, unsigned int grid, unsigned int total, unsigned int gran)
{
    const unsigned long long groups = total / gran;
    return (unsigned int)((((unsigned long long)(i / gran) + 1) * grid - 1) / groups);
}

// 3-D tiled TMA load, completion counted on an mbarrier.  c0 is always 0 here (the inner extent is
// one whole 16-byte-aligned run), so the 16-byte rule on the inner coordinate holds by construction.
__device__ __forceinline__ void tma_load_3d_hint(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar,
    uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], "
        "[%5], %6;" ::"r"(smem_u32(dst)),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}

// One k step (64 bytes of every weight row of the stage) of one consumer warp: dequantise the rows of
// its RT row tiles, load its activation fragments, issue the MMAs.  st: shared-memory address of the
// stage's weights (scales behind them); xt: address of the activation slabs of this stage, laid out
// [128-byte slab][token][128 B]; wr: this warp's position along the rows; g, t: lane >> 2, lane & 3.
// paired: the stage holds two 16-row boxes of two different matrices one after the other (rows 0-15 and
// 16-31 of the block) instead of one 32-row box, each laid out [k step][16 rows][64 B].
template <class Cfg>
__device__ __forceinline__ uint32_t stage_row_addr(const uint32_t st, const unsigned int step, const unsigned int row, const bool paired)
{
    return paired ? st + (row >> 4) * (Cfg::SKS * 16 * 64) + (step * 16 + (row & 15u)) * 64 : st + (step * Cfg::R + row) * 64;
}
template <class Cfg>
__device__ __forceinline__ uint32_t stage_scale_addr(const uint32_t st, const unsigned int step, const unsigned int row, const bool paired)
{
    return paired ? st + Cfg::W_BYTES + (row >> 4) * ((Cfg::SKS / 2) * 16 * 16) + ((step >> 1) * 16 + (row & 15u)) * 16 + (step & 1u) * 8
                  : st + Cfg::W_BYTES + ((step >> 1) * Cfg::R + row) * 16 + (step & 1u) * 8;
}

template <class Cfg, bool SCALED>
__device__ __forceinline__ void gemv_k_step(float (&acc)[Cfg::RT][Cfg::MT][2][4], const uint32_t st, const uint32_t xt,
    const unsigned int step, const unsigned int wr, const unsigned int g, const unsigned int t, const float w_scale,
    const bool paired = false, const float w_scale_second = 1.0f)
{
    constexpr int WT = Cfg::WT, MT = Cfg::MT, RT = Cfg::RT, R = Cfg::R;
    constexpr int AREGS = (WT == DT_FP4) ? 16 : 8;    // bf16x2 registers per weight row per k step
    // ---- weights: rows (g, g+8) of each of my RT tiles, 16 bytes per row ----
    uint32_t A[RT][2][AREGS];
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
    {
#pragma unroll
        for (int h = 0; h < 2; h++)
        {
            const unsigned int row = (wr * RT + rt) * 16 + h * 8 + g;
            const uint4 wv = lds128(stage_row_addr<Cfg>(st, step, row, paired) + t * 16);
            const uint32_t w[4] = { wv.x, wv.y, wv.z, wv.w };
            if (WT == DT_FP4)
            {
                uint32_t m01[2];
                fp4_block_multipliers(lds_u16(stage_scale_addr<Cfg>(st, step, row, paired) + t * 2), m01[0], m01[1]);
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
                    dequant_fp8x4<WT, SCALED>(w[i], (paired && rt == 1) ? w_scale_second : w_scale, A[rt][h][(2 * i) % AREGS], A[rt][h][(2 * i + 1) % AREGS]);
                }
            }
        }
    }
    // ---- activations of my token column and the MMAs ----
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
    {
        const unsigned int token = mt * 8 + g;
        // token rows past M were zero-filled by the TMA; rows past the box do not exist
        const bool live = token < (unsigned int)Cfg::XB;
        const unsigned int swz = Cfg::XSWZ ? (token & 7u) : 0u;
        if (WT == DT_FP4)
        {
            uint4 XBr[4];
            const uint32_t xrow = xt + ((step * 2 + (t >> 1)) * Cfg::XB + token) * 128;
#pragma unroll
            for (int i = 0; i < 4; i++)
            {
                // eight activations (x0..x7) -> (x0,x4)(x1,x5)(x2,x6)(x3,x7), the pairing of the
                // dequantised nibbles
                const unsigned int c = (t & 1u) * 4 + i;
                const uint4 v = live ? lds128(xrow + ((c ^ swz) << 4)) : make_uint4(0, 0, 0, 0);
                XBr[i].x = prmt(v.x, v.z, 0x5410u);
                XBr[i].y = prmt(v.x, v.z, 0x7632u);
                XBr[i].z = prmt(v.y, v.w, 0x5410u);
                XBr[i].w = prmt(v.y, v.w, 0x7632u);
            }
#pragma unroll
            for (int rt = 0; rt < RT; rt++)
            {
#pragma unroll
                for (int i = 0; i < 4; i++)
                {
                    mma_bf16_16816(acc[rt][mt][0], A[rt][0][(4 * i) % AREGS], A[rt][1][(4 * i) % AREGS],
                        A[rt][0][(4 * i + 1) % AREGS], A[rt][1][(4 * i + 1) % AREGS], XBr[i].x, XBr[i].y);
                    mma_bf16_16816(acc[rt][mt][1], A[rt][0][(4 * i + 2) % AREGS], A[rt][1][(4 * i + 2) % AREGS],
                        A[rt][0][(4 * i + 3) % AREGS], A[rt][1][(4 * i + 3) % AREGS], XBr[i].z, XBr[i].w);
                }
            }
        }
        else
        {
            const uint32_t xrow = xt + (step * Cfg::XB + token) * 128;
            const uint4 x0 = live ? lds128(xrow + (((2 * t) ^ swz) << 4)) : make_uint4(0, 0, 0, 0);
            const uint4 x1 = live ? lds128(xrow + (((2 * t + 1) ^ swz) << 4)) : make_uint4(0, 0, 0, 0);
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

// The same k step on the CUDA cores, for one or two tokens.  On B200 the legacy mma.sync path issues
// one m16n8k16 per ~8 clocks per SM whatever the token count, which caps a GEMV at ~32 weight bytes
// per clock per SM; with one or two tokens plain FP32 fused multiply-adds do better: every lane
// widens the 16 bytes it loaded to FP32 (exact: the decoded weight IS the BF16 operand when no
// per-weight multiplier applies, and table * block scale for FP4) and accumulates w * x per token in
// FP32, which is what the tensor core does with the BF16 operands.  Only for weights that need no
// per-weight multiplier (per-tensor scale a power of two, folded in after the sums, or FP4 block
// scales).  acc[rt][h][m]: row (rt*16 + h*8 + g) of this warp's rows, token m, this lane's k slice.
template <class Cfg, int NT>
__device__ __forceinline__ void gemv_k_step_fma(float (&acc)[Cfg::RT][2][NT], const uint32_t st, const uint32_t xt,
    const unsigned int step, const unsigned int wr, const unsigned int g, const unsigned int t, const bool paired = false)
{
    constexpr int WT = Cfg::WT, RT = Cfg::RT, R = Cfg::R;
    constexpr int NX = (WT == DT_FP4) ? 32 : 16;    // activations per lane and k step
    static_assert(!Cfg::XSWZ, "the CUDA-core k step reads the unswizzled two-token layout");
    float xf[NT][NX];
#pragma unroll
    for (int m = 0; m < NT; m++)
    {
        const uint32_t xrow = (WT == DT_FP4) ? xt + ((step * 2 + (t >> 1)) * Cfg::XB + m) * 128 + (t & 1u) * 64
                                             : xt + (step * Cfg::XB + m) * 128 + t * 32;
#pragma unroll
        for (int c = 0; c < NX / 8; c++)
        {
            const uint4 v = lds128(xrow + c * 16);
            const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
            for (int i = 0; i < 4; i++)
            {
                xf[m][c * 8 + 2 * i] = __uint_as_float(w[i] << 16);
                xf[m][c * 8 + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
        }
    }
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
    {
#pragma unroll
        for (int h = 0; h < 2; h++)
        {
            const unsigned int row = (wr * RT + rt) * 16 + h * 8 + g;
            const uint4 wv = lds128(stage_row_addr<Cfg>(st, step, row, paired) + t * 16);
            const uint32_t w[4] = { wv.x, wv.y, wv.z, wv.w };
            if (WT == DT_FP4)
            {
                // two blocks of 16 nibbles, one E4M3 multiplier each; table * multiplier is exact in FP16
                const uint32_t two = lds_u16(stage_scale_addr<Cfg>(st, step, row, paired) + t * 2);
                uint32_t s2[2];
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2[0]) : "h"((uint16_t)((two & 0xFFu) * 0x0101u)));
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2[1]) : "h"((uint16_t)((two >> 8) * 0x0101u)));
#pragma unroll
                for (int i = 0; i < 16; i++)
                {
                    const uint16_t b = (uint16_t)((w[i >> 2] >> (8 * (i & 3))) & 0xFFu);
                    uint32_t h2, p2;
                    asm("{\n\t.reg .b8 lo, hi;\n\tmov.b16 {lo, hi}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, lo;\n\t}" : "=r"(h2) : "h"(b));
                    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(p2) : "r"(h2), "r"(s2[i >> 3]));
                    const float2 f = half2_bits_to_float2(p2);
#pragma unroll
                    for (int m = 0; m < NT; m++)
                    {
                        acc[rt][h][m] = __fmaf_rn(f.x, xf[m][2 * i], acc[rt][h][m]);
                        acc[rt][h][m] = __fmaf_rn(f.y, xf[m][2 * i + 1], acc[rt][h][m]);
                    }
                }
            }
            else
            {
#pragma unroll
                for (int i = 0; i < 4; i++)
                {
                    uint32_t h01, h23;
                    if (WT == DT_E5M2)
                    {
                        h01 = prmt(w[i], 0u, 0x1404u);
                        h23 = prmt(w[i], 0u, 0x3424u);
                    }
                    else
                    {
                        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"((uint16_t)(w[i] & 0xFFFFu)));
                        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"((uint16_t)(w[i] >> 16)));
                    }
                    const float2 f01 = half2_bits_to_float2(h01);
                    const float2 f23 = half2_bits_to_float2(h23);
#pragma unroll
                    for (int m = 0; m < NT; m++)
                    {
                        acc[rt][h][m] = __fmaf_rn(f01.x, xf[m][4 * i], acc[rt][h][m]);
                        acc[rt][h][m] = __fmaf_rn(f01.y, xf[m][4 * i + 1], acc[rt][h][m]);
                        acc[rt][h][m] = __fmaf_rn(f23.x, xf[m][4 * i + 2], acc[rt][h][m]);
                        acc[rt][h][m] = __fmaf_rn(f23.y, xf[m][4 * i + 3], acc[rt][h][m]);
                    }
                }
            }
        }
    }
}

// ---- the kernel ------------------------------------------------------------------------------------
template <class Cfg, bool SCALED>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::OCC)
    gemv_wq_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
        const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmS1,
        const __grid_constant__ CUtensorMap tmW2, const __grid_constant__ CUtensorMap tmS2,
        const __grid_constant__ CUtensorMap tmX, const GemvParams p)
{
    constexpr int WT = Cfg::WT, MT = Cfg::MT, RT = Cfg::RT, WK = Cfg::WK, R = Cfg::R;
    constexpr int kConsumerWarps = Cfg::NCW;
    constexpr int CT = Cfg::NCW * 32;    // consumer threads
    constexpr int AREGS = (WT == DT_FP4) ? 16 : 8;    // bf16x2 registers per weight row per k step
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = full_bar + Cfg::kMaxStages;
    // sh_flags[0] = abort, [1] = "this CTA reduces the row block", [2] = exchange sequence number, [3] = a peer timed out
    volatile unsigned int* sh_flags = reinterpret_cast<volatile unsigned int*>(smem + 2 * Cfg::kMaxStages * 8);
    unsigned char* stages = smem + Cfg::HEADER_BYTES;
    float* red = reinterpret_cast<float*>(smem + Cfg::HEADER_BYTES + (size_t)p.n_stages * Cfg::STAGE_BYTES);
    const unsigned int NS = p.n_stages;

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const ItemRange items = cta_items(blockIdx.x, gridDim.x, p.total_items, p.gran);
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
        // =========================== producer: one elected lane ===========================
        if (lane != 0) { return; }
        const uint64_t pol_stream = l2_policy_evict_first();
        auto issue_weights = [&](unsigned int it) {
            const unsigned int item = items.beg + it;
            const unsigned int rb = item / p.n_kstages, ks = item % p.n_kstages;
            const unsigned int s = it % NS;
            unsigned char* st = stages + (size_t)s * Cfg::STAGE_BYTES;
            // which linear of the group this row block belongs to, and its row block there
            const unsigned int j = (rb >= p.seg[1].rb_begin ? 1u : 0u) + (rb >= p.seg[2].rb_begin ? 1u : 0u);
            const int row0 = (int)((rb - p.seg[j].rb_begin) * R);
            const CUtensorMap* mw = j == 0 ? &tmW : (j == 1 ? &tmW1 : &tmW2);
            const CUtensorMap* ms = j == 0 ? &tmS : (j == 1 ? &tmS1 : &tmS2);
            mbar_expect_tx(full_bar + s, Cfg::W_BYTES + Cfg::S_BYTES);
            tma_load_3d_hint(st, mw, 0, row0, (int)(ks * Cfg::SKS), full_bar + s, pol_stream);
            if (WT == DT_FP4) { tma_load_3d_hint(st + Cfg::W_BYTES, ms, 0, row0, (int)(ks * (Cfg::SKS / 2)), full_bar + s, pol_stream); }
        };
        auto issue_acts = [&](unsigned int it) {
            const unsigned int item = items.beg + it;
            const unsigned int ks = item % p.n_kstages;
            const unsigned int s = it % NS;
            unsigned char* st = stages + (size_t)s * Cfg::STAGE_BYTES;
            mbar_expect_tx(full_bar + s, Cfg::X_BYTES);
            tma_load_3d(st + Cfg::X_OFFSET, &tmX, 0, 0, (int)(ks * Cfg::XSLABS), full_bar + s);
            mbar_arrive(full_bar + s);
        };
        // Weights do not depend on the previous kernel of the stream: prefetch the first ring of
        // stages before waiting for it; activations only after.
        const unsigned int pre = min(NS, n_items);
        for (unsigned int it = 0; it < pre; it++) { issue_weights(it); }
        pdl_wait();
        for (unsigned int it = 0; it < pre; it++) { issue_acts(it); }
        bool ok = true;
        unsigned int issued = pre;
        for (unsigned int it = pre; it < n_items; it++)
        {
            const unsigned int s = it % NS;
            if (sh_flags[0] != 0 || !mbar_wait_bounded(empty_bar + s, ((it / NS) - 1) & 1u))
            {
                ok = false;
                atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                sh_flags[0] = 1;
                break;
            }
            issue_weights(it);
            issue_acts(it);
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
                if (ok && sh_flags[0] == 0) { atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY); }
                ok = false;
            }
        }
        return;
    }

    // =========================== consumer warps ===========================
    pdl_wait();
    const unsigned int g = lane >> 2, t = lane & 3;
    const unsigned int wr = warp / WK, wk = warp % WK;
    const unsigned int ctid = threadIdx.x;    // the consumer threads come first
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
        const unsigned int lj = (rb >= p.seg[1].rb_begin ? 1u : 0u) + (rb >= p.seg[2].rb_begin ? 1u : 0u);
        const GemvSeg& L = p.seg[lj];    // the linear this row block belongs to
        const float w_scale = L.w_scale;

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
            const unsigned int nsteps = kval / Cfg::KSTEP;    // beyond K the TMA fills zeros; skip them
            const uint32_t st = smem_u32(stages + (size_t)s * Cfg::STAGE_BYTES);
            const uint32_t xt = st + Cfg::X_OFFSET;
            auto do_step = [&](unsigned int step) { gemv_k_step<Cfg, SCALED>(acc, st, xt, step, wr, g, t, w_scale); };
            constexpr int SPW = (Cfg::SKS + WK - 1) / WK;    // k steps per warp in a full stage
            if (nsteps == (unsigned int)Cfg::SKS)
            {
                // full stage: unrolled, so that the loads of all my steps are in flight together
#pragma unroll
                for (int u = 0; u < SPW; u++)
                {
                    const unsigned int step = wk + u * WK;
                    if ((Cfg::SKS % WK) == 0 || step < (unsigned int)Cfg::SKS) { do_step(step); }
                }
            }
            else
            {
                for (unsigned int step = wk; step < nsteps; step += WK) { do_step(step); }
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
        consumer_bar_sync<CT>();
        const unsigned int n_out = p.M * R;    // live [token][row] entries
        const bool full = (ks0 == 0 && seg == p.n_kstages);
        const unsigned int n0 = (rb - L.rb_begin) * R;
        auto store_out = [&](unsigned int e, float v) {
            const unsigned int m = e / R, r = e - m * R;
            const unsigned int n = n0 + r;
            if (n < L.N)
            {
                const long long yi = (long long)m * L.ldy_m + (long long)n * L.ldy_n;
                float o = L.alpha * (v * L.post_scale);
                if (p.out_f32 == 1u)
                {
                    float* y = reinterpret_cast<float*>(L.Y) + yi;
                    if (L.beta != 0.f) { o += L.beta * *y; }
                    *y = o;
                }
                else
                {
                    uint16_t* y = L.Y + yi;
                    if (L.beta != 0.f) { o = (p.out_f32 == 2u ? __bfloat162float(__float2bfloat16_rn(o)) : o) + L.beta * bf16_bits_to_float(*y); }
                    *y = __bfloat16_as_ushort(__float2bfloat16_rn(o));
                }
            }
        };
        // Row-parallel shard with the exchange fused in: push this row block's FP32 partial into every
        // rank's receive area (own rank included), publish the row block's sequence number to every
        // rank, wait (bounded) for all ranks' numbers, add the slots in rank order and round once.
        // Every rank computes the same bits, the bits of the separate linear + all-reduce calls.
        auto exchange_out = [&](auto value_of) {
            const int W_ = p.ar.world, me = p.ar.rank;
            if (ctid == 0)
            {
                // seq[0] only moves when the last CTA of a call has finished, so every CTA of this
                // call reads the same number here
                sh_flags[2] = __ldcg(p.ar.seq) + 1;
                sh_flags[3] = 0;
            }
            consumer_bar_sync<CT>();
            const unsigned int seq = sh_flags[2], set = seq & 1u;
            const size_t slot = ((size_t)set * W_ + me) * p.ar.n_max;
            for (unsigned int e = ctid; e < n_out; e += CT)
            {
                const unsigned int m = e / R, r = e - m * R, n = n0 + r;
                if (n < L.N)
                {
                    const float o = L.alpha * (value_of(e) * L.post_scale);
                    const size_t idx = slot + (size_t)m * L.N + n;
                    for (int rr = 0; rr < W_; rr++) { p.ar.peer_recv[rr][idx] = o; }
                }
            }
            // The barrier orders every thread's peer stores before the flag stores of threads 0..world-1,
            // whose release at system scope is cumulative over them: no fence per storing thread.
            consumer_bar_sync<CT>();
            if ((int)ctid < W_)
            {
                st_release_sys(p.ar.peer_flag[ctid] + ((size_t)set * kArMaxRowBlocks + rb) * W_ + me, seq);
                const unsigned int* f = p.ar.peer_flag[me] + ((size_t)set * kArMaxRowBlocks + rb) * W_ + ctid;
                const unsigned long long t0 = global_timer_ns();
                unsigned int spins = 0;
                while (ld_acquire_sys(f) != seq)
                {
                    if ((++spins & 0xFFu) == 0 && global_timer_ns() - t0 > 1000000000ull)
                    {
                        atomicMax(p.status, (unsigned int)ST_TIMEOUT_PEER);    // a peer never arrived: report, do not hang
                        sh_flags[3] = 1;
                        break;
                    }
                }
            }
            consumer_bar_sync<CT>();
            if (sh_flags[3] == 0)
            {
                const float* mine = p.ar.peer_recv[me] + (size_t)set * W_ * p.ar.n_max;
                for (unsigned int e = ctid; e < n_out; e += CT)
                {
                    const unsigned int m = e / R, r = e - m * R, n = n0 + r;
                    if (n < L.N)
                    {
                        const size_t idx = (size_t)m * L.N + n;
                        float acc = __ldcv(mine + idx);    // peers wrote these: never from L1
                        for (int rr = 1; rr < W_; rr++) { acc += __ldcv(mine + (size_t)rr * p.ar.n_max + idx); }
                        const long long yi = (long long)m * L.ldy_m + (long long)n * L.ldy_n;
                        if (p.out_f32 == 1u) { reinterpret_cast<float*>(L.Y)[yi] = acc; }
                        else { L.Y[yi] = __bfloat16_as_ushort(__float2bfloat16_rn(acc)); }
                    }
                }
            }
        };
        const bool exchange = p.ar.world > 1;
        if (full)
        {
            if (ok)
            {
                auto value_of = [&](unsigned int e) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < WK; w++) { v += red[w * TILE + e]; }
                    return v;
                };
                if (exchange) { exchange_out(value_of); }
                else
                {
                    for (unsigned int e = ctid; e < n_out; e += CT) { store_out(e, value_of(e)); }
                }
            }
        }
        else
        {
            float* mine = p.partials + ((size_t)blockIdx.x * 2 + (first_segment ? 0 : 1)) * TILE;
            if (ok)
            {
                for (unsigned int e = ctid; e < n_out; e += CT)
                {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < WK; w++) { v += red[w * TILE + e]; }
                    __stcg(mine + e, v);
                }
            }
            // The barrier orders every thread's partial stores before thread 0's fence, which is
            // cumulative over them (one fence per CTA, not one per thread, on either side).
            consumer_bar_sync<CT>();
            const unsigned int c_first = cta_of_item(rb * p.n_kstages, gridDim.x, p.total_items, p.gran);
            const unsigned int c_last = cta_of_item(rb * p.n_kstages + p.n_kstages - 1, gridDim.x, p.total_items, p.gran);
            if (ctid == 0)
            {
                unsigned int last = 0;
                if (ok && sh_flags[0] == 0)
                {
                    __threadfence();
                    const unsigned int old = atomicAdd(p.counters + c_first, 1u);
                    last = (old == c_last - c_first) ? 1u : 0u;
                    __threadfence();
                }
                sh_flags[1] = last;
            }
            consumer_bar_sync<CT>();
            if (sh_flags[1] != 0)
            {
                auto value_of = [&](unsigned int e) {
                    float v = 0.f;
                    for (unsigned int c = c_first; c <= c_last; c++)
                    {
                        const unsigned int slot = (cta_items(c, gridDim.x, p.total_items, p.gran).beg / p.n_kstages == rb) ? 0u : 1u;
                        v += __ldcg(p.partials + ((size_t)c * 2 + slot) * TILE + e);
                    }
                    return v;
                };
                if (exchange) { exchange_out(value_of); }
                else
                {
                    for (unsigned int e = ctid; e < n_out; e += CT) { store_out(e, value_of(e)); }
                }
                if (ctid == 0) { p.counters[c_first] = 0; }
            }
        }
        consumer_bar_sync<CT>();    // `red` and sh_flags[1] are reused by the next segment
    }
    if (p.ar.world > 1 && ctid == 0)
    {
        // this CTA has finished the call; the last one to do so closes the call on this exchange area
        const unsigned int c = __ldcg(p.ar.seq) + 1;
        __threadfence();
        if (atomicAdd(p.ar.seq + 1, 1u) == gridDim.x - 1)
        {
            p.ar.seq[1] = 0;
            __stcg(p.ar.seq, c);
        }
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
                const long long yi = (long long)(m0 + mm) * p.ldy_m + (long long)n * p.ldy_n;
                float o = p.alpha * v;
                if (p.out_f32 == 1u)
                {
                    float* y = reinterpret_cast<float*>(p.Y) + yi;
                    if (p.beta != 0.f) { o += p.beta * *y; }
                    *y = o;
                }
                else
                {
                    uint16_t* y = p.Y + yi;
                    if (p.beta != 0.f) { o = (p.out_f32 == 2u ? __bfloat162float(__float2bfloat16_rn(o)) : o) + p.beta * bf16_bits_to_float(*y); }
                    *y = __bfloat16_as_ushort(__float2bfloat16_rn(o));
                }
            }
        }
    }
}

}    // namespace b200
