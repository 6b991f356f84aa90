// Prefill-side quantized-weight linear (M > 32 tokens): a dense contraction on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA computes a tile of 128 or 256 output features x up to 256 tokens over the whole K range.
// With 128 features two CTAs share an SM (each owns part of the 512 TMEM columns), so one CTA's
// epilogue overlaps the other's main loop; the 256-feature tile (one CTA per SM, all 512 TMEM
// columns, three stages) lets two weight tiles share each activation tile.  Large problems take the
// CTA-pair kernel (gemm_prefill_pair.cuh); this one serves those with too few tiles for it.
// Per 64-wide k block:
//   * a TMA lane copies the BF16 activation tile [256 (or 128) tokens][64 k] into shared memory with the
//     128-byte swizzle (token rows past M are zero-filled by the TMA),
//   * eight warps load the quantised weight tile [128 features][64 k] from global memory (16 bytes
//     per thread, prefetched two k blocks ahead), dequantise it to BF16 exactly as the reference's
//     conversion kernels do, store it into the A-operand stage in the same K-major 128-byte swizzled
//     layout the UMMA descriptor names, convert the next block while those stores land, then fence,
//   * the MMA warp (one elected lane issuing) issues four tcgen05.mma (M=128, N=tokens rounded up to
//     16, K=16) per 128 features and commits to the barrier that frees the stage.
// After the last k block the eight warps read the accumulator from TMEM (tcgen05.ld, one TMEM lane =
// one output feature per thread) and apply alpha; BF16 output with contiguous features goes through
// a tile in the idle stage memory and one TMA store (which clips ragged edges), anything else (beta,
// FP32 output, transposed Y) is stored from registers.  A launch may hold up to three linears that
// share their activations: blockIdx.y walks their feature tiles.
// Every wait is bounded; on expiry the status word is raised and the CTA drains, waits (bounded)
// for its copies in flight, frees its TMEM columns and returns.
#pragma once

#include <atomic>

#include "common.cuh"
#include "gemv_decode.cuh"
#include "tensor_map.cuh"

#include <cmath>
#include <cstring>

namespace b200
{

constexpr int PF_BM = 128;          // output features per tile (UMMA M)
constexpr int PF_BN_MAX = 512;      // tokens per tile: 512 (two N=256 UMMAs per A tile), 256, or 128
constexpr int PF_BK = 64;           // k per block: one 128-byte swizzle row of BF16
constexpr int PF_MAX_STAGES = 3;
constexpr int PF_DQ_WARPS = 8;      // dequantise, then epilogue
constexpr int PF_THREADS = 32 * (PF_DQ_WARPS + 2);    // + TMA warp + MMA warp
__host__ __device__ constexpr int pf_a_bytes(int fh) { return fh * PF_BM * PF_BK * 2; }    // 16 KB per 128 features
// two CTAs of the 128-feature tiles share an SM: 2 x 2 x 48 KB at 256 tokens, 2 x 3 x 32 KB at 128 tokens
__host__ __device__ constexpr int pf_stages(int bn, int fh) { return (fh == 2 || bn <= 128) ? 3 : 2; }
constexpr int PF_HEADER_BYTES = 1024;
__host__ __device__ constexpr int pf_x_bytes(int bn) { return bn * PF_BK * 2; }                       // 32 KB at 256 tokens
__host__ __device__ constexpr int pf_stage_bytes(int bn, int fh) { return pf_a_bytes(fh) + pf_x_bytes(bn); }
__host__ __device__ constexpr int pf_smem_bytes(int bn, int fh)
{
    return PF_HEADER_BYTES + pf_stages(bn, fh) * pf_stage_bytes(bn, fh) + 1024;    // + slack for 1 KB alignment
}

constexpr int PF_MAX_GROUP = 3;    // linears that share their activations in one launch (q/k/v, gate/up)

// One linear of a launch.  Its feature tiles are blockIdx.y = tile0 .. tile0 + tiles - 1.
struct PrefillSeg
{
    const uint8_t* W;
    const uint8_t* blk;
    uint16_t* Y;
    long long ldy_m, ldy_n;
    unsigned int N, ldw, tile0;
    float w_scale, alpha, beta, post_scale;
    unsigned int y_tma;    // 1: the epilogue stages BF16 tiles in shared memory and writes them with TMA stores
};

struct PrefillParams
{
    PrefillSeg seg[PF_MAX_GROUP];
    unsigned int n_seg;
    unsigned int* status;
    unsigned int M, K;
    unsigned int out_f32;
};

// The three output tensor maps of a launch (unused ones are zero).
struct PrefillYMaps
{
    CUtensorMap m[PF_MAX_GROUP];
};

// ---- tcgen05 wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem]; BF16 inputs, FP32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 TMEM lanes (one per thread of the warp) x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major BF16 tile whose rows are 128 bytes (64 k), stored
// with the 128-byte swizzle in 8-row groups of 1024 bytes: start address, stride between 8-row
// groups = 1024 B, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).  The leading-byte
// offset is not used by swizzled K-major tiles of one swizzle row; it is set to 16 B.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D = F32 (bits 4-5 = 1), A = B = BF16 (bits 7-9 = 1, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__device__ __forceinline__ uint32_t umma_idesc_bf16(uint32_t m, uint32_t n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// 2-D tiled TMA load.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
// 2-D tiled TMA store shared -> global; rows and columns past the tensor's extent are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0), "r"(c1),
                 "r"(smem_u32(src))
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait_read()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// True in exactly one lane of the (converged) warp, the same lane every time.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void sts16(uint32_t addr, uint16_t v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory"); }
__device__ __forceinline__ void bar_sync_named(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Sixteen E2M1 nibbles (8 bytes, natural order) times one E4M3 block scale -> eight bf16x2.
// e2m1x2 -> f16x2 in hardware, times the scale in FP16 (exact: at most 6 significant bits), then
// widened and packed to BF16 (exact again), so each value equals the reference's table * scale.
__device__ __forceinline__ void dequant_fp4x16_natural(uint2 nib, uint32_t scale_byte, uint32_t (&out)[8])
{
    uint32_t s2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(s2) : "h"((uint16_t)(scale_byte | (scale_byte << 8))));
    const uint32_t w[2] = { nib.x, nib.y };
#pragma unroll
    for (int i = 0; i < 8; i++)
    {
        const uint16_t b = (uint16_t)((w[i >> 2] >> (8 * (i & 3))) & 0xFFu);
        uint32_t h2;
        asm("{\n\t.reg .b8 lo, hi;\n\tmov.b16 {lo, hi}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, lo;\n\t}" : "=r"(h2) : "h"(b));
        uint32_t p2;
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(p2) : "r"(h2), "r"(s2));
        const float2 f = half2_bits_to_float2(p2);
        out[i] = pack_bf16x2(f.x, f.y);
    }
}

// ---- the kernel ------------------------------------------------------------------------------------
template <int WT, bool SCALED, int BN, int FH>
__global__ void __launch_bounds__(PF_THREADS, (BN > 256 || FH > 1) ? 1 : 2) gemm_wq_prefill_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ PrefillYMaps tmY, const PrefillParams p)
{
    extern __shared__ unsigned char pf_smem_raw[];
    // 1 KB alignment for the swizzled tiles
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int PF_STAGES = pf_stages(BN, FH);
    constexpr int PF_A_BYTES = pf_a_bytes(FH);
    uint64_t* full_x = reinterpret_cast<uint64_t*>(smem);          // [PF_MAX_STAGES]
    uint64_t* full_a = full_x + PF_MAX_STAGES;                     // [PF_MAX_STAGES]
    uint64_t* empty = full_a + PF_MAX_STAGES;                      // [PF_MAX_STAGES]
    uint64_t* acc_full = empty + PF_MAX_STAGES;                    // [1]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    unsigned char* stages = smem + PF_HEADER_BYTES;

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // token tiles vary fastest, so the CTAs that share a weight tile run together
    // which linear of the launch this feature tile belongs to
    unsigned int si = 0;
    if (p.n_seg > 1 && blockIdx.y >= p.seg[1].tile0) { si = 1; }
    if (p.n_seg > 2 && blockIdx.y >= p.seg[2].tile0) { si = 2; }
    const PrefillSeg& g = p.seg[si];
    const unsigned int n0 = (blockIdx.y - g.tile0) * (PF_BM * FH);    // first output feature of the tile
    constexpr int PF_X_BYTES = pf_x_bytes(BN), PF_STAGE_BYTES = pf_stage_bytes(BN, FH), PF_TMEM_COLS = BN * FH;
    static_assert(BN * FH <= 512, "TMEM has 512 columns");
    const unsigned int m0 = blockIdx.x * BN;         // first token of the tile
    const unsigned int n_kblocks = p.K / PF_BK;
    const unsigned int tile_tokens = min((unsigned int)BN, p.M - m0);
    constexpr int NB = BN > 256 ? BN / 256 : 1;      // UMMAs (of up to 256 tokens) that share one A tile
    constexpr int BNU = BN / NB;                     // tokens per UMMA

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < PF_STAGES; s++)
        {
            mbar_init(full_x + s, 1);
            mbar_init(full_a + s, PF_DQ_WARPS);
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == PF_DQ_WARPS + 1) { tmem_alloc(tmem_base_slot, PF_TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == PF_DQ_WARPS)
    {
        // =========================== TMA lane: activations ===========================
        if (lane == 0)
        {
            bool ok = true;
            unsigned int issued = 0;
            for (unsigned int kb = 0; kb < n_kblocks; kb++)
            {
                const unsigned int s = kb % PF_STAGES;
                if (kb >= PF_STAGES && (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((kb / PF_STAGES) - 1) & 1u)))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                    break;
                }
                mbar_expect_tx(full_x + s, PF_X_BYTES);
#pragma unroll
                for (int nb = 0; nb < NB; nb++)
                {
                    tma_load_2d(stages + s * PF_STAGE_BYTES + PF_A_BYTES + nb * (BNU * PF_BK * 2), &tmX, (int)(kb * PF_BK),
                        (int)(m0 + nb * BNU), full_x + s);
                }
                mbar_arrive(full_x + s);
                issued = kb + 1;
            }
            if (!ok)
            {
                // wait (bounded) for my copies in flight before the CTA may leave
                const unsigned int first = issued > PF_STAGES ? issued - PF_STAGES : 0;
                for (unsigned int kb = first; kb < issued; kb++) { mbar_wait_bounded(full_x + (kb % PF_STAGES), (kb / PF_STAGES) & 1u); }
            }
        }
    }
    else if (warp == PF_DQ_WARPS + 1)
    {
        // =========================== MMA warp ===========================
        // The whole warp runs the loop (waits and descriptor arithmetic stay warp-uniform); one
        // elected lane issues the UMMAs and the commits.
        {
            bool ok = true;
            for (unsigned int kb = 0; kb < n_kblocks && ok; kb++)
            {
                const unsigned int s = kb % PF_STAGES;
                const uint32_t par = (kb / PF_STAGES) & 1u;
                if (*abort_flag != 0 || !mbar_wait_bounded(full_x + s, par) || !mbar_wait_bounded(full_a + s, par))
                {
                    ok = false;
                    if (lane == 0)
                    {
                        atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                        *abort_flag = 1;
                    }
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(stages + s * PF_STAGE_BYTES);
                const uint32_t b_addr = a_addr + PF_A_BYTES;
                if (elect_one())
                {
#pragma unroll
                for (int nb = 0; nb < NB; nb++)
                {
                    if (tile_tokens <= (unsigned int)(nb * BNU)) { break; }    // no live token in this part
                    const unsigned int live = min((unsigned int)BNU, tile_tokens - nb * BNU);
                    const uint32_t idesc = umma_idesc_bf16(PF_BM, (live + 15u) & ~15u);
#pragma unroll
                    for (int k = 0; k < PF_BK / 16; k++)
                    {
#pragma unroll
                        for (int fh = 0; fh < FH; fh++)
                        {
                            // 16 k = 32 bytes further along the 128-byte swizzle row; the second 128-feature
                            // tile sits 16 KB further in the A stage and accumulates BN columns further in TMEM
                            umma_bf16(tmem_base + fh * BN + nb * BNU, umma_desc_kmajor_sw128(a_addr + fh * (PF_BM * PF_BK * 2) + k * 32),
                                umma_desc_kmajor_sw128(b_addr + nb * (BNU * PF_BK * 2) + k * 32), idesc,
                                (kb | (unsigned int)k) != 0 ? 1u : 0u);
                        }
                    }
                }
                umma_commit(empty + s);
                }
                __syncwarp();
            }
            __syncwarp();
            if (elect_one())
            {
                if (ok) { umma_commit(acc_full); }
                else
                {
                    mbar_arrive(acc_full);    // let the epilogue warps fall through; they see the abort flag
                }
            }
        }
    }
    else
    {
        // =========================== dequantise, then epilogue (warps 0..7) ===========================
        const unsigned int tid = threadIdx.x;    // 0..255
        // 2*FH (row, 16-element group) pieces per thread per k block
        constexpr int NP = 2 * FH;
        unsigned int prow[NP], pq[NP];
#pragma unroll
        for (int i = 0; i < NP; i++)
        {
            const unsigned int piece = tid + 256u * i;
            prow[i] = piece >> 2;
            pq[i] = piece & 3u;
        }
        // raw weight bytes of two k blocks in flight (kb and kb+1): one L2 latency is about one k block
        uint4 raw8[2][NP];      // [slot][piece] FP8: 16 bytes per piece
        uint2 raw4[2][NP];      // FP4: 8 bytes per piece
        uint32_t rawsc[2][NP];  // FP4: the piece's block scale
        auto load_raw = [&](unsigned int kb, int slot) {
#pragma unroll
            for (int i = 0; i < NP; i++)
            {
                const unsigned int n = n0 + prow[i];
                raw8[slot][i] = make_uint4(0, 0, 0, 0);
                raw4[slot][i] = make_uint2(0, 0);
                rawsc[slot][i] = 0;
                if (n < g.N)
                {
                    const size_t e = (size_t)n * g.ldw + (size_t)kb * PF_BK + pq[i] * 16;
                    if (WT == DT_FP4)
                    {
                        raw4[slot][i] = __ldg(reinterpret_cast<const uint2*>(g.W + e / 2));
                        rawsc[slot][i] = __ldg(g.blk + e / 16);
                    }
                    else { raw8[slot][i] = __ldg(reinterpret_cast<const uint4*>(g.W + e)); }
                }
            }
        };
        bool ok = true;
        if (n_kblocks > 0) { load_raw(0, 0); }
        if (n_kblocks > 1) { load_raw(1, 1); }
        auto convert_and_refill = [&](unsigned int kb, int slot, uint32_t (&out)[NP][8]) {
#pragma unroll
            for (int i = 0; i < NP; i++)
            {
                if (WT == DT_FP4) { dequant_fp4x16_natural(raw4[slot][i], rawsc[slot][i], out[i]); }
                else
                {
                    const uint32_t w[4] = { raw8[slot][i].x, raw8[slot][i].y, raw8[slot][i].z, raw8[slot][i].w };
#pragma unroll
                    for (int j = 0; j < 4; j++) { dequant_fp8x4<WT, SCALED>(w[j], g.w_scale, out[i][2 * j], out[i][2 * j + 1]); }
                }
            }
            if (kb + 2 < n_kblocks) { load_raw(kb + 2, slot); }    // in flight for two k blocks
        };
        // The conversion of block kb+1 is issued between the stores of block kb and their proxy fence,
        // so the fence finds the stores already performed.
        uint32_t out[NP][8];
        if (n_kblocks > 0) { convert_and_refill(0, 0, out); }
        for (unsigned int kb = 0; kb < n_kblocks; kb++)
        {
            const unsigned int s = kb % PF_STAGES;
            if (ok && kb >= PF_STAGES && (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((kb / PF_STAGES) - 1) & 1u)))
            {
                ok = false;
                if (*abort_flag == 0)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                }
            }
            if (ok)
            {
                const uint32_t a_addr = smem_u32(stages + s * PF_STAGE_BYTES);
#pragma unroll
                for (int i = 0; i < NP; i++)
                {
                    // row r, 16-byte chunks 2q and 2q+1 of its 128-byte row, XOR-swizzled by (r & 7)
                    const uint32_t rowaddr = a_addr + prow[i] * 128;
                    const uint32_t sw = prow[i] & 7u;
                    sts128(rowaddr + (((2 * pq[i]) ^ sw) << 4), out[i][0], out[i][1], out[i][2], out[i][3]);
                    sts128(rowaddr + (((2 * pq[i] + 1) ^ sw) << 4), out[i][4], out[i][5], out[i][6], out[i][7]);
                }
            }
            if (kb + 1 < n_kblocks)
            {
                // the slot index must be a compile-time constant for the arrays to stay in registers
                if ((kb & 1u) != 0) { convert_and_refill(kb + 1, 0, out); }
                else { convert_and_refill(kb + 1, 1, out); }
            }
            if (ok)
            {
                fence_proxy_async();    // make the generic-proxy stores visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) { mbar_arrive(full_a + s); }
            }
        }

        // ---- epilogue: warps w and w+4 share TMEM lanes 32*(w%4).., and split the token columns ----
        if (!mbar_wait_bounded(acc_full, 0))
        {
            ok = false;
            atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
            *abort_flag = 1;
        }
        if (*abort_flag != 0) { ok = false; }
        tc_fence_after();
        if (ok && n_kblocks > 0 && g.y_tma != 0)
        {
            // BF16 tile [BN tokens][128 features] per feature half in the (now idle) stage memory,
            // then one TMA store per half; the store clips rows past M and features past N
            const unsigned int quarter = warp & 3u;
            const unsigned int half = warp >> 2;
#pragma unroll
            for (int fh = 0; fh < FH; fh++)
            {
                const uint32_t ytile = smem_u32(stages) + fh * (BN * PF_BM * 2) + (quarter * 32 + lane) * 2;
                for (unsigned int c0 = half * (BN / 2); c0 < half * (BN / 2) + BN / 2 && c0 < tile_tokens; c0 += 32)
                {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + fh * BN + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                    {
                        sts16(ytile + (c0 + j) * (PF_BM * 2), __bfloat16_as_ushort(__float2bfloat16_rn(g.alpha * (__uint_as_float(r[j]) * g.post_scale))));
                    }
                }
            }
            fence_proxy_async();
            bar_sync_named(1, 32 * PF_DQ_WARPS);
            if (tid == 0)
            {
#pragma unroll
                for (int fh = 0; fh < FH; fh++) { tma_store_2d(&tmY.m[si], stages + fh * (BN * PF_BM * 2), (int)(n0 + fh * PF_BM), (int)m0); }
                tma_store_commit_and_wait_read();
            }
        }
        else if (ok && n_kblocks > 0)
        {
            const unsigned int quarter = warp & 3u;
            const unsigned int half = warp >> 2;    // the two warps of a TMEM lane quarter split the token columns
#pragma unroll
            for (int fh = 0; fh < FH; fh++)
            {
                const unsigned int n = n0 + fh * PF_BM + quarter * 32 + lane;
                for (unsigned int c0 = half * (BN / 2); c0 < half * (BN / 2) + BN / 2 && c0 < tile_tokens; c0 += 32)
                {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + fh * BN + c0, r);
                    tmem_ld_wait();
                    if (n < g.N)
                    {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                        {
                            const unsigned int m = m0 + c0 + j;
                            if (c0 + j < tile_tokens)
                            {
                                const long long yi = (long long)m * g.ldy_m + (long long)n * g.ldy_n;
                                float o = g.alpha * (__uint_as_float(r[j]) * g.post_scale);
                                if (p.out_f32 == 1u)
                                {
                                    float* y = reinterpret_cast<float*>(g.Y) + yi;
                                    if (g.beta != 0.f) { o += g.beta * *y; }
                                    *y = o;
                                }
                                else
                                {
                                    uint16_t* y = g.Y + yi;
                                    if (g.beta != 0.f) { o = (p.out_f32 == 2u ? __bfloat162float(__float2bfloat16_rn(o)) : o) + g.beta * bf16_bits_to_float(*y); }
                                    *y = __bfloat16_as_ushort(__float2bfloat16_rn(o));
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == PF_DQ_WARPS + 1) { tmem_dealloc(tmem_base, PF_TMEM_COLS); }
}

inline bool prefill_supported(int w_type, unsigned int N, unsigned int M, unsigned int K, unsigned int ldw, unsigned int ldx,
    unsigned int ldy_m, unsigned int ldy_n)
{
    (void)ldy_m;
    (void)ldy_n;
    (void)w_type;
    if (M <= 32 || K == 0 || (K % PF_BK) != 0 || (ldx % 8) != 0 || (ldw % 16) != 0) { return false; }
    return (N + PF_BM - 1) / PF_BM <= 65535u;    // grid.y
}

template <int WT, bool SCALED, int BN, int FH>
static int launch_prefill_bn(const CUtensorMap& tmX, const PrefillYMaps& tmY, const PrefillParams& pp, unsigned int feature_tiles, int device,
    cudaStream_t stream)
{
    auto kernel = gemm_wq_prefill_kernel<WT, SCALED, BN, FH>;
    static std::atomic<bool> attr_set[64];    // zero-initialised; setting the attribute twice is harmless
    if (!attr_set[device].load(std::memory_order_acquire))
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem_bytes(BN, FH)) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16");
            return 1;
        }
        attr_set[device].store(true, std::memory_order_release);
    }
    const dim3 grid((pp.M + BN - 1) / BN, feature_tiles);
    count_launch();
    kernel<<<grid, PF_THREADS, pf_smem_bytes(BN, FH), stream>>>(tmX, tmY, pp);
    return report_launch("gemm_wq_bf16");
}

}    // namespace b200
