// Quantized-weight linear for a few dozen tokens (up to 128): the regime between the decode GEMV and the
// prefill GEMM, where the weights are still read once and HBM is the bound, but there are too many tokens for
// CUDA-core or mma.sync dot products to keep up with the stream.
//
// The contraction runs on tcgen05.mma with the accumulator in TMEM, like the prefill kernel, but the launch is
// shaped for streaming:
//   * a tile is 128 output features x all tokens (16 .. 128, one UMMA N), so every weight byte is read once;
//   * the k range is cut into 1, 2, 4 or 8 slices that run as ONE thread-block cluster: small linears (4096 x
//     4096 has 32 feature tiles) still fill the CTA slots of every SM, and the slices' FP32 partial tiles are
//     summed through distributed shared memory in slice order (no workspace, no atomics, the same bits every
//     run), each CTA of the cluster finishing a share of the token columns;
//   * a TMA lane streams the QUANTISED weights into a ring of raw stages, [runs][128 rows][64 B] each (64-byte
//     swizzle, so that a warp whose lanes walk the rows reads it without bank conflicts);
//   * eight warps, one thread per output feature and k half, read their 32 weights of a k block from the raw
//     stage, dequantise them to BF16 exactly as the reference's conversion kernels do, and write them with ONE
//     tcgen05.st into the A operand's columns of TENSOR MEMORY: the UMMA takes A from TMEM and only the small
//     activation tile from shared memory.  (Staging A in shared memory, as the prefill kernel does, costs 4
//     bytes of shared-memory traffic per weight and a UMMA that re-reads every 128-byte row of the tile for each
//     of its four k steps: measured, that pipeline moved one 64-k block per 0.5 us and CTA whatever else was
//     changed.)  Both operands are BF16: a kind::f16 UMMA whose descriptor names FP16 for A and BF16 for B is
//     an illegal instruction on this part, so FP4 cannot stay in the FP16 its hardware conversion produces;
//   * a second TMA lane brings the [tokens][64 k] BF16 activation tiles, an MMA lane issues four UMMAs per
//     k block.
// Every wait is bounded; on expiry the status word is raised, the CTA stops issuing, still meets its cluster
// at both cluster barriers (so no peer reads freed shared memory or waits for it), frees its TMEM and returns.
#pragma once

#include <cooperative_groups.h>

#include "prefill_launch.cuh"

namespace b200
{

constexpr int SK_BM = 128;                     // output features per tile (UMMA M)
constexpr int SK_BK = 64;                      // k per block
constexpr int SK_DQ_WARPS = 8;                 // warp w: TMEM lanes 32 (w & 3) .., k half w >> 2 of every block
constexpr int SK_THREADS = 32 * (SK_DQ_WARPS + 3);    // + activation TMA warp, MMA warp, weight TMA warp
constexpr int SK_HEADER_BYTES = 1024;
constexpr int SK_MAX_SPLIT = 8;
constexpr int SK_SLICE_ELEMS = 256;            // slices begin on multiples of this many k (one FP4 scale run)
constexpr int SK_PAIR = 2;                     // k blocks per stage: one barrier round trip per 128 k
constexpr int SK_A_COLS = SK_PAIR * SK_BK / 2; // TMEM columns of one A stage: 128 BF16 per lane
// A / X stages (A in TMEM, X in shared memory) and the raw ring.  A raw stage holds `runs` 64-byte runs of each of
// the 128 rows (64 k of FP8, 128 k of FP4 per run).
__host__ __device__ constexpr int sk_stages(int bn) { return 2; }
__host__ __device__ constexpr int sk_runs(int wt, int bn) { return bn > 64 ? 2 : 4; }    // 128 tokens: shorter runs, so that two CTAs share an SM
__host__ __device__ constexpr int sk_raw_stages(int wt, int bn) { return (wt != DT_FP4 && bn <= 16) ? 3 : 2; }    // two CTAs per SM
__host__ __device__ constexpr int sk_raw_w_bytes(int runs) { return runs * SK_BM * 64; }
__host__ __device__ constexpr int sk_raw_s_bytes(int wt, int runs) { return wt == DT_FP4 ? (runs / 2) * SK_BM * 16 : 0; }
__host__ __device__ constexpr int sk_raw_bytes(int wt, int runs) { return sk_raw_w_bytes(runs) + sk_raw_s_bytes(wt, runs); }
__host__ __device__ constexpr int sk_kb_per_raw(int wt, int runs) { return wt == DT_FP4 ? 2 * runs : runs; }    // k blocks per raw stage
__host__ __device__ constexpr int sk_x_bytes(int bn) { return SK_PAIR * bn * SK_BK * 2; }    // two [tokens][64 k] tiles
__host__ __device__ constexpr int sk_smem_bytes(int wt, int bn)
{
    return SK_HEADER_BYTES + sk_stages(bn) * sk_x_bytes(bn) + sk_raw_stages(wt, bn) * sk_raw_bytes(wt, sk_runs(wt, bn)) + 1024;
}
// accumulator columns, then the A stages; allocations are powers of two
__host__ __device__ constexpr int sk_tmem_cols(int bn) { return (bn + sk_stages(bn) * SK_A_COLS) <= 256 ? 256 : 512; }

// 32 TMEM lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t* r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]; BF16 inputs, FP32 accumulate.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ uint4 sk_lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t sk_lds16(uint32_t addr)
{
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

struct StreamParams
{
    PrefillSeg seg[PF_MAX_GROUP];    // y_tma unused
    unsigned int n_seg;
    unsigned int* status;
    unsigned int M, K;
    unsigned int out_f32;            // 0 BF16, 1 FP32, 2 BF16 with the product rounded before beta * Y
    unsigned int split;              // cluster size along x = k slices
};

// The weight (and FP4 scale) maps of the up to three linears of a launch.
struct StreamWMaps
{
    CUtensorMap w[PF_MAX_GROUP];
    CUtensorMap s[PF_MAX_GROUP];
};

template <int WT, bool SCALED, int BN>
__global__ void __launch_bounds__(SK_THREADS, 2) gemm_wq_stream_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ StreamWMaps tmW, const StreamParams p)
{
    namespace cg = cooperative_groups;
    constexpr int STAGES = sk_stages(BN);
    constexpr int X_BYTES = sk_x_bytes(BN);
    constexpr int TMEM_COLS = sk_tmem_cols(BN);
    constexpr int RUNS = sk_runs(WT, BN);
    constexpr int RAW_STAGES = sk_raw_stages(WT, BN);
    constexpr int RAW_W_BYTES = sk_raw_w_bytes(RUNS);
    constexpr int RAW_BYTES = sk_raw_bytes(WT, RUNS);
    constexpr int KB_PER_RAW = sk_kb_per_raw(WT, RUNS);
    static_assert(BN * SK_BM * 4 <= STAGES * X_BYTES + RAW_STAGES * RAW_BYTES, "the partial tile reuses the activation stages and the raw ring");
    static_assert(BN + STAGES * SK_A_COLS <= TMEM_COLS, "accumulator and A stages fit the allocation");
    extern __shared__ unsigned char sk_smem_raw[];
    // The offset of the aligned base inside the dynamic shared memory is the same in every CTA of the cluster
    // (same kernel, same static layout), so peers address each other's tiles through map_shared_rank.
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sk_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_x = reinterpret_cast<uint64_t*>(smem);
    uint64_t* full_a = full_x + 4;
    uint64_t* empty = full_a + 4;
    uint64_t* raw_full = empty + 4;
    uint64_t* raw_empty = raw_full + 4;
    uint64_t* acc_full = raw_empty + 4;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    unsigned char* xs = smem + SK_HEADER_BYTES;
    unsigned char* raws = xs + STAGES * X_BYTES;

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned int S = p.split;
    const unsigned int rank = S > 1 ? cluster.block_rank() : 0u;
    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned int si = 0;
    if (p.n_seg > 1 && blockIdx.y >= p.seg[1].tile0) { si = 1; }
    if (p.n_seg > 2 && blockIdx.y >= p.seg[2].tile0) { si = 2; }
    const PrefillSeg& g = p.seg[si];
    const unsigned int n0 = (blockIdx.y - g.tile0) * SK_BM;
    const unsigned int m0 = blockIdx.z * BN;
    const unsigned int tile_tokens = min((unsigned int)BN, p.M - m0);
    // slices in units of 256 k (four k blocks): a raw run and an FP4 scale run never straddle two slices
    const unsigned int units = p.K / SK_SLICE_ELEMS;
    const unsigned int kb_begin = (unsigned int)(((unsigned long long)units * rank) / S) * (SK_SLICE_ELEMS / SK_BK);
    const unsigned int kb_end = (unsigned int)(((unsigned long long)units * (rank + 1)) / S) * (SK_SLICE_ELEMS / SK_BK);
    const unsigned int nkb = kb_end - kb_begin;
    const unsigned int n_raw = (nkb + KB_PER_RAW - 1) / KB_PER_RAW;
    const unsigned int npair = nkb / SK_PAIR;    // slices are whole multiples of four k blocks

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; s++)
        {
            mbar_init(full_x + s, 1);
            mbar_init(full_a + s, SK_DQ_WARPS);
            mbar_init(empty + s, 1);
        }
        for (int s = 0; s < RAW_STAGES; s++)
        {
            mbar_init(raw_full + s, 1);
            mbar_init(raw_empty + s, SK_DQ_WARPS);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == SK_DQ_WARPS + 1) { tmem_alloc(tmem_base_slot, TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t tmem_a = tmem_base + BN;    // the A stages follow the accumulator's columns
    // the next kernel of the stream may start its own weight prefetch as soon as SM resources allow
    pdl_launch_dependents();

    if (warp == SK_DQ_WARPS + 2)
    {
        // =========================== TMA lane: quantised weights ===========================
        if (lane == 0)
        {
            const uint64_t pol = l2_policy_evict_first();
            bool ok = true;
            unsigned int issued = 0;
            for (unsigned int r = 0; r < n_raw; r++)
            {
                const unsigned int s = r % RAW_STAGES;
                if (r >= RAW_STAGES && (*abort_flag != 0 || !mbar_wait_bounded(raw_empty + s, ((r / RAW_STAGES) - 1) & 1u)))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                    break;
                }
                unsigned char* dst = raws + s * RAW_BYTES;
                // a run is 64 bytes of every row: 64 k of FP8, 128 k of FP4; runs past the row's end are zero-filled
                const unsigned int kb0 = kb_begin + r * KB_PER_RAW;
                const int run0 = (int)(WT == DT_FP4 ? kb0 / 2 : kb0);
                mbar_expect_tx(raw_full + s, RAW_BYTES);
                tma_load_3d_hint(dst, &tmW.w[si], 0, (int)n0, run0, raw_full + s, pol);
                if (WT == DT_FP4) { tma_load_3d_hint(dst + RAW_W_BYTES, &tmW.s[si], 0, (int)n0, (int)(kb0 / 4), raw_full + s, pol); }
                mbar_arrive(raw_full + s);
                issued = r + 1;
            }
            if (!ok)
            {
                const unsigned int first = issued > RAW_STAGES ? issued - RAW_STAGES : 0;
                for (unsigned int r = first; r < issued; r++) { mbar_wait_bounded(raw_full + (r % RAW_STAGES), (r / RAW_STAGES) & 1u); }
            }
        }
    }
    else if (warp == SK_DQ_WARPS)
    {
        // =========================== TMA lane: activations ===========================
        if (lane == 0)
        {
            pdl_wait();    // the activations are the previous kernel's output
            bool ok = true;
            unsigned int issued = 0;
            for (unsigned int j = 0; j < npair; j++)
            {
                const unsigned int s = j % STAGES;
                if (j >= STAGES && (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((j / STAGES) - 1) & 1u)))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                    break;
                }
                mbar_expect_tx(full_x + s, X_BYTES);
#pragma unroll
                for (int h = 0; h < SK_PAIR; h++)
                {
                    tma_load_2d(xs + s * X_BYTES + h * (X_BYTES / SK_PAIR), &tmX, (int)((kb_begin + SK_PAIR * j + h) * SK_BK), (int)m0, full_x + s);
                }
                mbar_arrive(full_x + s);
                issued = j + 1;
            }
            if (!ok)
            {
                const unsigned int first = issued > STAGES ? issued - STAGES : 0;
                for (unsigned int j = first; j < issued; j++) { mbar_wait_bounded(full_x + (j % STAGES), (j / STAGES) & 1u); }
            }
        }
    }
    else if (warp == SK_DQ_WARPS + 1)
    {
        // =========================== MMA warp ===========================
        bool ok = true;
        const uint32_t idesc = umma_idesc_bf16(SK_BM, (tile_tokens + 15u) & ~15u);
        for (unsigned int j = 0; j < npair && ok; j++)
        {
            const unsigned int s = j % STAGES;
            const uint32_t par = (j / STAGES) & 1u;
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
            const uint32_t b_addr = smem_u32(xs + s * X_BYTES);
            if (elect_one())
            {
#pragma unroll
                for (int k = 0; k < SK_PAIR * SK_BK / 16; k++)
                {
                    // 16 k of A = 8 TMEM columns; of B = 32 bytes further along the 128-byte swizzle row of its tile
                    umma_bf16_ts(tmem_base, tmem_a + s * SK_A_COLS + k * 8,
                        umma_desc_kmajor_sw128(b_addr + (k / 4) * (X_BYTES / SK_PAIR) + (k % 4) * 32), idesc, (j | (unsigned int)k) != 0 ? 1u : 0u);
                }
                umma_commit(empty + s);
            }
            __syncwarp();
        }
        __syncwarp();
        if (elect_one())
        {
            if (ok) { umma_commit(acc_full); }
            else { mbar_arrive(acc_full); }
        }
    }
    else
    {
        // =========================== dequantise (warps 0..7) ===========================
        // thread = (output feature, k half): TMEM lane 32 (warp & 3) + lane, and of each k block of a stage the
        // columns 16 half .. ; two k blocks per round, so that one wait and one arrival serve 128 k
        const unsigned int row = (warp & 3u) * 32 + lane;
        const unsigned int half = warp >> 2;
        const uint32_t lane_field = ((warp & 3u) * 32u) << 16;
        const uint32_t sw64 = (row >> 1) & 3u;    // the TMA's 64-byte swizzle: 16-byte chunk index ^= row bits 1-2
        bool ok = true;
        for (unsigned int j = 0; j < npair; j++)
        {
            const unsigned int kb = SK_PAIR * j;               // first k block of the pair; pairs never straddle raw stages
            const unsigned int r = kb / KB_PER_RAW, jr = kb % KB_PER_RAW;
            const unsigned int rs = r % RAW_STAGES;
            if (ok && jr == 0 && (*abort_flag != 0 || !mbar_wait_bounded(raw_full + rs, (r / RAW_STAGES) & 1u)))
            {
                ok = false;
                if (*abort_flag == 0)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    *abort_flag = 1;
                }
            }
            // Ask early whether the A stage is free: the answer (about a hundred cycles away even when it is yes)
            // arrives while the blocks are dequantised.
            const unsigned int s = j % STAGES;
            const bool stage_free = (j < STAGES) || mbar_try_wait(empty + s, ((j / STAGES) - 1) & 1u);
            uint32_t out[SK_PAIR][16];
            if (ok)
            {
                const uint32_t raw = smem_u32(raws + rs * RAW_BYTES);
                if (WT == DT_FP4)
                {
                    // run jr / 2 holds 128 k of the row = both k blocks of the pair; my 32 k of block h are one 16-byte chunk
                    const uint32_t wrow = raw + (jr >> 1) * (SK_BM * 64) + row * 64;
                    const uint32_t srow = raw + RAW_W_BYTES + (jr >> 2) * (SK_BM * 16) + row * 16 + (jr & 3u) * 4 + half * 2;
                    uint4 v[SK_PAIR];
                    uint32_t sc[SK_PAIR];
#pragma unroll
                    for (int h = 0; h < SK_PAIR; h++)
                    {
                        v[h] = sk_lds128(wrow + (((h * 2 + half) ^ sw64) << 4));
                        sc[h] = sk_lds16(srow + h * 4);
                    }
#pragma unroll
                    for (int h = 0; h < SK_PAIR; h++)
                    {
                        uint32_t lo[8], hi[8];
                        dequant_fp4x16_natural(make_uint2(v[h].x, v[h].y), sc[h] & 0xFFu, lo);
                        dequant_fp4x16_natural(make_uint2(v[h].z, v[h].w), sc[h] >> 8, hi);
#pragma unroll
                        for (int q = 0; q < 8; q++)
                        {
                            out[h][q] = lo[q];
                            out[h][8 + q] = hi[q];
                        }
                    }
                }
                else
                {
                    uint4 v[SK_PAIR][2];
#pragma unroll
                    for (int h = 0; h < SK_PAIR; h++)
                    {
                        const uint32_t base = raw + (jr + h) * (SK_BM * 64) + row * 64;
                        v[h][0] = sk_lds128(base + (((2 * half) ^ sw64) << 4));
                        v[h][1] = sk_lds128(base + (((2 * half + 1) ^ sw64) << 4));
                    }
#pragma unroll
                    for (int h = 0; h < SK_PAIR; h++)
                    {
                        const uint32_t w[8] = { v[h][0].x, v[h][0].y, v[h][0].z, v[h][0].w, v[h][1].x, v[h][1].y, v[h][1].z, v[h][1].w };
#pragma unroll
                        for (int q = 0; q < 8; q++) { dequant_fp8x4<WT, SCALED>(w[q], g.w_scale, out[h][2 * q], out[h][2 * q + 1]); }
                    }
                }
            }
            // the raw stage is free once its last k block has been read into registers
            if (ok && (jr + SK_PAIR == KB_PER_RAW || j + 1 == npair))
            {
                __syncwarp();
                if (lane == 0) { mbar_arrive(raw_empty + rs); }
            }
            if (ok && !stage_free && (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((j / STAGES) - 1) & 1u)))
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
                tc_fence_after();    // the UMMAs that read this stage last have completed (the empty barrier said so)
#pragma unroll
                for (int h = 0; h < SK_PAIR; h++) { tmem_st_32x16(tmem_a + lane_field + s * SK_A_COLS + h * (SK_BK / 2) + half * 16, out[h]); }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(full_a + s); }
            }
        }
    }

    // ---- the slices' partial tiles: TMEM -> this CTA's shared memory  ----
    float* part = reinterpret_cast<float*>(xs);    // [BN tokens][128 features]; the activation stages and the raw ring are idle now
    bool good = true;
    if (warp < SK_DQ_WARPS) { pdl_wait(); }    // Y (and beta * Y) belong to the stream's order
    if (warp < SK_DQ_WARPS)
    {
        if (!mbar_wait_bounded(acc_full, 0))
        {
            atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
            *abort_flag = 1;
        }
        good = *abort_flag == 0;
        tc_fence_after();
        const unsigned int quarter = warp & 3u, half = warp >> 2;
        constexpr int COLS_PER_HALF = BN >= 64 ? BN / 2 : BN;    // below 64 tokens only warps 0..3 read
        if (BN >= 64 || half == 0)
        {
            const unsigned int f = quarter * 32 + lane;
#pragma unroll
            for (int c = 0; c < COLS_PER_HALF; c += 16)
            {
                // sixteen columns at a time: the register budget of two 19-warp CTAs per SM has no room for more
                const unsigned int c0 = half * COLS_PER_HALF + c;
                uint32_t r[16];
                if (good && nkb > 0)
                {
                    tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + c0, r);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int q = 0; q < 16; q++) { part[(c0 + q) * SK_BM + f] = (good && nkb > 0) ? __uint_as_float(r[q]) : 0.f; }
            }
        }
    }
    tc_fence_before();
    if (S > 1) { cluster.sync(); }
    else { __syncthreads(); }

    // ---- sum the slices in slice order; CTA `rank` finishes token columns rank, rank + S, ... ----
    if (warp < SK_DQ_WARPS && *abort_flag == 0)
    {
        const float* peer[SK_MAX_SPLIT];
#pragma unroll
        for (int r = 0; r < SK_MAX_SPLIT; r++) { peer[r] = ((unsigned int)r < S && S > 1) ? cluster.map_shared_rank(part, r) : part; }
        const unsigned int tid = threadIdx.x;
        const unsigned int f = tid & (SK_BM - 1);
        const unsigned int n = n0 + f;
        for (unsigned int t = rank + S * (tid >> 7); t < tile_tokens; t += 2 * S)
        {
            float sum = 0.f;
#pragma unroll
            for (int r = 0; r < SK_MAX_SPLIT; r++)
            {
                if ((unsigned int)r < S) { sum += peer[r][t * SK_BM + f]; }
            }
            if (n < g.N)
            {
                const unsigned int m = m0 + t;
                const long long yi = (long long)m * g.ldy_m + (long long)n * g.ldy_n;
                float o = g.alpha * (sum * g.post_scale);
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
    // nobody leaves while a peer may still read its partial tile
    if (S > 1) { cluster.sync(); }
    else { __syncthreads(); }
    tc_fence_after();
    if (warp == SK_DQ_WARPS + 1) { tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---- host side -----------------------------------------------------------------------------------------
static inline bool sk_al16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

inline bool stream_supported(int w_type, const void* blk, unsigned int N, unsigned int M, unsigned int K, unsigned int ldw, unsigned int ldx)
{
    if (M == 0 || M > 128 || N == 0 || K == 0 || (K % SK_SLICE_ELEMS) != 0 || (ldx % 8) != 0) { return false; }
    if (w_type == DT_FP4) { return blk != nullptr && sk_al16(blk) && (ldw % 256) == 0; }    // 16-byte rows of scales
    return (ldw % 16) == 0;
}

// k slices per tile: the largest power of two (clusters of 3, 5, 6 or 7 CTAs did not all become resident together
// and ran as two waves) that keeps all CTAs within ONE wave of two per SM, with a margin for SMs whose cluster
// slots do not divide evenly; each slice is at least 256 k long.
static unsigned int sk_pick_split(unsigned int feature_tiles, unsigned int K, int sm_count)
{
    const unsigned int units = K / SK_SLICE_ELEMS;
    const unsigned int slots = (2u * (unsigned)sm_count * 9u) / 10u;
    unsigned int s = 1;
    while (2 * s <= (unsigned)SK_MAX_SPLIT && feature_tiles * 2 * s <= slots && 2 * s <= units) { s *= 2; }
    return s;
}

template <int WT, bool SCALED, int BN>
static int launch_stream_bn(const void* X, unsigned int ldx, const StreamParams& sp, unsigned int feature_tiles, int device, cudaStream_t stream,
    bool pdl)
{
    constexpr int RUNS = sk_runs(WT, BN);
    CUtensorMap tmX;
    StreamWMaps tmW;
    memset(&tmW, 0, sizeof(tmW));
    bool ok = make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, sp.K, sp.M, (unsigned long long)ldx * 2, SK_BK, BN, true);
    const unsigned long long kbytes = (WT == DT_FP4) ? sp.K / 2 : sp.K;
    for (unsigned int j = 0; j < (unsigned)PF_MAX_GROUP && ok; j++)
    {
        const PrefillSeg& g = sp.seg[j < sp.n_seg ? j : 0];
        const unsigned long long ldw_bytes = (WT == DT_FP4) ? g.ldw / 2 : g.ldw;
        ok = make_map(&tmW.w[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.W, 64, g.N, kbytes / 64, ldw_bytes, SK_BM, RUNS, false, true);
        if (ok && WT == DT_FP4)
        {
            ok = make_map(&tmW.s[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.blk, 16, g.N, sp.K / 256, g.ldw / 16, SK_BM, RUNS / 2, false);
        }
    }
    if (!ok) { return -2; }
    auto kernel = gemm_wq_stream_kernel<WT, SCALED, BN>;
    static std::atomic<bool> attr_set[64];
    if (!attr_set[device].load(std::memory_order_acquire))
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sk_smem_bytes(WT, BN)) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16");
            return 1;
        }
        attr_set[device].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(sp.split, feature_tiles, 1);
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = sk_smem_bytes(WT, BN);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (sp.split > 1)
    {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = sp.split;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    if (pdl)
    {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, kernel, tmX, tmW, sp) != cudaSuccess)
    {
        report_launch("gemm_wq_bf16");
        return 1;
    }
    return 0;
}

template <int WT, bool SCALED>
static int launch_stream_t(const void* X, unsigned int ldx, StreamParams& sp, int device, int sm_count, cudaStream_t stream, bool pdl)
{
    unsigned int feature_tiles = 0;
    for (unsigned int j = 0; j < sp.n_seg; j++)
    {
        sp.seg[j].tile0 = feature_tiles;
        feature_tiles += (sp.seg[j].N + SK_BM - 1) / SK_BM;
    }
    if (feature_tiles == 0 || feature_tiles > 65535u) { return -2; }
    sp.split = sk_pick_split(feature_tiles, sp.K, sm_count);
    if (sp.M <= 16) { return launch_stream_bn<WT, SCALED, 16>(X, ldx, sp, feature_tiles, device, stream, pdl); }
    if (sp.M <= 32) { return launch_stream_bn<WT, SCALED, 32>(X, ldx, sp, feature_tiles, device, stream, pdl); }
    if (sp.M <= 64) { return launch_stream_bn<WT, SCALED, 64>(X, ldx, sp, feature_tiles, device, stream, pdl); }
    return launch_stream_bn<WT, SCALED, 128>(X, ldx, sp, feature_tiles, device, stream, pdl);
}

// One launch for up to PF_MAX_GROUP linears that share X; items as for launch_prefill.  -2: not taken.
static int launch_stream(int w_type, const GemvParams* items, unsigned int count, int device, int sm_count, cudaStream_t stream, bool pdl)
{
    if (count == 0 || count > (unsigned)PF_MAX_GROUP) { return -2; }
    StreamParams sp;
    memset(&sp, 0, sizeof(sp));
    sp.n_seg = count;
    sp.status = items[0].status;
    sp.M = items[0].M;
    sp.K = items[0].K;
    sp.out_f32 = items[0].out_f32;
    bool all_pow2 = true;
    for (unsigned int j = 0; j < count; j++)
    {
        if (!stream_supported(w_type, items[j].blk, items[j].N, items[j].M, items[j].K, items[j].ldw, items[j].ldx)) { return -2; }
        if (!sk_al16(items[j].W)) { return -2; }
        all_pow2 = all_pow2 && pf_is_pow2_scale(items[j].w_scale);
    }
    if (!sk_al16(items[0].X)) { return -2; }
    const bool scaled = w_type != DT_FP4 && !all_pow2;
    for (unsigned int j = 0; j < count; j++)
    {
        PrefillSeg& g = sp.seg[j];
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
    if (w_type == DT_FP4) { return launch_stream_t<DT_FP4, false>(X, ldx, sp, device, sm_count, stream, pdl); }
    if (!scaled)
    {
        return w_type == DT_E5M2 ? launch_stream_t<DT_E5M2, false>(X, ldx, sp, device, sm_count, stream, pdl)
                                 : launch_stream_t<DT_E4M3, false>(X, ldx, sp, device, sm_count, stream, pdl);
    }
    return w_type == DT_E5M2 ? launch_stream_t<DT_E5M2, true>(X, ldx, sp, device, sm_count, stream, pdl)
                             : launch_stream_t<DT_E4M3, true>(X, ldx, sp, device, sm_count, stream, pdl);
}

}    // namespace b200
