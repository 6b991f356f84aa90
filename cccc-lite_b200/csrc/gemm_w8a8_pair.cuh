// W8A8 linear for more than 32 tokens: E4M3 weights x E4M3 activations on CTA pairs (tcgen05.mma cta_group::2,
// kind::f8f6f4), FP32 accumulation in tensor memory.  The mode of cccc/cublas_real.h:619-666 at prefill sizes, where the
// reference runs a cublasLt FP8 x FP8 matmul.
//
// Two CTAs on the two SMs of a TPC compute 256*FH output features x up to 256 tokens over the whole K range.  Nothing is
// converted: both operands are copied by TMA as they lie in memory (128 k = one 128-byte swizzle row per k block).  Per
// k block each CTA's TMA lane brings the [128 features][128 k] weight tiles of its own features and its HALF of the
// [256 tokens][128 k] quantised activations into one stage; rank 1 forwards "stage full" to the leader with one remote
// arrive; one lane of the leader issues 4*FH UMMAs of M=256, N=tokens, K=32 and commits to the "done" barrier of the
// stage in BOTH CTAs.  After the last k block eight warps of each CTA read their 128*FH features' accumulators, apply
// alpha * activation multiplier * weight multiplier and write BF16 tiles with TMA stores (or element by element for the
// other output forms).
// Every mbarrier wait is bounded; a CTA whose wait ran out raises the status word and drains.  Both CTAs always reach
// the cluster barrier before the TMEM columns are freed.
#pragma once

#include <atomic>

#include "gemm_native.cuh"
#include "gemm_prefill_pair.cuh"
#include "gemm_stream.cuh"

namespace b200
{

constexpr int WP_BK = 128;                      // k per block: one 128-byte swizzle row of E4M3
constexpr int WP_TILE_BYTES = 128 * WP_BK;      // 16 KB: 128 rows of one k block
constexpr int WP_EPI_WARPS = 8;
constexpr int WP_THREADS = 32 * (WP_EPI_WARPS + 2);    // TMA warp, MMA warp, epilogue warps
__host__ __device__ constexpr int wp_stage_bytes(int fh) { return (fh + 1) * WP_TILE_BYTES; }
__host__ __device__ constexpr int wp_stages(int fh) { return fh == 2 ? 4 : 6; }    // 192 KB either way
__host__ __device__ constexpr int wp_smem_bytes(int fh) { return PF_HEADER_BYTES + wp_stages(fh) * wp_stage_bytes(fh) + 1024; }

__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One member of a W8A8 launch (up to PF_MAX_GROUP members share the activations and their quantisation).
struct W8A8Member
{
    const void* W;
    void* Y;
    float w_inv_scale, alpha, beta;
    unsigned int N_out, ldw, ldy_m, ldy_n;
};

template <int FH>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(WP_THREADS, 1)
    gemm_w8a8_pair_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ StreamWMaps tmW, const __grid_constant__ PrefillYMaps tmY,
        const NativeParams p)
{
    extern __shared__ unsigned char wp_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(wp_smem_raw) + 1023) & ~(uintptr_t)1023);
    static_assert(FH == 1 || FH == 2, "512 TMEM columns");
    constexpr int NS = wp_stages(FH);
    constexpr int STAGE = wp_stage_bytes(FH);
    constexpr int TMEM_COLS = PP_TOKENS * FH;
    static_assert(FH * PP_TOKENS * PF_BM * 2 <= NS * STAGE, "the epilogue tiles reuse the ring memory");
    static_assert(NS <= 8, "barrier arrays hold eight stages");
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);    // [8]: my copies (+ on the leader: rank 1's forward)
    uint64_t* done = full + 8;                             // [8]: the UMMAs of the stage are complete (both CTAs)
    uint64_t* acc_full = done + 8;                         // [1]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    volatile unsigned int* go_flag = abort_flag + 1;
    unsigned char* stages = smem + PF_HEADER_BYTES;

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const unsigned int m0 = (blockIdx.x >> 1) * PP_TOKENS;    // first token of the pair's tile
    unsigned int si = 0;
    if (p.n_seg > 1 && blockIdx.y >= p.seg[1].tile0) { si = 1; }
    if (p.n_seg > 2 && blockIdx.y >= p.seg[2].tile0) { si = 2; }
    const PrefillSeg& g = p.seg[si];
    const unsigned int n0 = (blockIdx.y - g.tile0) * (2 * PF_BM * FH);    // first feature of the pair's tile
    const unsigned int n_kblocks = p.K / WP_BK;
    const unsigned int tile_tokens = min((unsigned int)PP_TOKENS, p.M - m0);
    const unsigned int live = (tile_tokens + 15u) & ~15u;    // UMMA N; each CTA supplies live / 2 token rows

    if (threadIdx.x == 0)
    {
        for (unsigned int s = 0; s < (unsigned int)NS; s++)
        {
            mbar_init(full + s, 1 + (rank == 0 ? 1 : 0));
            mbar_init(done + s, 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) { tmem_alloc_pair(tmem_base_slot, TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // both CTAs' barriers exist before any remote arrive, copy or commit
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0)
    {
        // =========================== TMA lane: my weight tiles and my half of the activations ===========================
        if (lane == 0)
        {
            bool ok = true;
            unsigned int issued = 0;
            for (unsigned int kb = 0; kb < n_kblocks; kb++)
            {
                const unsigned int s = kb % NS;
                if (kb >= (unsigned int)NS && (*abort_flag != 0 || !mbar_wait_bounded(done + s, ((kb / NS) - 1u) & 1u)))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                    break;
                }
                unsigned char* st = stages + s * STAGE;
                mbar_expect_tx(full + s, STAGE);
#pragma unroll
                for (int fh = 0; fh < FH; fh++)
                {
                    // feature tile fh of the pair = rows 0..127 from rank 0, 128..255 from rank 1; rows past N are zero-filled
                    tma_load_2d(st + fh * WP_TILE_BYTES, &tmW.w[si], (int)(kb * WP_BK), (int)(n0 + (fh * 2 + rank) * PF_BM), full + s);
                }
                tma_load_2d(st + FH * WP_TILE_BYTES, &tmX, (int)(kb * WP_BK), (int)(m0 + rank * (live / 2)), full + s);
                mbar_arrive(full + s);
                issued = kb + 1;
            }
            if (!ok)
            {
                // wait (bounded) for my copies in flight before the CTA may leave
                const unsigned int first = issued > (unsigned int)NS ? issued - NS : 0;
                for (unsigned int kb = first; kb < issued; kb++)
                {
                    const unsigned long long t0 = global_timer_ns();
                    while (!mbar_try_wait(full + (kb % NS), (kb / NS) & 1u) && global_timer_ns() - t0 < 100000ull) {}
                }
            }
        }
    }
    else if (warp == 1)
    {
        if (lane == 0 && rank != 0)
        {
            // =========================== rank 1: forward "stage full" to the leader ===========================
            const uint32_t peer_bar0 = map_to_cta(full, 0);
            for (unsigned int kb = 0; kb < n_kblocks; kb++)
            {
                const unsigned int s = kb % NS;
                const bool w = *abort_flag == 0 && mbar_wait_bounded(full + s, (kb / NS) & 1u);
                if (!w)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    *abort_flag = 1;
                    break;
                }
                mbar_arrive_cluster(peer_bar0 + s * 8);
            }
        }
        else if (rank == 0)
        {
            // =========================== leader: UMMA warp ===========================
            bool ok = true;
            const uint32_t idesc = umma_idesc_f8(false, false, 2 * PF_BM, live);
            for (unsigned int kb = 0; kb < n_kblocks && ok; kb++)
            {
                const unsigned int s = kb % NS;
                const bool w = *abort_flag == 0 && mbar_wait_bounded(full + s, (kb / NS) & 1u);
                if (!w)
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
                const uint32_t a_addr = smem_u32(stages + s * STAGE);
                const uint32_t b_addr = a_addr + FH * WP_TILE_BYTES;
                if (elect_one())
                {
#pragma unroll
                    for (int k = 0; k < WP_BK / 32; k++)
                    {
#pragma unroll
                        for (int fh = 0; fh < FH; fh++)
                        {
                            umma_f8_pair(tmem_base + fh * PP_TOKENS, umma_desc_kmajor_sw128(a_addr + fh * WP_TILE_BYTES + k * 32),
                                umma_desc_kmajor_sw128(b_addr + k * 32), idesc, (kb | (unsigned int)k) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit_pair(done + s);
                }
                __syncwarp();
            }
            __syncwarp();
            // also on the abort path: the barrier completes once the UMMAs in flight have stopped reading both CTAs' shared memory
            if (elect_one()) { umma_commit_pair(acc_full); }
        }
    }
    else
    {
        // =========================== epilogue (warps 2..9): my 128*FH features x the live tokens ===========================
        if (!mbar_wait_bounded(acc_full, 0))
        {
            atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
            *abort_flag = 1;
        }
        // one decision for all epilogue warps (they meet at a named barrier below): taken by one thread between two barriers
        bar_sync_named(1, 32 * WP_EPI_WARPS);
        if (threadIdx.x == 64) { *go_flag = (*abort_flag == 0 && *reinterpret_cast<volatile unsigned int*>(p.status) == 0) ? 1u : 0u; }
        bar_sync_named(1, 32 * WP_EPI_WARPS);
        const bool ok = *go_flag != 0;
        tc_fence_after();
        const unsigned int quarter = warp & 3u;                   // the TMEM lane quarter this warp may read
        const unsigned int cbeg = ((warp - 2u) >> 2) * (PP_TOKENS / 2);    // two warps per quarter split the token columns
        const float act_inv = p.inv_scale != nullptr ? __ldg(p.inv_scale) : p.act_inv;
        if (ok && n_kblocks > 0 && g.y_tma != 0)
        {
            // BF16 tiles [256 tokens][128 features] in the idle stage memory, then one TMA store each; the store clips
            // rows past M and features past N
#pragma unroll
            for (int fh = 0; fh < FH; fh++)
            {
                const uint32_t ytile = smem_u32(stages) + fh * (PP_TOKENS * PF_BM * 2) + (quarter * 32 + lane) * 2;
                for (unsigned int c0 = cbeg; c0 < cbeg + PP_TOKENS / 2 && c0 < tile_tokens; c0 += 32)
                {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + fh * PP_TOKENS + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                    {
                        sts16(ytile + (c0 + j) * (PF_BM * 2),
                            __bfloat16_as_ushort(__float2bfloat16_rn(g.alpha * ((__uint_as_float(r[j]) * act_inv) * g.post_scale))));
                    }
                }
            }
            fence_proxy_async();
            bar_sync_named(1, 32 * WP_EPI_WARPS);
            if (threadIdx.x == 64)
            {
#pragma unroll
                for (int fh = 0; fh < FH; fh++)
                {
                    const unsigned int nf = n0 + (fh * 2 + rank) * PF_BM;
                    if (nf < g.N) { tma_store_2d(&tmY.m[si], stages + fh * (PP_TOKENS * PF_BM * 2), (int)nf, (int)m0); }
                }
                tma_store_commit_and_wait_read();
            }
        }
        else if (ok && n_kblocks > 0)
        {
#pragma unroll
            for (int fh = 0; fh < FH; fh++)
            {
                const unsigned int n = n0 + (fh * 2 + rank) * PF_BM + quarter * 32 + lane;
                for (unsigned int c0 = cbeg; c0 < cbeg + PP_TOKENS / 2 && c0 < tile_tokens; c0 += 32)
                {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + fh * PP_TOKENS + c0, r);
                    tmem_ld_wait();
                    if (n < g.N)
                    {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                        {
                            if (c0 + j >= tile_tokens) { continue; }
                            const long long yi = (long long)(m0 + c0 + j) * g.ldy_m + (long long)n * g.ldy_n;
                            float o = g.alpha * ((__uint_as_float(r[j]) * act_inv) * g.post_scale);
                            if (p.out_f32 == 1u)
                            {
                                float* y = reinterpret_cast<float*>(g.Y) + yi;
                                if (g.beta != 0.f) { o += g.beta * *y; }
                                *y = o;
                            }
                            else if (p.out_f32 == 3u)
                            {
                                // E4M3 output: the BF16 result re-encoded at scale 1 with the reference's encoder, beta
                                // ignored (cccc/cublas_real.h:787-834)
                                reinterpret_cast<uint8_t*>(g.Y)[yi] = float_to_e4m3(__bfloat162float(__float2bfloat16_rn(o)), 1.0f);
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
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // neither CTA frees TMEM or leaves while the other may still use the pair
    if (warp == 1) { tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

// ---- the persistent form -----------------------------------------------------------------------------------
// One CTA pair per SM pair walks tiles of 256 features x 256 tokens (tile t, t + pairs, ...; the token tile runs
// fastest, so the pairs of a wave share a few weight tiles and all of the activations in L2).  Two accumulators of 256
// columns: while the eight epilogue warps of each CTA read tile i out of tensor memory, convert it and hand it to a TMA
// store, the leader already issues the UMMAs of tile i + 1 into the other accumulator, and the copy ring (four stages,
// counted across tiles) never drains.  acc_full[a] (leader's commit, both CTAs) hands an accumulator to the epilogues;
// acc_empty[a] on the leader collects one arrive from each CTA's epilogue once its warps have read their half.
constexpr int WQ_STAGES = 4;
constexpr int WQ_STAGE_BYTES = 2 * WP_TILE_BYTES;
constexpr int WQ_YTILE_BYTES = PP_TOKENS * PF_BM * 2;    // 64 KB: [256 tokens][128 features] BF16
constexpr int WQ_SMEM_BYTES = PF_HEADER_BYTES + WQ_STAGES * WQ_STAGE_BYTES + WQ_YTILE_BYTES + 1024;

__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(WP_THREADS, 1)
    gemm_w8a8_pair_persistent_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ StreamWMaps tmW,
        const __grid_constant__ PrefillYMaps tmY, const NativeParams p, const unsigned int token_tiles, const unsigned int total_tiles)
{
    extern __shared__ unsigned char wp_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(wp_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr unsigned int NS = WQ_STAGES;
    constexpr int TMEM_COLS = 2 * PP_TOKENS;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);    // [8]
    uint64_t* done = full + 8;                             // [8]
    uint64_t* acc_full = done + 8;                         // [2]
    uint64_t* acc_empty = acc_full + 2;                    // [2] (used on the leader)
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    unsigned char* stages = smem + PF_HEADER_BYTES;
    unsigned char* ytile_mem = stages + WQ_STAGES * WQ_STAGE_BYTES;

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const unsigned int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const unsigned int n_kblocks = p.K / WP_BK;
    // tile t -> member si, first feature n0, first token m0
    auto coords = [&](unsigned int t, unsigned int& si, unsigned int& n0, unsigned int& m0) {
        const unsigned int ft = t / token_tiles;
        m0 = (t % token_tiles) * PP_TOKENS;
        si = 0;
        if (p.n_seg > 1 && ft >= p.seg[1].tile0) { si = 1; }
        if (p.n_seg > 2 && ft >= p.seg[2].tile0) { si = 2; }
        n0 = (ft - p.seg[si].tile0) * (2 * PF_BM);
    };

    if (threadIdx.x == 0)
    {
        for (unsigned int s = 0; s < NS; s++)
        {
            mbar_init(full + s, 1 + (rank == 0 ? 1 : 0));
            mbar_init(done + s, 1);
        }
        for (unsigned int a = 0; a < 2; a++)
        {
            mbar_init(acc_full + a, 1);
            mbar_init(acc_empty + a, 2);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) { tmem_alloc_pair(tmem_base_slot, TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0)
    {
        // =========================== TMA lane ===========================
        if (lane == 0)
        {
            bool ok = true;
            unsigned int it = 0;    // k blocks issued so far, over all tiles
            for (unsigned int t = pair; t < total_tiles && ok; t += n_pairs)
            {
                unsigned int si, n0, m0;
                coords(t, si, n0, m0);
                const unsigned int live = (min((unsigned int)PP_TOKENS, p.M - m0) + 15u) & ~15u;
                for (unsigned int kb = 0; kb < n_kblocks; kb++, it++)
                {
                    const unsigned int s = it % NS;
                    if (it >= NS && (*abort_flag != 0 || !mbar_wait_bounded(done + s, ((it / NS) - 1u) & 1u)))
                    {
                        ok = false;
                        atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                        *abort_flag = 1;
                        break;
                    }
                    unsigned char* st = stages + s * WQ_STAGE_BYTES;
                    mbar_expect_tx(full + s, WQ_STAGE_BYTES);
                    tma_load_2d(st, &tmW.w[si], (int)(kb * WP_BK), (int)(n0 + rank * PF_BM), full + s);
                    tma_load_2d(st + WP_TILE_BYTES, &tmX, (int)(kb * WP_BK), (int)(m0 + rank * (live / 2)), full + s);
                    mbar_arrive(full + s);
                }
            }
            if (!ok)
            {
                // wait (bounded) for my copies in flight before the CTA may leave
                const unsigned int first = it > NS ? it - NS : 0;
                for (unsigned int j = first; j < it; j++)
                {
                    const unsigned long long t0 = global_timer_ns();
                    while (!mbar_try_wait(full + (j % NS), (j / NS) & 1u) && global_timer_ns() - t0 < 100000ull) {}
                }
            }
        }
    }
    else if (warp == 1)
    {
        if (lane == 0 && rank != 0)
        {
            // =========================== rank 1: forward "stage full" to the leader ===========================
            const uint32_t peer_bar0 = map_to_cta(full, 0);
            bool ok = true;
            unsigned int it = 0;
            for (unsigned int t = pair; t < total_tiles && ok; t += n_pairs)
            {
                for (unsigned int kb = 0; kb < n_kblocks; kb++, it++)
                {
                    const unsigned int s = it % NS;
                    if (*abort_flag != 0 || !mbar_wait_bounded(full + s, (it / NS) & 1u))
                    {
                        ok = false;
                        atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                        *abort_flag = 1;
                        break;
                    }
                    mbar_arrive_cluster(peer_bar0 + s * 8);
                }
            }
        }
        else if (rank == 0)
        {
            // =========================== leader: UMMA warp ===========================
            bool ok = true;
            unsigned int it = 0, i = 0;
            for (unsigned int t = pair; t < total_tiles && ok; t += n_pairs, i++)
            {
                unsigned int si, n0, m0;
                coords(t, si, n0, m0);
                const unsigned int live = (min((unsigned int)PP_TOKENS, p.M - m0) + 15u) & ~15u;
                const uint32_t idesc = umma_idesc_f8(false, false, 2 * PF_BM, live);
                const unsigned int acc = i & 1u;
                // the epilogues of both CTAs have read this accumulator's previous tile
                if (i >= 2 && (*abort_flag != 0 || !mbar_wait_bounded_cluster(acc_empty + acc, ((i >> 1) - 1u) & 1u)))
                {
                    ok = false;
                    if (lane == 0)
                    {
                        atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                        *abort_flag = 1;
                    }
                    break;
                }
                tc_fence_after();
                for (unsigned int kb = 0; kb < n_kblocks; kb++, it++)
                {
                    const unsigned int s = it % NS;
                    if (*abort_flag != 0 || !mbar_wait_bounded(full + s, (it / NS) & 1u))
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
                    const uint32_t a_addr = smem_u32(stages + s * WQ_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + WP_TILE_BYTES;
                    if (elect_one())
                    {
#pragma unroll
                        for (int k = 0; k < WP_BK / 32; k++)
                        {
                            umma_f8_pair(tmem_base + acc * PP_TOKENS, umma_desc_kmajor_sw128(a_addr + k * 32), umma_desc_kmajor_sw128(b_addr + k * 32),
                                idesc, (kb | (unsigned int)k) != 0 ? 1u : 0u);
                        }
                        umma_commit_pair(done + s);
                    }
                    __syncwarp();
                }
                __syncwarp();
                // also when the k loop gave up: the barrier completes once the UMMAs in flight have stopped
                if (elect_one()) { umma_commit_pair(acc_full + acc); }
                __syncwarp();
            }
        }
    }
    else
    {
        // =========================== epilogue (warps 2..9) ===========================
        // The two named barriers of a tile are met by every epilogue thread whatever happened: a thread whose wait ran
        // out only skips the data work.
        bool ok = true;
        const unsigned int quarter = warp & 3u;
        const unsigned int cbeg = ((warp - 2u) >> 2) * (PP_TOKENS / 2);
        const float act_inv = p.inv_scale != nullptr ? __ldg(p.inv_scale) : p.act_inv;
        const uint32_t acc_empty_leader = map_to_cta(acc_empty, 0);
        unsigned int i = 0;
        for (unsigned int t = pair; t < total_tiles; t += n_pairs, i++)
        {
            const unsigned int acc = i & 1u;
            unsigned int si, n0, m0;
            coords(t, si, n0, m0);
            const PrefillSeg& g = p.seg[si];
            const unsigned int tile_tokens = min((unsigned int)PP_TOKENS, p.M - m0);
            if (ok && (*abort_flag != 0 || !mbar_wait_bounded(acc_full + acc, (i >> 1) & 1u)))
            {
                ok = false;
                atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                *abort_flag = 1;
            }
            if (*reinterpret_cast<volatile unsigned int*>(p.status) != 0) { ok = false; }
            tc_fence_after();
            bar_sync_named(1, 32 * WP_EPI_WARPS);    // the previous tile's store has read the staging tile (thread 64 waited)
            const unsigned int n = n0 + rank * PF_BM + quarter * 32 + lane;
            if (ok && n_kblocks > 0)
            {
                const uint32_t ytile = smem_u32(ytile_mem) + (quarter * 32 + lane) * 2;
                for (unsigned int c0 = cbeg; c0 < cbeg + PP_TOKENS / 2 && c0 < tile_tokens; c0 += 32)
                {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * PP_TOKENS + c0, r);
                    tmem_ld_wait();
                    if (g.y_tma != 0)
                    {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                        {
                            sts16(ytile + (c0 + j) * (PF_BM * 2),
                                __bfloat16_as_ushort(__float2bfloat16_rn(g.alpha * ((__uint_as_float(r[j]) * act_inv) * g.post_scale))));
                        }
                    }
                    else if (n < g.N)
                    {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                        {
                            if (c0 + j >= tile_tokens) { continue; }
                            const long long yi = (long long)(m0 + c0 + j) * g.ldy_m + (long long)n * g.ldy_n;
                            float o = g.alpha * ((__uint_as_float(r[j]) * act_inv) * g.post_scale);
                            if (p.out_f32 == 1u)
                            {
                                float* y = reinterpret_cast<float*>(g.Y) + yi;
                                if (g.beta != 0.f) { o += g.beta * *y; }
                                *y = o;
                            }
                            else if (p.out_f32 == 3u) { reinterpret_cast<uint8_t*>(g.Y)[yi] = float_to_e4m3(__bfloat162float(__float2bfloat16_rn(o)), 1.0f); }
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
            tc_fence_before();
            fence_proxy_async();
            bar_sync_named(2, 32 * WP_EPI_WARPS);    // every warp has read its part of the accumulator and written the staging tile
            if (threadIdx.x == 64)
            {
                if (rank == 0) { mbar_arrive(acc_empty + acc); }
                else { mbar_arrive_cluster_release(acc_empty_leader + acc * 8); }
                const unsigned int nf = n0 + rank * PF_BM;
                if (ok && n_kblocks > 0 && g.y_tma != 0 && nf < g.N) { tma_store_2d(&tmY.m[si], ytile_mem, (int)nf, (int)m0); }
                tma_store_commit_and_wait_read();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // neither CTA frees TMEM or leaves while the other may still use the pair
    if (warp == 1) { tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

// Feature tiles of 256 * fh features over the members of a launch; fills tile0 of every member.
static inline unsigned int wp_feature_tiles(NativeParams& np, unsigned int fh)
{
    unsigned int tiles = 0;
    for (unsigned int j = 0; j < np.n_seg; j++)
    {
        np.seg[j].tile0 = tiles;
        tiles += (np.seg[j].N + 2 * PF_BM * fh - 1) / (2 * PF_BM * fh);
    }
    return tiles;
}

// Which form (1: one 256-feature tile per pair, 2: one 512-feature tile, 3: the persistent form).  A model fitted to
// measurements at K = 4096 and 12288, 256 to 4096 tokens, in units of one 256-feature k block: a tile costs its k blocks
// plus about ten for start-up and epilogue, which the persistent form pays once per launch instead of once per tile; a
// 512-feature tile costs 1.84 per k block (it stages a third less per flop) plus fifteen.  What decides is mostly how
// the tiles round up to whole rounds of the SM pairs.
static inline unsigned int wp_pick_fh(const NativeParams& np_in, int sm_count)
{
    NativeParams np = np_in;
    const unsigned long long slots = (unsigned long long)sm_count / 2;
    const unsigned long long mt = (np.M + PP_TOKENS - 1) / PP_TOKENS;
    const unsigned long long p1 = mt * wp_feature_tiles(np, 1), p2 = mt * wp_feature_tiles(np, 2);
    const double nkb = (double)(np.K / WP_BK);
    const double r1 = (double)((p1 + slots - 1) / slots), r2 = (double)((p2 + slots - 1) / slots);
    const double c1 = r1 * (nkb + 10.0), c3 = r1 * nkb + 10.0, c2 = r2 * (1.84 * nkb + 15.0);
    if (r1 <= 1.0) { return c2 < c1 ? 2u : 1u; }
    return c2 < c3 ? 2u : 3u;
}

template <int FH>
static int launch_w8a8_pair_fh(const CUtensorMap& tmX, const StreamWMaps& tmW, const PrefillYMaps& tmY, const NativeParams& np, unsigned int feature_tiles,
    int device, cudaStream_t stream)
{
    auto kernel = gemm_w8a8_pair_kernel<FH>;
    static std::atomic<bool> attr_set[64];    // zero-initialised; setting the attribute twice is harmless
    if (!attr_set[device].load(std::memory_order_acquire))
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wp_smem_bytes(FH)) != cudaSuccess)
        {
            report_launch("gemm_w8a8_bf16");
            return 1;
        }
        attr_set[device].store(true, std::memory_order_release);
    }
    const dim3 grid(2 * ((np.M + PP_TOKENS - 1) / PP_TOKENS), feature_tiles);
    count_launch();
    kernel<<<grid, WP_THREADS, wp_smem_bytes(FH), stream>>>(tmX, tmW, tmY, np);
    return report_launch("gemm_w8a8_bf16");
}

// The launch behind the quantiser for more than 32 tokens.  np carries the members (W, Y, N, ldw, ldy, alpha, beta,
// post_scale), M, K, out_f32, status and inv_scale (or act_inv); Q is the [M][K] E4M3 activations, rows ldq bytes apart.  fh: 0 picks the form (wp_pick_fh).
// Returns -1 for what this path does not serve.
static int launch_w8a8_pair(NativeParams np, const W8A8Member* mem, const uint8_t* Q, unsigned int ldq, int device, int sm_count, unsigned int fh,
    cudaStream_t stream)
{
    if (fh < 1 || fh > 3) { fh = wp_pick_fh(np, sm_count); }
    const bool persistent = fh == 3;    // 256-feature tiles walked by one pair per SM pair
    if (persistent) { fh = 1; }
    const unsigned int feature_tiles = wp_feature_tiles(np, fh);
    if (feature_tiles == 0 || feature_tiles > 65535u || (np.M + PP_TOKENS - 1) / PP_TOKENS > 32767u) { return -1; }
    CUtensorMap tmX;
    StreamWMaps tmW;
    PrefillYMaps tmY;
    memset(&tmW, 0, sizeof(tmW));
    memset(&tmY, 0, sizeof(tmY));
    bool ok = make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Q, np.K, np.M, ldq, WP_BK, PP_HALF, true);
    for (unsigned int j = 0; j < (unsigned int)PF_MAX_GROUP && ok; j++)
    {
        const W8A8Member& m = mem[j < np.n_seg ? j : 0];
        ok = make_map_2d(&tmW.w[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, m.W, np.K, m.N_out, m.ldw, WP_BK, PF_BM, true);
    }
    if (!ok) { return -1; }
    for (unsigned int j = 0; j < np.n_seg; j++)
    {
        PrefillSeg& g = np.seg[j];
        // BF16 output with contiguous features and no accumulate: the epilogue writes whole tiles with TMA stores
        g.y_tma = 0;
        if ((np.out_f32 == 0u || np.out_f32 == 2u) && g.beta == 0.f && g.ldy_n == 1 && (g.ldy_m % 8) == 0 && g.ldy_m >= (long long)g.N
            && (reinterpret_cast<uintptr_t>(g.Y) & 15u) == 0
            && make_map_2d(&tmY.m[j], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g.Y, g.N, np.M, (unsigned long long)g.ldy_m * 2, PF_BM, PP_TOKENS, false))
        {
            g.y_tma = 1;
        }
    }
    if (persistent)
    {
        auto kernel = gemm_w8a8_pair_persistent_kernel;
        static std::atomic<bool> attr_set[64];
        if (!attr_set[device].load(std::memory_order_acquire))
        {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WQ_SMEM_BYTES) != cudaSuccess)
            {
                report_launch("gemm_w8a8_bf16");
                return 1;
            }
            attr_set[device].store(true, std::memory_order_release);
        }
        const unsigned int token_tiles = (np.M + PP_TOKENS - 1) / PP_TOKENS;
        const unsigned long long total = (unsigned long long)token_tiles * feature_tiles;
        if (total > 0x7FFFFFFFull) { return -1; }
        const unsigned int pairs = (unsigned int)(total < (unsigned long long)(sm_count / 2) ? total : (unsigned long long)(sm_count / 2));
        count_launch();
        kernel<<<2 * pairs, WP_THREADS, WQ_SMEM_BYTES, stream>>>(tmX, tmW, tmY, np, token_tiles, (unsigned int)total);
        return report_launch("gemm_w8a8_bf16");
    }
    return fh == 2 ? launch_w8a8_pair_fh<2>(tmX, tmW, tmY, np, feature_tiles, device, stream)
                   : launch_w8a8_pair_fh<1>(tmX, tmW, tmY, np, feature_tiles, device, stream);
}

}    // namespace b200
