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
        const float act_inv = __ldg(p.inv_scale);
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

// Which tile shape: a 512-feature tile occupies a pair of SMs for two units of time, a 256-feature tile for one; the
// larger stages a third less per flop, taken as 10 % faster at equal occupancy.
static inline unsigned int wp_pick_fh(const NativeParams& np_in, int sm_count)
{
    NativeParams np = np_in;
    const unsigned long long slots = (unsigned long long)sm_count / 2;
    const unsigned long long mt = (np.M + PP_TOKENS - 1) / PP_TOKENS;
    const unsigned long long p1 = mt * wp_feature_tiles(np, 1), p2 = mt * wp_feature_tiles(np, 2);
    const double c1 = (double)((p1 + slots - 1) / slots), c2 = 2.0 * 0.9 * (double)((p2 + slots - 1) / slots);
    return c2 < c1 ? 2u : 1u;
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
// post_scale), M, K, out_f32, status and inv_scale; Q is the [M][K] E4M3 activations.  fh: 0 picks the tile shape.
// Returns -1 for what this path does not serve.
static int launch_w8a8_pair(NativeParams np, const W8A8Member* mem, const uint8_t* Q, int device, int sm_count, unsigned int fh, cudaStream_t stream)
{
    if (fh != 1 && fh != 2) { fh = wp_pick_fh(np, sm_count); }
    const unsigned int feature_tiles = wp_feature_tiles(np, fh);
    if (feature_tiles == 0 || feature_tiles > 65535u || (np.M + PP_TOKENS - 1) / PP_TOKENS > 32767u) { return -1; }
    CUtensorMap tmX;
    StreamWMaps tmW;
    PrefillYMaps tmY;
    memset(&tmW, 0, sizeof(tmW));
    memset(&tmY, 0, sizeof(tmY));
    bool ok = make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Q, np.K, np.M, np.K, WP_BK, PP_HALF, true);
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
    return fh == 2 ? launch_w8a8_pair_fh<2>(tmX, tmW, tmY, np, feature_tiles, device, stream)
                   : launch_w8a8_pair_fh<1>(tmX, tmW, tmY, np, feature_tiles, device, stream);
}

}    // namespace b200
