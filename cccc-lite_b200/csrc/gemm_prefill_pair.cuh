// Prefill-side quantized-weight linear on CTA pairs (tcgen05.mma with cta_group::2).
//
// Two CTAs on the two SMs of a TPC form a cluster and compute 256*FH output features x up to 256
// tokens over the whole K range.  Each CTA converts the weight tiles of its own 128*FH features and
// loads HALF of the token tile; one lane of the leader CTA (cluster rank 0) issues UMMAs of
// M=256, N=tokens, K=16 that read the A rows of both CTAs and the B rows of both halves, and each
// CTA's tensor core accumulates its own 128 features in its own TMEM.  Against the one-CTA kernel
// this halves the activation bytes each SM copies into and reads out of shared memory per flop,
// which is the bound of that kernel (see gemm_prefill.cuh).
//
// Per 64-wide k block and CTA:
//   * the TMA lane copies [128 tokens][64 k] BF16 activations (swizzle 128 B, rows past M zero),
//   * eight warps dequantise [128*FH features][64 k] weights into the swizzled A stage,
//   * rank 1 forwards "my stage is full" to a barrier of the leader (remote mbarrier arrive),
//   * the leader issues 4*FH UMMAs and commits to the stage's "empty" barrier of BOTH CTAs.
// After the last k block each CTA reads its accumulator (tcgen05.ld) and stores its features.
// Every mbarrier wait is bounded; a CTA whose wait ran out raises the status word and drains.  Both
// CTAs always reach the cluster barrier before the TMEM columns are freed, so neither leaves while
// the other may still read its shared memory.
#pragma once

#include "gemm_prefill.cuh"

namespace b200
{

constexpr int PP_TOKENS = 256;    // tokens per CTA pair (UMMA N)
constexpr int PP_HALF = 128;      // tokens each CTA stages
__host__ __device__ constexpr int pp_stages(int fh) { return fh == 2 ? 4 : 3; }
__host__ __device__ constexpr int pp_stage_bytes(int fh) { return pf_a_bytes(fh) + PP_HALF * PF_BK * 2; }
__host__ __device__ constexpr int pp_smem_bytes(int fh) { return PF_HEADER_BYTES + pp_stages(fh) * pp_stage_bytes(fh) + 1024; }

// ---- cluster / cta_group::2 wrappers ------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait_cluster(bar, parity)) { return true; }
    const unsigned long long t0 = global_timer_ns();
    unsigned int spins = 0;
    while (!mbar_try_wait_cluster(bar, parity))
    {
        if ((++spins & 0x3FFu) == 0 && global_timer_ns() - t0 > kWaitLimitNs) { return false; }
    }
    return true;
}
// One warp of EACH CTA of the pair allocates; both receive the same column range.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of both CTAs: 128 rows each] * B[smem of both CTAs: N/2 rows each].
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the barrier at this offset in both CTAs once every UMMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"(mask)
                 : "memory");
}

// ---- the kernel ------------------------------------------------------------------------------------
template <int WT, bool SCALED, int FH>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PF_THREADS, FH > 1 ? 1 : 2)
    gemm_wq_prefill_pair_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY, const PrefillParams p)
{
    extern __shared__ unsigned char pf_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int ST = pp_stages(FH);
    constexpr int A_BYTES = pf_a_bytes(FH);
    constexpr int X_BYTES = PP_HALF * PF_BK * 2;
    constexpr int STAGE_BYTES = pp_stage_bytes(FH);
    constexpr int TMEM_COLS = PP_TOKENS * FH;
    uint64_t* full_x = reinterpret_cast<uint64_t*>(smem);    // [ST] my activation half has landed
    uint64_t* full_a = full_x + 4;                           // [ST] my weight tile is converted
    uint64_t* peer_full = full_a + 4;                        // [ST] leader only: rank 1's stage is full
    uint64_t* empty = peer_full + 4;                         // [ST] the UMMAs that read the stage are done
    uint64_t* acc_full = empty + 4;                          // [1]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    unsigned char* stages = smem + PF_HEADER_BYTES;
    static_assert(ST <= 4, "barrier arrays hold four stages");

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const unsigned int m0 = (blockIdx.x >> 1) * PP_TOKENS;            // first token of the pair's tile
    const unsigned int n0 = blockIdx.y * (2 * PF_BM * FH);            // first feature of the pair's tile
    const unsigned int n_kblocks = p.K / PF_BK;
    const unsigned int tile_tokens = min((unsigned int)PP_TOKENS, p.M - m0);
    const unsigned int live = (tile_tokens + 15u) & ~15u;             // UMMA N; each CTA supplies live/2 token rows
    const unsigned int my_tok0 = m0 + rank * (live / 2);

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < ST; s++)
        {
            mbar_init(full_x + s, 1);
            mbar_init(full_a + s, PF_DQ_WARPS);
            mbar_init(peer_full + s, 1);
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == PF_DQ_WARPS + 1) { tmem_alloc_pair(tmem_base_slot, TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // both CTAs' barriers exist before any remote arrive or commit
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == PF_DQ_WARPS)
    {
        // =========================== TMA lane: my half of the activations ===========================
        if (lane == 0)
        {
            bool ok = true;
            unsigned int issued = 0;
            for (unsigned int kb = 0; kb < n_kblocks; kb++)
            {
                const unsigned int s = kb % ST;
                if (kb >= ST && (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((kb / ST) - 1) & 1u)))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                    break;
                }
                mbar_expect_tx(full_x + s, X_BYTES);
                tma_load_2d(stages + s * STAGE_BYTES + A_BYTES, &tmX, (int)(kb * PF_BK), (int)my_tok0, full_x + s);
                mbar_arrive(full_x + s);
                issued = kb + 1;
            }
            if (!ok)
            {
                const unsigned int first = issued > ST ? issued - ST : 0;
                for (unsigned int kb = first; kb < issued; kb++) { mbar_wait_bounded(full_x + (kb % ST), (kb / ST) & 1u); }
            }
        }
    }
    else if (warp == PF_DQ_WARPS + 1)
    {
        if (lane == 0 && rank != 0)
        {
            // =========================== rank 1: forward "stage full" to the leader ===========================
            for (unsigned int kb = 0; kb < n_kblocks; kb++)
            {
                const unsigned int s = kb % ST;
                const uint32_t par = (kb / ST) & 1u;
                if (*abort_flag != 0 || !mbar_wait_bounded(full_x + s, par) || !mbar_wait_bounded(full_a + s, par))
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    *abort_flag = 1;
                    break;
                }
                mbar_arrive_remote(peer_full + s, 0);
            }
        }
        else if (lane == 0)
        {
            // =========================== leader: UMMA lane ===========================
            bool ok = true;
            const uint32_t idesc = umma_idesc_bf16(2 * PF_BM, live);
            for (unsigned int kb = 0; kb < n_kblocks && ok; kb++)
            {
                const unsigned int s = kb % ST;
                const uint32_t par = (kb / ST) & 1u;
                if (*abort_flag != 0 || !mbar_wait_bounded(full_x + s, par) || !mbar_wait_bounded(full_a + s, par)
                    || !mbar_wait_bounded_cluster(peer_full + s, par))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(stages + s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < PF_BK / 16; k++)
                {
#pragma unroll
                    for (int fh = 0; fh < FH; fh++)
                    {
                        umma_bf16_pair(tmem_base + fh * PP_TOKENS, umma_desc_kmajor_sw128(a_addr + fh * (PF_BM * PF_BK * 2) + k * 32),
                            umma_desc_kmajor_sw128(b_addr + k * 32), idesc, (kb | (unsigned int)k) != 0 ? 1u : 0u);
                    }
                }
                umma_commit_pair(empty + s);
            }
            // also on the abort path: the barrier completes once the UMMAs in flight have stopped
            // reading both CTAs' shared memory; the epilogue warps then see the abort flag or the status
            umma_commit_pair(acc_full);
        }
    }
    else
    {
        // =========================== dequantise, then epilogue (warps 0..7) ===========================
        const unsigned int tid = threadIdx.x;    // 0..255
        constexpr int NP = 2 * FH;               // (row, 16-element group) pieces per thread per k block
        unsigned int prow[NP], pq[NP], pfeat[NP];
#pragma unroll
        for (int i = 0; i < NP; i++)
        {
            const unsigned int piece = tid + 256u * i;
            prow[i] = piece >> 2;    // row within the A stage: 128 rows per feature tile
            pq[i] = piece & 3u;
            // feature tile fh of the pair = rows 0..127 from rank 0, 128..255 from rank 1
            pfeat[i] = n0 + ((prow[i] >> 7) * 2 + rank) * PF_BM + (prow[i] & 127u);
        }
        uint4 raw8[2][NP];
        uint2 raw4[2][NP];
        uint32_t rawsc[2][NP];
        auto load_raw = [&](unsigned int kb, int slot) {
#pragma unroll
            for (int i = 0; i < NP; i++)
            {
                raw8[slot][i] = make_uint4(0, 0, 0, 0);
                raw4[slot][i] = make_uint2(0, 0);
                rawsc[slot][i] = 0;
                if (pfeat[i] < p.N)
                {
                    const size_t e = (size_t)pfeat[i] * p.ldw + (size_t)kb * PF_BK + pq[i] * 16;
                    if (WT == DT_FP4)
                    {
                        raw4[slot][i] = __ldg(reinterpret_cast<const uint2*>(p.W + e / 2));
                        rawsc[slot][i] = __ldg(p.blk + e / 16);
                    }
                    else { raw8[slot][i] = __ldg(reinterpret_cast<const uint4*>(p.W + e)); }
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
                    for (int j = 0; j < 4; j++) { dequant_fp8x4<WT, SCALED>(w[j], p.w_scale, out[i][2 * j], out[i][2 * j + 1]); }
                }
            }
            if (kb + 2 < n_kblocks) { load_raw(kb + 2, slot); }
        };
        // The conversion of block kb+1 is issued between the stores of block kb and their proxy fence,
        // so the fence finds the stores already performed.
        uint32_t out[NP][8];
        if (n_kblocks > 0) { convert_and_refill(0, 0, out); }
        for (unsigned int kb = 0; kb < n_kblocks; kb++)
        {
            const unsigned int s = kb % ST;
            if (ok && kb >= ST && (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((kb / ST) - 1) & 1u)))
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
                const uint32_t a_addr = smem_u32(stages + s * STAGE_BYTES);
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

        // ---- epilogue: my 128*FH features x all live tokens ----
        if (!mbar_wait_bounded(acc_full, 0))
        {
            ok = false;
            atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
            *abort_flag = 1;
        }
        if (*abort_flag != 0 || *reinterpret_cast<volatile unsigned int*>(p.status) != 0) { ok = false; }
        tc_fence_after();
        if (ok && n_kblocks > 0 && p.y_tma != 0)
        {
            // BF16 tile [256 tokens][128 features] per feature tile in the idle stage memory, then TMA stores
            const unsigned int quarter = warp & 3u;
            const unsigned int half = warp >> 2;
#pragma unroll
            for (int fh = 0; fh < FH; fh++)
            {
                const uint32_t ytile = smem_u32(stages) + fh * (PP_TOKENS * PF_BM * 2) + (quarter * 32 + lane) * 2;
                for (unsigned int c0 = half * (PP_TOKENS / 2); c0 < half * (PP_TOKENS / 2) + PP_TOKENS / 2 && c0 < tile_tokens; c0 += 32)
                {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + fh * PP_TOKENS + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                    {
                        sts16(ytile + (c0 + j) * (PF_BM * 2), __bfloat16_as_ushort(__float2bfloat16_rn(p.alpha * (__uint_as_float(r[j]) * p.post_scale))));
                    }
                }
            }
            fence_proxy_async();
            bar_sync_named(1, 32 * PF_DQ_WARPS);
            if (tid == 0)
            {
#pragma unroll
                for (int fh = 0; fh < FH; fh++)
                {
                    tma_store_2d(&tmY, stages + fh * (PP_TOKENS * PF_BM * 2), (int)(n0 + (fh * 2 + rank) * PF_BM), (int)m0);
                }
                tma_store_commit_and_wait_read();
            }
        }
        else if (ok && n_kblocks > 0)
        {
            const unsigned int quarter = warp & 3u;
            const unsigned int half = warp >> 2;
#pragma unroll
            for (int fh = 0; fh < FH; fh++)
            {
                const unsigned int n = n0 + (fh * 2 + rank) * PF_BM + quarter * 32 + lane;
                for (unsigned int c0 = half * (PP_TOKENS / 2); c0 < half * (PP_TOKENS / 2) + PP_TOKENS / 2 && c0 < tile_tokens; c0 += 32)
                {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + fh * PP_TOKENS + c0, r);
                    tmem_ld_wait();
                    if (n < p.N)
                    {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                        {
                            const unsigned int m = m0 + c0 + j;
                            if (c0 + j < tile_tokens)
                            {
                                const long long yi = (long long)m * p.ldy_m + (long long)n * p.ldy_n;
                                float o = p.alpha * (__uint_as_float(r[j]) * p.post_scale);
                                if (p.out_f32)
                                {
                                    float* y = reinterpret_cast<float*>(p.Y) + yi;
                                    if (p.beta != 0.f) { o += p.beta * *y; }
                                    *y = o;
                                }
                                else
                                {
                                    uint16_t* y = p.Y + yi;
                                    if (p.beta != 0.f) { o += p.beta * bf16_bits_to_float(*y); }
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
    cluster_sync_all();    // neither CTA frees TMEM or leaves while the other may still use the pair
    if (warp == PF_DQ_WARPS + 1) { tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

template <int WT, bool SCALED, int FH>
static int launch_prefill_pair(const CUtensorMap& tmX, const CUtensorMap& tmY, const PrefillParams& pp, int device, cudaStream_t stream)
{
    auto kernel = gemm_wq_prefill_pair_kernel<WT, SCALED, FH>;
    static bool attr_set[64] = {};
    if (!attr_set[device])
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pp_smem_bytes(FH)) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16");
            return 1;
        }
        attr_set[device] = true;
    }
    const dim3 grid(2 * ((pp.M + PP_TOKENS - 1) / PP_TOKENS), (pp.N + 2 * PF_BM * FH - 1) / (2 * PF_BM * FH));
    count_launch();
    kernel<<<grid, PF_THREADS, pp_smem_bytes(FH), stream>>>(tmX, tmY, pp);
    return report_launch("gemm_wq_bf16");
}

}    // namespace b200
