// Prefill-side quantized-weight linear on CTA pairs (tcgen05.mma with cta_group::2).
//
// Two CTAs on the two SMs of a TPC form a cluster and compute 256*FH output features x up to 256*TH
// tokens over the whole K range (FH*TH <= 2: 512 TMEM columns per CTA).  Each CTA converts the weight
// tiles of its own 128*FH features and loads HALF of every 256-token tile; one lane of the leader CTA
// (cluster rank 0) issues UMMAs of M=256, N=tokens, K=16 that read the A rows of both CTAs and the B
// rows of both halves, and each CTA's tensor core accumulates its own 128 features in its own TMEM.
// Against the one-CTA kernel a CTA stages half the activation bytes per flop, and with TH=2 also
// converts half the weights per flop, so four stages of 1024 tensor cycles each fit in shared memory:
// enough to cover the latency of the activation loads and of the barrier round trips.
//
// Per 64-wide k block and CTA:
//   * the TMA lane copies TH x [128 tokens][64 k] BF16 activations (swizzle 128 B, rows past M zero),
//   * 8 or 16 warps dequantise [128*FH features][64 k] weights into the swizzled A stage,
//   * both arrive on ONE "full" barrier of the k block (slot kb % 8); one lane of rank 1 forwards its
//     completion to the leader's barrier with ONE remote arrive at CTA scope (remote arrives from all
//     dequantise warps, activation copies completing on the leader's barrier, or a release at
//     cluster scope each measured 40 % slower),
//   * the leader issues 4*FH*TH UMMAs and commits to ONE "done" barrier of the k block in BOTH CTAs,
//     which frees the activation stage and the weight stage (rings of different depth).
// After the last k block each CTA reads its accumulators (tcgen05.ld) and stores its features.
// Every mbarrier wait is bounded; a CTA whose wait ran out raises the status word and drains.  Both
// CTAs always reach the cluster barrier before the TMEM columns are freed, so neither leaves while
// the other may still read its shared memory or signal its barriers.
#pragma once

#include <atomic>

#include "gemm_prefill.cuh"

namespace b200
{

constexpr int PP_TOKENS = 256;    // tokens per UMMA of the pair (UMMA N)
constexpr int PP_HALF = 128;      // tokens each CTA stages per UMMA
constexpr int PP_XH_BYTES = PP_HALF * PF_BK * 2;    // 16 KB
// The converted weights and the activations have rings of their own: the activation copies have the
// longer latency (L2 and the copy itself) and get the deeper ring.  224 KB per SM in all three shapes.
__host__ __device__ constexpr int pp_a_stages(int fh, int th) { return fh * th == 2 ? 4 : 3; }
__host__ __device__ constexpr int pp_x_stages(int fh, int th) { return fh * th == 1 ? 3 : (fh == 2 ? 6 : 5); }
__host__ __device__ constexpr int pp_ring_bytes(int fh, int th)
{
    return pp_a_stages(fh, th) * pf_a_bytes(fh) + pp_x_stages(fh, th) * th * PP_XH_BYTES;
}
__host__ __device__ constexpr int pp_smem_bytes(int fh, int th) { return PF_HEADER_BYTES + pp_ring_bytes(fh, th) + 1024; }

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
// shared::cluster address of the object at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(p)), "r"(rank));
    return remote;
}
// Arrive on a barrier of another CTA of the cluster.  The default semantics (release at CTA scope)
// are what the data path needs: the shared-memory stores this orders were already made visible to
// the async proxy by their writers before they arrived on the local barrier, and a release at
// cluster scope measured 600 ns per arrive.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
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
template <int WT, bool SCALED, int FH, int TH, int DQW>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(32 * (DQW + 2), FH * TH > 1 ? 1 : 2)
    gemm_wq_prefill_pair_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ PrefillYMaps tmY, const PrefillParams p)
{
    extern __shared__ unsigned char pf_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~(uintptr_t)1023);
    static_assert(FH * TH <= 2, "512 TMEM columns");
    static_assert(DQW == 8 || DQW == 16, "dequantise warps: two or four per TMEM lane quarter");
    constexpr int NA = pp_a_stages(FH, TH), NX = pp_x_stages(FH, TH);
    constexpr int A_BYTES = pf_a_bytes(FH);
    constexpr int X_BYTES = TH * PP_XH_BYTES;
    static_assert(FH * TH * PP_TOKENS * PF_BM * 2 <= pp_ring_bytes(FH, TH), "the epilogue tiles reuse the ring memory");
    constexpr int TMEM_COLS = PP_TOKENS * FH * TH;
    // One barrier pair per k block in flight (slot kb % 8), whatever the depth of the two stage rings:
    // every tcgen05 / mbarrier instruction of the leader's issue loop costs 50-100 cycles of a single
    // warp's time, so the loop waits on ONE barrier and commits to ONE per k block.
    //   full[kb % 8]: my activation bytes (TMA) + my dequantise warps (+ on the leader: rank 1's forward)
    //   done[kb % 8]: the UMMAs of k block kb are complete (multicast commit to both CTAs)
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);      // [8]
    uint64_t* done = full + 8;                               // [8]
    uint64_t* acc_full = done + 8;                           // [1]
    constexpr unsigned int RING = 8;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    unsigned char* stages = smem + PF_HEADER_BYTES;    // weight ring, then activation ring
    unsigned char* xring = stages + NA * A_BYTES;
    static_assert(NA <= 8 && NX <= 8, "barrier arrays hold eight stages");

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const unsigned int m0 = (blockIdx.x >> 1) * (PP_TOKENS * TH);     // first token of the pair's tile
    // which linear of the launch this feature tile belongs to
    unsigned int si = 0;
    if (p.n_seg > 1 && blockIdx.y >= p.seg[1].tile0) { si = 1; }
    if (p.n_seg > 2 && blockIdx.y >= p.seg[2].tile0) { si = 2; }
    const PrefillSeg& g = p.seg[si];
    const unsigned int n0 = (blockIdx.y - g.tile0) * (2 * PF_BM * FH);    // first feature of the pair's tile
    const unsigned int n_kblocks = p.K / PF_BK;
    const unsigned int tile_tokens = min((unsigned int)(PP_TOKENS * TH), p.M - m0);
    // UMMA N of each 256-token part (0: no live token); each CTA supplies live/2 token rows of it
    unsigned int live[TH];
#pragma unroll
    for (int th = 0; th < TH; th++)
    {
        const unsigned int t = tile_tokens > (unsigned int)(th * PP_TOKENS) ? min((unsigned int)PP_TOKENS, tile_tokens - th * PP_TOKENS) : 0u;
        live[th] = (t + 15u) & ~15u;
    }

    if (threadIdx.x == 0)
    {
        for (unsigned int s = 0; s < RING; s++)
        {
            mbar_init(full + s, 1 + DQW + (rank == 0 ? 1 : 0));
            mbar_init(done + s, 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DQW + 1) { tmem_alloc_pair(tmem_base_slot, TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // both CTAs' barriers exist before any remote arrive, copy or commit
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == DQW)
    {
        // =========================== TMA lane: my halves of the activations ===========================
        if (lane == 0)
        {
            bool ok = true;
            unsigned int issued = 0;
            for (unsigned int kb = 0; kb < n_kblocks; kb++)
            {
                const unsigned int s = kb % NX;
                if (kb >= NX && (*abort_flag != 0 || !mbar_wait_bounded(done + ((kb - NX) % RING), ((kb - NX) / RING) & 1u)))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                    break;
                }
                mbar_expect_tx(full + (kb % RING), X_BYTES);
#pragma unroll
                for (int th = 0; th < TH; th++)
                {
                    // a part without live tokens is still copied (zero fill) so that the byte count is fixed
                    tma_load_2d(xring + s * X_BYTES + th * PP_XH_BYTES, &tmX, (int)(kb * PF_BK),
                        (int)(m0 + th * PP_TOKENS + rank * (live[th] / 2)), full + (kb % RING));
                }
                mbar_arrive(full + (kb % RING));
                issued = kb + 1;
            }
            if (!ok)
            {
                // wait (bounded) for my copies in flight before the CTA may leave
                const unsigned int first = issued > NX ? issued - NX : 0;
                // The barrier also counts the dequantise warps, which may have given up too, so it may
                // never complete: the copies land within microseconds, 100 us per barrier is ample.
                for (unsigned int kb = first; kb < issued; kb++)
                {
                    const unsigned long long t0 = global_timer_ns();
                    while (!mbar_try_wait(full + (kb % RING), (kb / RING) & 1u) && global_timer_ns() - t0 < 100000ull) {}
                }
            }
        }
    }
    else if (warp == DQW + 1)
    {
        if (lane == 0 && rank != 0)
        {
            // =========================== rank 1: forward "stage full" to the leader ===========================
            const uint32_t peer_bar0 = map_to_cta(full, 0);
            for (unsigned int kb = 0; kb < n_kblocks; kb++)
            {
                const bool w = *abort_flag == 0 && mbar_wait_bounded(full + (kb % RING), (kb / RING) & 1u);
                if (!w)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    *abort_flag = 1;
                    break;
                }
                mbar_arrive_cluster(peer_bar0 + (kb & 7u) * 8);
            }
        }
        else if (rank == 0)
        {
            // =========================== leader: UMMA warp ===========================
            // The whole warp runs the loop (waits and descriptor arithmetic stay warp-uniform); one
            // elected lane issues the UMMAs and the commits.
            bool ok = true;
            uint32_t idesc[TH];
#pragma unroll
            for (int th = 0; th < TH; th++) { idesc[th] = umma_idesc_bf16(2 * PF_BM, live[th]); }
            for (unsigned int kb = 0; kb < n_kblocks && ok; kb++)
            {
                const unsigned int sx = kb % NX, sa = kb % NA;
                const bool w = *abort_flag == 0 && mbar_wait_bounded(full + (kb % RING), (kb / RING) & 1u);
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
                const uint32_t a_addr = smem_u32(stages + sa * A_BYTES);
                const uint32_t b_addr = smem_u32(xring + sx * X_BYTES);
                if (elect_one())
                {
#pragma unroll
                for (int th = 0; th < TH; th++)
                {
                    if (live[th] == 0) { continue; }
#pragma unroll
                    for (int k = 0; k < PF_BK / 16; k++)
                    {
#pragma unroll
                        for (int fh = 0; fh < FH; fh++)
                        {
                            umma_bf16_pair(tmem_base + (fh * TH + th) * PP_TOKENS,
                                umma_desc_kmajor_sw128(a_addr + fh * (PF_BM * PF_BK * 2) + k * 32),
                                umma_desc_kmajor_sw128(b_addr + th * PP_XH_BYTES + k * 32), idesc[th], (kb | (unsigned int)k) != 0 ? 1u : 0u);
                        }
                    }
                }
                umma_commit_pair(done + (kb % RING));
                }
                __syncwarp();
            }
            __syncwarp();
            // also on the abort path: the barrier completes once the UMMAs in flight have stopped
            // reading both CTAs' shared memory; the epilogue warps then see the abort flag or the status
            if (elect_one()) { umma_commit_pair(acc_full); }
        }
    }
    else
    {
        // =========================== dequantise, then epilogue (warps 0..DQW-1) ===========================
        const unsigned int tid = threadIdx.x;
        constexpr int NP = 512 * FH / (32 * DQW);    // (row, 16-element group) pieces per thread per k block
        unsigned int prow[NP], pq[NP], pfeat[NP];
#pragma unroll
        for (int i = 0; i < NP; i++)
        {
            const unsigned int piece = tid + (32u * DQW) * i;
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
                if (pfeat[i] < g.N)
                {
                    const size_t e = (size_t)pfeat[i] * g.ldw + (size_t)kb * PF_BK + pq[i] * 16;
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
            if (kb + 2 < n_kblocks) { load_raw(kb + 2, slot); }
        };
        // The conversion of block kb+1 is issued between the stores of block kb and their proxy fence,
        // so the fence finds the stores already performed.
        uint32_t out[NP][8];
        if (n_kblocks > 0) { convert_and_refill(0, 0, out); }
        for (unsigned int kb = 0; kb < n_kblocks; kb++)
        {
            const unsigned int s = kb % NA;
            if (ok && kb >= NA && (*abort_flag != 0 || !mbar_wait_bounded(done + ((kb - NA) % RING), ((kb - NA) / RING) & 1u)))
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
                const uint32_t a_addr = smem_u32(stages + s * A_BYTES);
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
                fence_proxy_async();    // make the generic-proxy stores visible to the tensor cores' reads
                __syncwarp();
                if (lane == 0) { mbar_arrive(full + (kb % RING)); }
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
        const unsigned int quarter = warp & 3u;
        // the DQW/4 warps of a TMEM lane quarter split each 256-token part's columns
        constexpr unsigned int CPW = PP_TOKENS / (DQW / 4);
        const unsigned int cbeg = (warp >> 2) * CPW;
        if (ok && n_kblocks > 0 && g.y_tma != 0)
        {
            // BF16 tiles [256 tokens][128 features] in the idle stage memory, then one TMA store each;
            // the store clips rows past M and features past N
#pragma unroll
            for (int fh = 0; fh < FH; fh++)
            {
#pragma unroll
                for (int th = 0; th < TH; th++)
                {
                    const unsigned int part_tokens = min((unsigned int)PP_TOKENS, tile_tokens - min(tile_tokens, (unsigned int)(th * PP_TOKENS)));
                    const uint32_t ytile = smem_u32(stages) + (fh * TH + th) * (PP_TOKENS * PF_BM * 2) + (quarter * 32 + lane) * 2;
                    for (unsigned int c0 = cbeg; c0 < cbeg + CPW && c0 < part_tokens; c0 += 32)
                    {
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + (fh * TH + th) * PP_TOKENS + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j++)
                        {
                            sts16(ytile + (c0 + j) * (PF_BM * 2),
                                __bfloat16_as_ushort(__float2bfloat16_rn(g.alpha * (__uint_as_float(r[j]) * g.post_scale))));
                        }
                    }
                }
            }
            fence_proxy_async();
            bar_sync_named(1, 32 * DQW);
            if (tid == 0)
            {
#pragma unroll
                for (int fh = 0; fh < FH; fh++)
                {
#pragma unroll
                    for (int th = 0; th < TH; th++)
                    {
                        if (tile_tokens > (unsigned int)(th * PP_TOKENS))
                        {
                            tma_store_2d(&tmY.m[si], stages + (fh * TH + th) * (PP_TOKENS * PF_BM * 2), (int)(n0 + (fh * 2 + rank) * PF_BM),
                                (int)(m0 + th * PP_TOKENS));
                        }
                    }
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
#pragma unroll
                for (int th = 0; th < TH; th++)
                {
                    const unsigned int part_tokens = min((unsigned int)PP_TOKENS, tile_tokens - min(tile_tokens, (unsigned int)(th * PP_TOKENS)));
                    for (unsigned int c0 = cbeg; c0 < cbeg + CPW && c0 < part_tokens; c0 += 32)
                    {
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + (fh * TH + th) * PP_TOKENS + c0, r);
                        tmem_ld_wait();
                        if (n < g.N)
                        {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                            {
                                const unsigned int m = m0 + th * PP_TOKENS + c0 + j;
                                if (c0 + j < part_tokens)
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
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // neither CTA frees TMEM or leaves while the other may still use the pair
    if (warp == DQW + 1) { tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

template <int WT, bool SCALED, int FH, int TH, int DQW>
static int launch_prefill_pair(const CUtensorMap& tmX, const PrefillYMaps& tmY, const PrefillParams& pp, unsigned int feature_tiles, int device,
    cudaStream_t stream)
{
    auto kernel = gemm_wq_prefill_pair_kernel<WT, SCALED, FH, TH, DQW>;
    static std::atomic<bool> attr_set[64];    // zero-initialised; setting the attribute twice is harmless
    if (!attr_set[device].load(std::memory_order_acquire))
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pp_smem_bytes(FH, TH)) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16");
            return 1;
        }
        attr_set[device].store(true, std::memory_order_release);
    }
    const dim3 grid(2 * ((pp.M + PP_TOKENS * TH - 1) / (PP_TOKENS * TH)), feature_tiles);
    count_launch();
    kernel<<<grid, 32 * (DQW + 2), pp_smem_bytes(FH, TH), stream>>>(tmX, tmY, pp);
    return report_launch("gemm_wq_bf16");
}

}    // namespace b200
