// FP4 (E2M1, one E4M3 scale per 16 weights) linear for 1 .. 32 tokens with the weights AND their block scales fed to
// the tensor cores as they lie in memory: tcgen05.mma kind::mxf4nvf4 with block-16 scales multiplies
// (e2m1 * ue4m3) by (e2m1 * ue4m3) exactly and accumulates in FP32 - the reference's FP4 format IS that operand
// format.  No thread touches a weight; four warps only carry each stage's 2 KB of scale bytes from shared memory
// into the tensor-memory columns the UMMA reads them from.
//
// The BF16 activations are split by a small kernel into SEVEN E2M1 rows per token, each with its own power-of-two
// scale per 16-element block: piece j of a block is the remainder truncated (the last one: rounded) to E2M1 at scale
// 2^(p - 2 j), p chosen from the block's largest magnitude.  Every piece takes two more significant bits of every
// element, whatever the element's own exponent, so the sum of the seven rows equals the activation to within 2^-16 of
// the block's largest magnitude (and exactly for elements within 2^6 of it).  The seven rows are seven columns of the UMMA's N dimension;
// the epilogue adds them and undoes the per-token power of two that keeps all scales inside E4M3's normal range.
// A token row that holds an infinity or a NaN gives NaN outputs.
//
// Work is dealt out as in the FP8 kernel (stream-K ranges of (feature tile, 256-k block) units over a persistent
// grid, partial tiles of cut tiles added in k order by the last CTA to arrive); every wait is bounded.
#pragma once

#include "gemm_native.cuh"

namespace b200
{

constexpr int NF_PIECES = 7;
constexpr int NF_BK = 256;                  // k per block: one 128-byte swizzle row of packed nibbles
constexpr int NF_THREADS = 32 * 10;         // TMA warp, MMA warp, four scale warps, four epilogue warps
constexpr int NF_W_BYTES = NK_BM * 128;     // one weight stage
constexpr int NF_SFA_BYTES = NK_BM * 16;    // its block scales: 16 per row
constexpr int NF_MAX_TOKENS = 32;           // 7 * 32 = 224 rows of B
constexpr int NF_NARROW_TOKENS = 13;        // up to here (7 * 13 = 91 of 96 rows) two CTAs share an SM
// Two shapes.  Narrow (N <= 96): two CTAs per SM, 256 TMEM columns each: 96 for the accumulators, then 16 scale columns
// of A and 16 of B per stage, at most 5 stages.  Wide (N = 224, 14 .. 32 tokens): one CTA per SM with all 512 columns:
// 224 + 4 stages x (16 + 32).
__host__ __device__ constexpr bool nf_wide(int bnp) { return bnp > 96; }
__host__ __device__ constexpr int nf_acc_cols(int bnp) { return nf_wide(bnp) ? 224 : 96; }
__host__ __device__ constexpr int nf_sfb_words(int bnp) { return nf_wide(bnp) ? 8 : 4; }    // 32-row groups of B whose scales a 64-k step reads
__host__ __device__ constexpr int nf_max_stages(int bnp) { return nf_wide(bnp) ? 4 : 5; }
__host__ __device__ constexpr int nf_stage_bytes(int bnp) { return (NF_W_BYTES + bnp * 128 + NF_SFA_BYTES + bnp * 16 + 1023) & ~1023; }
__host__ __device__ constexpr int nf_stages(int bnp)
{
    return ((nf_wide(bnp) ? 227 : 113) * 1024 - 2048) / nf_stage_bytes(bnp) > nf_max_stages(bnp)
        ? nf_max_stages(bnp)
        : ((nf_wide(bnp) ? 227 : 113) * 1024 - 2048) / nf_stage_bytes(bnp);
}
__host__ __device__ constexpr int nf_smem_bytes(int bnp) { return NK_HEADER_BYTES + nf_stages(bnp) * nf_stage_bytes(bnp) + 1024; }

struct NativeFp4Maps
{
    CUtensorMap w[PF_MAX_GROUP];    // packed nibbles [N][K / 2]
    CUtensorMap s[PF_MAX_GROUP];    // block scales [N][K / 16]
    CUtensorMap x;                  // the pieces [6 M][K / 2]
    CUtensorMap xs;                 // their scales [6 M][K / 16]
};

// D[tmem] (+)= (A * SFA)[smem, tmem] * (B * SFB)[smem, tmem]; E2M1 values, UE4M3 scales per 16 k, FP32 accumulate, 64 k.
__device__ __forceinline__ void umma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
    uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// Instruction descriptor of the block-scaled kinds: A = B = E2M1 (format 1 at bits 7-9 and 10-12), both K-major,
// N >> 3 at bits 17-22, scale format UE4M3 (bit 23 = 0), M >> 4 at bits 24-28, scale-factor ids 0, 64 k (bit 31 = 0).
__device__ __forceinline__ uint32_t umma_idesc_nvf4(uint32_t m, uint32_t n) { return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24); }

// ---- the activations as seven E2M1 rows per token ------------------------------------------------------------
constexpr int NF_SPLIT_CHUNK = 256 * 4;    // k per block of the split kernel: four per thread, four threads per 16-k block
// Grid (k chunks, tokens).  pieces [7 M][K / 2] bytes (low nibble = even k), scales [7 M][K / 16] UE4M3 bytes, row
// 7 t + j = piece j of token t; inv_scale[t] undoes the token's power of two.
static __global__ void __launch_bounds__(256) split_activations_fp4_kernel(const uint16_t* __restrict__ X, unsigned int ldx, unsigned int K,
    uint8_t* __restrict__ pieces, uint8_t* __restrict__ scales, float* __restrict__ inv_scale, unsigned int pad_rows)
{
    __shared__ unsigned int red[16];
    pdl_launch_dependents();
    pdl_wait();
    const unsigned int t = blockIdx.y, tid = threadIdx.x;
    if (t == 0 && pad_rows != 0)
    {
        // the rows between 6 M and the UMMA's N are zero: the tensor maps then cover whole boxes
        const unsigned int k0 = blockIdx.x * NF_SPLIT_CHUNK + tid * 4;
        if (k0 < K)
        {
            for (unsigned int r = NF_PIECES * gridDim.y; r < NF_PIECES * gridDim.y + pad_rows; r++)
            {
                *reinterpret_cast<uint16_t*>(pieces + (size_t)r * (K / 2) + k0 / 2) = 0;
                if ((tid & 3u) == 0) { scales[(size_t)r * (K / 16) + k0 / 16] = 0; }
            }
        }
    }
    const uint16_t* x = X + (size_t)t * ldx;
    unsigned int amax, bad;
    row_absmax_bits(x, K, red, amax, bad);
    // 2^s lifts the row's largest magnitude to exponent 10: its block's first scale is then 2^8, the largest power
    // of two E4M3 holds; a block's first scale is at least 2^6, so that its seventh is never below 2^-6, E4M3's
    // smallest normal (blocks far below the row's largest magnitude are held to 2^-17 of that magnitude instead)
    int s = 0;
    if (amax != 0 && bad == 0)
    {
        s = 137 - (int)(amax >> 7);
        s = s > 126 ? 126 : s;
    }
    const float scale = __uint_as_float((unsigned int)(127 + s) << 23);
    if (blockIdx.x == 0 && tid == 0) { inv_scale[t] = bad ? __uint_as_float(0x7FC00000u) : __uint_as_float((unsigned int)(127 - s) << 23); }
    const unsigned int k0 = blockIdx.x * NF_SPLIT_CHUNK + tid * 4;    // K is a multiple of 256: whole warps stay or leave together
    if (k0 >= K) { return; }
    const uint2 va = *reinterpret_cast<const uint2*>(x + k0);
    const unsigned int w[2] = { va.x, va.y };
    float r[4];
    unsigned int sign = 0, top = 0;
#pragma unroll
    for (int q = 0; q < 4; q++)
    {
        const unsigned int bits = (q & 1) ? (w[q >> 1] >> 16) : (w[q >> 1] & 0xFFFFu);
        sign |= ((bits >> 15) & 1u) << q;
        r[q] = bad ? 0.f : __uint_as_float((bits & 0x7FFFu) << 16) * scale;
        top = max(top, __float_as_uint(r[q]));
    }
    // the four threads of a 16-k block agree on its largest magnitude
    top = max(top, __shfl_xor_sync(0xFFFFFFFFu, top, 1));
    top = max(top, __shfl_xor_sync(0xFFFFFFFFu, top, 2));
    // the first scale: 2^(exponent of the block's largest magnitude - 2), so that magnitude lands in [4, 8)
    int p = (int)(top >> 23) - 127 - 2;
    p = p < 6 ? 6 : (p > 8 ? 8 : p);
    const unsigned int kh = K / 2, kb16 = K / 16;
#pragma unroll
    for (int j = 0; j < NF_PIECES; j++)
    {
        const int pj = p - 2 * j;
        const float sj = __uint_as_float((unsigned int)(127 + pj) << 23), inv_sj = __uint_as_float((unsigned int)(127 - pj) << 23);
        unsigned int out = 0;
#pragma unroll
        for (int q = 0; q < 4; q++)
        {
            // the remainder truncated to E2M1: 0, 0.5, then one mantissa bit on exponents 0, 1, 2
            const float qf = r[q] * inv_sj;
            const unsigned int qb = __float_as_uint(qf);
            const unsigned int ex = qb >> 23;
            unsigned int code, vb2;
            if (j == NF_PIECES - 1) { code = float_to_fp4(qf); vb2 = 0u; }    // the last piece: to the nearest value
            else if (ex < 126u) { code = 0u; vb2 = 0u; }
            else if (ex == 126u) { code = 1u; vb2 = 0x3F000000u; }
            else if (ex > 129u) { code = 7u; vb2 = 0x40C00000u; }
            else { code = ((ex - 126u) << 1) | ((qb >> 22) & 1u); vb2 = qb & 0xFFC00000u; }
            r[q] -= __uint_as_float(vb2) * sj;
            out |= (code | (code != 0u ? ((sign >> q) & 1u) << 3 : 0u)) << (4 * q);
        }
        const size_t row = (size_t)(NF_PIECES * t + j);
        *reinterpret_cast<uint16_t*>(pieces + row * kh + k0 / 2) = (uint16_t)out;
        if ((tid & 3u) == 0) { scales[row * kb16 + k0 / 16] = (uint8_t)((unsigned int)(pj + 7) << 3); }
    }
}

// ---- the linear -------------------------------------------------------------------------------------------
// BNP = UMMA N = 7 * tokens rounded up to a multiple of 16.
template <int BNP>
// (the narrow shape's bounds name 32 threads more than are launched, see gemm_wq_native_kernel)
__global__ void __launch_bounds__(nf_wide(BNP) ? NF_THREADS : NF_THREADS + 32, nf_wide(BNP) ? 1 : 2) gemm_wq_native_fp4_kernel(const __grid_constant__ NativeFp4Maps tm, const NativeParams p)
{
    constexpr int STAGES = nf_stages(BNP);
    constexpr int STAGE_BYTES = nf_stage_bytes(BNP);
    constexpr int B_BYTES = BNP * 128, SFB_BYTES = BNP * 16;
    constexpr int TMEM_COLS = nf_wide(BNP) ? 512 : 256;
    constexpr int ACC_COLS = nf_acc_cols(BNP), MAX_STAGES = nf_max_stages(BNP), SFB_WORDS = nf_sfb_words(BNP);
    constexpr int TOK = BNP / NF_PIECES;
    constexpr int ACCS = ACC_COLS / BNP >= 4 ? 4 : (ACC_COLS / BNP >= 2 ? 2 : 1);    // independent accumulators, see nk_accs
    constexpr int SFA_COL = ACC_COLS, SFB_COL = ACC_COLS + 16 * MAX_STAGES, SFB_STAGE_COLS = 4 * SFB_WORDS;
    static_assert(STAGES >= 2 && STAGES <= MAX_STAGES && BNP <= ACC_COLS && BNP % 16 == 0, "shape");
    static_assert(SFB_COL + SFB_STAGE_COLS * MAX_STAGES <= TMEM_COLS && 32 * SFB_WORDS >= BNP, "tensor memory");
    extern __shared__ unsigned char nf_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(nf_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + 8;
    uint64_t* sf_full = empty + 8;
    uint64_t* acc_full = sf_full + 8;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    volatile unsigned int* last_flag = abort_flag + 1;
    volatile unsigned int* go_flag = abort_flag + 2;
    unsigned char* stages = smem + NK_HEADER_BYTES;

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned long long U = (unsigned long long)p.tiles * p.nkb;
    const unsigned int G = gridDim.x;
    const unsigned int u0 = (unsigned int)((U * blockIdx.x) / G), u1 = (unsigned int)((U * (blockIdx.x + 1ull)) / G);
    const unsigned int n_units = u1 - u0;

    auto member_of = [&](unsigned int tile) -> unsigned int {
        unsigned int si = 0;
        if (p.n_seg > 1 && tile >= p.seg[1].tile0) { si = 1; }
        if (p.n_seg > 2 && tile >= p.seg[2].tile0) { si = 2; }
        return si;
    };
    const uint64_t pol = l2_policy_evict_first();
    auto issue_weights = [&](unsigned int i) {
        const unsigned int u = u0 + i, tile = u / p.nkb, kb = u % p.nkb, s = i % STAGES;
        const unsigned int si = member_of(tile);
        const int row0 = (int)((tile - p.seg[si].tile0) * NK_BM);
        unsigned char* st = stages + s * STAGE_BYTES;
        mbar_expect_tx(full + s, NF_W_BYTES + NF_SFA_BYTES);
        tma_load_2d_hint(st, &tm.w[si], (int)(kb * 128), row0, full + s, pol);
        tma_load_2d_hint(st + NF_W_BYTES + B_BYTES, &tm.s[si], (int)(kb * 16), row0, full + s, pol);
    };
    const unsigned int pre = n_units < (unsigned int)STAGES ? n_units : (unsigned int)STAGES;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; s++)
        {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
            mbar_init(sf_full + s, 4);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the weights and their scales depend on nothing: the first ring of stages is asked for before the CTA has met
        for (unsigned int i = 0; i < pre; i++) { issue_weights(i); }
    }
    if (warp == 1) { tmem_alloc(tmem_base_slot, TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    pdl_launch_dependents();

    if (warp == 0)
    {
        // =========================== TMA lane ===========================
        if (lane == 0)
        {
            auto issue_acts = [&](unsigned int i) {
                const unsigned int u = u0 + i, kb = u % p.nkb, s = i % STAGES;
                unsigned char* st = stages + s * STAGE_BYTES;
                mbar_expect_tx(full + s, B_BYTES + SFB_BYTES);
                tma_load_2d(st + NF_W_BYTES, &tm.x, (int)(kb * 128), 0, full + s);
                tma_load_2d(st + NF_W_BYTES + B_BYTES + NF_SFA_BYTES, &tm.xs, (int)(kb * 16), 0, full + s);
                mbar_arrive(full + s);
            };
            pdl_wait();
            for (unsigned int i = 0; i < pre; i++) { issue_acts(i); }
            bool ok = true;
            unsigned int issued = pre;
            for (unsigned int i = pre; i < n_units; i++)
            {
                const unsigned int s = i % STAGES;
                if (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((i / STAGES) - 1) & 1u))
                {
                    ok = false;
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                    *abort_flag = 1;
                    break;
                }
                issue_weights(i);
                issue_acts(i);
                issued = i + 1;
            }
            const unsigned int first = issued > (unsigned int)STAGES ? issued - STAGES : 0;
            for (unsigned int i = first; i < issued; i++)
            {
                if (!mbar_wait_bounded(full + (i % STAGES), (i / STAGES) & 1u) && ok)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    *abort_flag = 1;
                    ok = false;
                }
            }
        }
    }
    else if (warp == 1)
    {
        // =========================== MMA warp ===========================
        const uint32_t idesc = umma_idesc_nvf4(NK_BM, BNP);
        unsigned int runs_done = 0;
        bool ok = true;
        for (unsigned int i = 0; i < n_units && ok; i++)
        {
            const unsigned int kb = (u0 + i) % p.nkb, s = i % STAGES;
            const bool first = kb == 0 || i == 0;
            const bool last = kb + 1 == p.nkb || i + 1 == n_units;
            if (first && runs_done > 0 && (*abort_flag != 0 || !mbar_wait_bounded(acc_empty, (runs_done - 1) & 1u))) { ok = false; }
            if (ok && (*abort_flag != 0 || !mbar_wait_bounded(full + s, (i / STAGES) & 1u) || !mbar_wait_bounded(sf_full + s, (i / STAGES) & 1u)))
            {
                ok = false;
            }
            if (!ok)
            {
                if (lane == 0)
                {
                    atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                    *abort_flag = 1;
                }
                break;
            }
            tc_fence_after();
            if (elect_one())
            {
                const uint32_t a_addr = smem_u32(stages + s * STAGE_BYTES), b_addr = a_addr + NF_W_BYTES;
#pragma unroll
                for (int m = 0; m < NF_BK / 64; m++)
                {
                    // 64 k = 32 bytes further along the swizzle row; its scales are the next four columns
                    umma_nvf4(tmem_base + (m % ACCS) * BNP, umma_desc_kmajor_sw128(a_addr + m * 32), umma_desc_kmajor_sw128(b_addr + m * 32), idesc,
                        tmem_base + SFA_COL + s * 16 + m * 4, tmem_base + SFB_COL + s * SFB_STAGE_COLS + m * SFB_WORDS, (first && m < ACCS) ? 0u : 1u);
                }
                umma_commit(empty + s);
                if (last) { umma_commit(acc_full); }
            }
            __syncwarp();
            if (last) { runs_done++; }
        }
    }
    else if (warp < 6)
    {
        // =========================== scale warps (2..5) ===========================
        // The UMMA reads the scale of operand row r and 16-k block j of a 64-k step from tensor-memory lane r % 32
        // (every lane quarter holds a copy), byte 4 (r / 32) + j of the step's four columns.  Each of the four warps
        // fills its own lane quarter: lane l writes, for each of the stage's four steps m, the words m of the
        // sixteen-byte scale rows l, 32 + l, 64 + l, 96 + l.
        const unsigned int quarter = warp & 3u;
        const uint32_t lane_field = (quarter * 32u) << 16;
        for (unsigned int i = 0; i < n_units; i++)
        {
            const unsigned int s = i % STAGES;
            if (*abort_flag != 0 || !mbar_wait_bounded(full + s, (i / STAGES) & 1u))
            {
                atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                *abort_flag = 1;
                break;
            }
            const uint32_t sfa = smem_u32(stages + s * STAGE_BYTES + NF_W_BYTES + B_BYTES), sfb = sfa + NF_SFA_BYTES;
            uint32_t ra[16], rb[SFB_STAGE_COLS];
#pragma unroll
            for (int q = 0; q < 4; q++)
            {
                const uint4 a = sk_lds128(sfa + (q * 32 + lane) * 16);
                ra[q] = a.x;
                ra[4 + q] = a.y;
                ra[8 + q] = a.z;
                ra[12 + q] = a.w;
            }
#pragma unroll
            for (int q = 0; q < SFB_WORDS; q++)
            {
                uint4 b = make_uint4(0, 0, 0, 0);
                if (q * 32 + (int)lane < BNP) { b = sk_lds128(sfb + (q * 32 + lane) * 16); }
                rb[q] = b.x;
                rb[SFB_WORDS + q] = b.y;
                rb[2 * SFB_WORDS + q] = b.z;
                rb[3 * SFB_WORDS + q] = b.w;
            }
            tmem_st_32x16(tmem_base + lane_field + SFA_COL + s * 16, ra);
#pragma unroll
            for (int c = 0; c < SFB_STAGE_COLS; c += 16) { tmem_st_32x16(tmem_base + lane_field + SFB_COL + s * SFB_STAGE_COLS + c, rb + c); }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(sf_full + s); }
        }
    }
    else
    {
        // =========================== epilogue (warps 6..9) ===========================
        const unsigned int quarter = warp & 3u;
        const unsigned int f = quarter * 32 + lane;
        const unsigned int etid = threadIdx.x - 192;
        pdl_wait();
        unsigned int run = 0;
        for (unsigned int u = u0; u < u1; run++)
        {
            const unsigned int tile = u / p.nkb;
            const unsigned int tile_begin = tile * p.nkb, tile_end = tile_begin + p.nkb;
            const unsigned int e = u1 < tile_end ? u1 : tile_end;
            if (*abort_flag != 0 || !mbar_wait_bounded(acc_full, run & 1u))
            {
                atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
                *abort_flag = 1;
            }
            bar_sync_named(1, 128);
            if (etid == 0) { *go_flag = *abort_flag == 0 ? 1u : 0u; }
            bar_sync_named(1, 128);
            if (*go_flag == 0) { break; }
            tc_fence_after();
            float v[TOK];
            {
                // at most 112 columns (16 tokens) in registers at a time
                constexpr int CH = BNP > 112 ? 112 : BNP, TPC = CH / NF_PIECES;
                static_assert(BNP % CH == 0 && (BNP / CH) * TPC >= TOK, "chunks");
#pragma unroll
                for (int h = 0; h < BNP / CH; h++)
                {
                    float acc[CH];
#pragma unroll
                    for (int a = 0; a < ACCS; a++)
                    {
#pragma unroll
                        for (int c = 0; c < CH; c += 16)
                        {
                            uint32_t r[16];
                            tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + a * BNP + h * CH + c, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int q = 0; q < 16; q++) { acc[c + q] = a == 0 ? __uint_as_float(r[q]) : acc[c + q] + __uint_as_float(r[q]); }
                        }
                    }
#pragma unroll
                    for (int t = 0; t < TPC; t++)
                    {
                        if (h * TPC + t < TOK)
                        {
                            float sum = acc[NF_PIECES * t];
#pragma unroll
                            for (int j = 1; j < NF_PIECES; j++) { sum += acc[NF_PIECES * t + j]; }
                            v[h * TPC + t] = sum;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(acc_empty); }

            const unsigned int si = member_of(tile);
            const PrefillSeg& g = p.seg[si];
            const unsigned int n = (tile - g.tile0) * NK_BM + f;
            bool write_out = u == tile_begin && e == tile_end;
            if (!write_out)
            {
                const unsigned int slot = 2 * blockIdx.x + (u == tile_begin ? 1u : 0u);
                float* mine = p.partials + (size_t)slot * p.M * NK_BM;
#pragma unroll
                for (int t = 0; t < TOK; t++)
                {
                    if ((unsigned int)t < p.M) { mine[t * NK_BM + f] = v[t]; }
                }
                __threadfence();
                bar_sync_named(1, 128);
                const unsigned int c_first = (unsigned int)(((tile_begin + 1ull) * G - 1ull) / U);
                const unsigned int c_last = (unsigned int)(((unsigned long long)tile_end * G - 1ull) / U);
                if (etid == 0)
                {
                    const unsigned int old = atomicAdd(p.counters + c_first, 1u);
                    const unsigned int is_last = old == c_last - c_first ? 1u : 0u;
                    if (is_last) { p.counters[c_first] = 0; }
                    *last_flag = is_last;
                }
                bar_sync_named(1, 128);
                write_out = *last_flag != 0;
                if (write_out)
                {
                    __threadfence();
                    nk_sum_parts<TOK>(p.partials, p.M, c_first, c_last, f, v);
                }
                bar_sync_named(1, 128);
            }
            if (write_out && n < g.N)
            {
#pragma unroll
                for (int t = 0; t < TOK; t++)
                {
                    if ((unsigned int)t >= p.M) { break; }
                    const long long yi = (long long)t * g.ldy_m + (long long)n * g.ldy_n;
                    float o = g.alpha * (v[t] * __ldg(p.inv_scale + t));
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
            u = e;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) { tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---- host side -----------------------------------------------------------------------------------------
inline bool native_fp4_supported(const void* blk, unsigned int N, unsigned int M, unsigned int K, unsigned int ldw, unsigned int ldx)
{
    return blk != nullptr && sk_al16(blk) && M >= 1 && M <= (unsigned int)NF_MAX_TOKENS && N > 0 && K > 0 && (K % NF_BK) == 0 && (ldx % 8) == 0
        && (ldw % 256) == 0;
}

template <int BNP>
static int launch_native_fp4_bn(const void* X, unsigned int ldx, NativeParams& np, unsigned char* scratch, size_t scratch_bytes, unsigned int n_counters,
    int device, int sm_count, cudaStream_t stream, bool pdl)
{
    const unsigned long long U = (unsigned long long)np.tiles * np.nkb;
    if (U == 0 || U > 0x7FFFFFFFull) { return -2; }
    const unsigned long long slots = (nf_wide(BNP) ? 1ull : 2ull) * (unsigned)sm_count;
    const unsigned int grid = nk_grid(np.tiles, np.nkb, slots);
    // BNP rows, those past 7 M zeroed by the split kernel: a TMA box with rows out of bounds is slow (measured: 88 us
    // instead of 56 us for 128256 x 4096 at one token, where 26 of a box's 32 rows were out of bounds)
    const size_t rows = (size_t)BNP;
    const unsigned int pad_rows = (unsigned int)(rows - (size_t)NF_PIECES * np.M);
    const size_t piece_bytes = (rows * (np.K / 2) + 1023) & ~(size_t)1023;
    const size_t scale_bytes = (rows * (np.K / 16) + 1023) & ~(size_t)1023;
    const size_t part_bytes = (size_t)2 * grid * np.M * NK_BM * sizeof(float);
    if (NK_SCALE_BYTES + piece_bytes + scale_bytes + part_bytes > scratch_bytes || grid > n_counters || ((uintptr_t)scratch & 255u) != 0) { return -2; }
    float* inv_scale = reinterpret_cast<float*>(scratch);
    uint8_t* pieces = scratch + NK_SCALE_BYTES;
    uint8_t* xscales = pieces + piece_bytes;
    np.inv_scale = inv_scale;
    np.partials = reinterpret_cast<float*>(xscales + scale_bytes);

    NativeFp4Maps tm;
    memset(&tm, 0, sizeof(tm));
    bool ok = make_map_2d(&tm.x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pieces, np.K / 2, rows, np.K / 2, 128, BNP, true)
        && make_map_2d(&tm.xs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xscales, np.K / 16, rows, np.K / 16, 16, BNP, false);
    for (unsigned int j = 0; j < (unsigned)PF_MAX_GROUP && ok; j++)
    {
        const PrefillSeg& g = np.seg[j < np.n_seg ? j : 0];
        ok = make_map_2d(&tm.w[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.W, np.K / 2, g.N, g.ldw / 2, 128, NK_BM, true)
            && make_map_2d(&tm.s[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.blk, np.K / 16, g.N, g.ldw / 16, 16, NK_BM, false);
    }
    if (!ok) { return -2; }
    auto kernel = gemm_wq_native_fp4_kernel<BNP>;
    static std::atomic<bool> attr_set[64];
    if (!attr_set[device].load(std::memory_order_acquire))
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, nf_smem_bytes(BNP)) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16");
            return 1;
        }
        attr_set[device].store(true, std::memory_order_release);
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((np.K + NF_SPLIT_CHUNK - 1) / NF_SPLIT_CHUNK, np.M);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, split_activations_fp4_kernel, (const uint16_t*)X, ldx, np.K, pieces, xscales, inv_scale, pad_rows) != cudaSuccess)
    {
        report_launch("gemm_wq_bf16");
        return 1;
    }
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NF_THREADS);
    cfg.dynamicSmemBytes = nf_smem_bytes(BNP);
    cfg.numAttrs = 1;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, kernel, tm, np) != cudaSuccess)
    {
        report_launch("gemm_wq_bf16");
        return 1;
    }
    return 0;
}

// One launch (plus the split of the activations) for up to PF_MAX_GROUP FP4 linears that share X.  -2: not taken.
static int launch_native_fp4(const GemvParams* items, unsigned int count, float* scratch, size_t scratch_bytes, unsigned int* counters,
    unsigned int n_counters, int device, int sm_count, cudaStream_t stream, bool pdl)
{
    if (count == 0 || count > (unsigned)PF_MAX_GROUP || !scratch || !counters) { return -2; }
    NativeParams np;
    memset(&np, 0, sizeof(np));
    np.n_seg = count;
    np.status = items[0].status;
    np.M = items[0].M;
    np.K = items[0].K;
    np.out_f32 = items[0].out_f32;
    np.counters = counters;
    np.nkb = np.K / NF_BK;
    for (unsigned int j = 0; j < count; j++)
    {
        if (!native_fp4_supported(items[j].blk, items[j].N, items[j].M, items[j].K, items[j].ldw, items[j].ldx) || !sk_al16(items[j].W)) { return -2; }
        PrefillSeg& g = np.seg[j];
        g.W = items[j].W;
        g.blk = items[j].blk;
        g.Y = items[j].Y;
        g.N = items[j].N;
        g.ldw = items[j].ldw;
        g.ldy_m = items[j].ldy_m;
        g.ldy_n = items[j].ldy_n;
        g.alpha = items[j].alpha;
        g.beta = items[j].beta;
        g.w_scale = 1.0f;
        g.post_scale = 1.0f;
        g.tile0 = np.tiles;
        np.tiles += (items[j].N + NK_BM - 1) / NK_BM;
    }
    if (!sk_al16(items[0].X)) { return -2; }
    const void* X = items[0].X;
    const unsigned int ldx = items[0].ldx;
    unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
#define NF_LAUNCH(BNP_) launch_native_fp4_bn<BNP_>(X, ldx, np, sc, scratch_bytes, n_counters, device, sm_count, stream, pdl)
    if (np.M <= 2) { return NF_LAUNCH(16); }
    if (np.M <= 4) { return NF_LAUNCH(32); }
    if (np.M <= 6) { return NF_LAUNCH(48); }
    if (np.M <= 9) { return NF_LAUNCH(64); }
    if (np.M <= (unsigned int)NF_NARROW_TOKENS) { return NF_LAUNCH(96); }
    return NF_LAUNCH(224);
#undef NF_LAUNCH
}

}    // namespace b200
