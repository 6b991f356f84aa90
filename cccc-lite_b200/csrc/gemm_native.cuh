// FP8-weight linear for 1 .. 32 tokens with the weights fed to the tensor cores AS THEY LIE IN MEMORY.
//
// The decode kernel turns every weight into BF16 in registers and multiplies it there; at about four issue
// slots per weight that arithmetic, not HBM, is what bounds it from a few tokens on (and FP4 at every batch).  tcgen05.mma kind::f8f6f4 takes E4M3 and E5M2
// operands directly and multiplies them exactly with FP32 accumulation, so here a TMA lane streams the weight
// bytes into shared memory and the UMMA reads them from there: no thread ever touches a weight.
//
// The activations are BF16 (8 significant bits), which that UMMA kind does not take.  A small kernel first
// writes each token row as the exact sum of three E5M2 rows (3 significant bits each):
//     x * 2^s = p0 + p1 + p2,   p0 = x * 2^s truncated to 3 bits, p1 = the remainder truncated, p2 = the rest,
// with one power of two 2^s per token that puts the row's largest magnitude at the top of E5M2's range (what
// falls below E5M2's smallest subnormal, 2^-31 of the row's maximum, is dropped).  The three rows are three
// columns of the UMMA's N dimension; the epilogue adds them and multiplies by 2^-s.  Every product the tensor
// core forms is therefore the exact product of a weight and a piece of the BF16 activation.
//
// With PIECES = 1 the same kernel is the W8A8 linear: the activations are E4M3 themselves, one row per token
// (gemm_w8a8.cuh).
//
// Work: the (feature tile, 128-k block) units of the whole launch, in order, are cut into one range per CTA of a
// persistent grid (nk_grid: whole tiles when the launch has one to two tiles per SM, equal parts of every tile when
// it has fewer, equal ranges wherever they fall - stream-K - when it has more).  A tile that one CTA covers alone
// is finished by it; a tile cut across CTAs leaves FP32 partial tiles in scratch memory and the CTA that
// arrives last adds them in k order, so the bits do not depend on who was last.
// Every wait is bounded; on expiry the status word is raised and the CTA stops issuing, frees its TMEM and returns.
#pragma once

#include "gemm_stream.cuh"

namespace b200
{

constexpr int NK_BM = 128;                 // output features per tile (UMMA M)
constexpr int NK_BK = 128;                 // k per block: one 128-byte swizzle row of FP8
constexpr int NK_THREADS = 32 * 6;         // TMA warp, MMA warp, four epilogue warps (one per TMEM lane quarter)
constexpr int NK_HEADER_BYTES = 1024;
constexpr int NK_W_BYTES = NK_BM * NK_BK;  // one weight stage
constexpr int NK_MAX_TOKENS = 32;
constexpr int NK_SCALE_BYTES = 1024;       // the per-token 2^-s, ahead of the pieces in scratch memory
__host__ __device__ constexpr int nk_x_bytes(int bnp) { return bnp * NK_BK; }
__host__ __device__ constexpr int nk_stage_bytes(int bnp) { return NK_W_BYTES + nk_x_bytes(bnp); }
// two CTAs per SM: 113 KB each, less the header and the alignment slack
__host__ __device__ constexpr int nk_stages(int bnp)
{
    return (113 * 1024 - NK_HEADER_BYTES - 1024) / nk_stage_bytes(bnp) > 8 ? 8 : (113 * 1024 - NK_HEADER_BYTES - 1024) / nk_stage_bytes(bnp);
}
__host__ __device__ constexpr int nk_smem_bytes(int bnp) { return NK_HEADER_BYTES + nk_stages(bnp) * nk_stage_bytes(bnp) + 1024; }
// Consecutive UMMAs into ONE accumulator wait for each other (about 0.1 us each, whatever their size): the k steps of a
// block go round-robin to several accumulators, which the epilogue adds.
__host__ __device__ constexpr int nk_accs(int bnp) { return bnp <= 48 ? 4 : 2; }
__host__ __device__ constexpr int nk_tmem_cols(int bnp)
{
    return nk_accs(bnp) * bnp <= 32 ? 32 : (nk_accs(bnp) * bnp <= 64 ? 64 : (nk_accs(bnp) * bnp <= 128 ? 128 : 256));
}

struct NativeParams
{
    PrefillSeg seg[PF_MAX_GROUP];    // y_tma, blk, w_scale unused
    unsigned int n_seg;
    unsigned int* status;
    unsigned int M, K;
    unsigned int out_f32;            // 0 BF16, 1 FP32, 2 BF16 with the product rounded before beta * Y, 3 E4M3 (PIECES = 1 only)
    unsigned int tiles;              // feature tiles of all members
    unsigned int nkb;                // 128-k blocks of one tile
    const float* inv_scale;          // [M]: 2^-s of each token
    float act_inv;                   // the W8A8 pair kernels' activation multiplier when inv_scale is null (known on the host)
    float* partials;                 // [2 * grid][M][128]
    unsigned int* counters;          // [grid], zero between launches
    const uint16_t* X;               // the BF16 activations and their leading dimension (the form that splits them itself)
    unsigned int ldx;
};

// D[tmem] (+)= A[smem] * B[smem]; FP8 inputs (formats in the instruction descriptor), FP32 accumulate, 32 k.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor, kind::f8f6f4: D = F32 (bits 4-5 = 1), A format at bits 7-9 and B format at bits 10-12
// (0 E4M3, 1 E5M2), both K-major, N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__device__ __forceinline__ uint32_t umma_idesc_f8(bool a_e5m2, bool b_e5m2, uint32_t m, uint32_t n)
{
    return (1u << 4) | ((a_e5m2 ? 1u : 0u) << 7) | ((b_e5m2 ? 1u : 0u) << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// ---- the activations as three E5M2 rows per token ---------------------------------------------------------
// The largest finite magnitude of a token row (as BF16 bits) and whether it holds an infinity or a NaN: every block
// of the split kernels reads its whole row for this (a few KB out of L2), so that no second launch is needed.
__device__ __forceinline__ void row_absmax_bits(const uint16_t* __restrict__ x, unsigned int K, unsigned int* shared16, unsigned int& amax, unsigned int& bad)
{
    const unsigned int tid = threadIdx.x;
    amax = 0;
    bad = 0;
    for (unsigned int k0 = tid * 8; k0 < K; k0 += 256 * 8)
    {
        const uint4 v = *reinterpret_cast<const uint4*>(x + k0);
        const unsigned int w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int q = 0; q < 4; q++)
        {
            const unsigned int lo = w[q] & 0x7FFFu, hi = (w[q] >> 16) & 0x7FFFu;
            if (lo < 0x7F80u) { amax = max(amax, lo); }
            else { bad = 1; }
            if (hi < 0x7F80u) { amax = max(amax, hi); }
            else { bad = 1; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, o);
    }
    if ((tid & 31u) == 0)
    {
        shared16[tid >> 5] = amax;
        shared16[8 + (tid >> 5)] = bad;
    }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; w++)
    {
        amax = max(amax, shared16[w]);
        bad |= shared16[8 + w];
    }
}

// x * scale (a power of two) as three E5M2 bytes whose values add up to it: E5M2 is the upper byte of FP16, so rounding
// toward zero and dropping the lower byte truncates the magnitude to three significant bits (subnormals included), and
// every remainder keeps the sign and is exact in FP32.  An infinity or a NaN is carried by the first byte.
__device__ __forceinline__ void split_bf16_e5m2x3(unsigned int bits, float scale, unsigned int& a, unsigned int& b, unsigned int& c)
{
    const float v = __uint_as_float(bits << 16) * scale;
    a = __half_as_ushort(__float2half_rz(v));
    b = 0;
    c = 0;
    if ((bits & 0x7F80u) == 0x7F80u) { a = (bits & 0x007Fu) ? 0x7F00u : ((bits & 0x8000u) | 0x7C00u); }
    else
    {
        const float r1 = v - __half2float(__ushort_as_half((unsigned short)(a & 0xFF00u)));
        b = __half_as_ushort(__float2half_rz(r1));
        const float r2 = r1 - __half2float(__ushort_as_half((unsigned short)(b & 0xFF00u)));
        c = __half_as_ushort(__float2half_rz(r2));
    }
    a >>= 8;
    b >>= 8;
    c >>= 8;
}
// The power of two that lifts a row's largest finite magnitude (BF16 bits) to exponent 15: E5M2's largest finite value
// is 1.75 * 2^15, and a BF16 at that exponent is below 2^16, which FP16 still holds exactly.
__device__ __forceinline__ int e5m2_row_shift(unsigned int amax_bits)
{
    if (amax_bits == 0) { return 0; }
    const int s = 142 - (int)(amax_bits >> 7);
    return s > 126 ? 126 : s;
}

constexpr int NK_SPLIT_CHUNK = 256 * 8;    // k per block of the split kernel: eight per thread
// Grid (k chunks, tokens).  pieces [3 * M][K] bytes, row 3 t + j = piece j of token t; inv_scale[t] = 2^-s.
static __global__ void __launch_bounds__(256) split_activations_kernel(const uint16_t* __restrict__ X, unsigned int ldx, unsigned int K,
    uint8_t* __restrict__ pieces, float* __restrict__ inv_scale, unsigned int pad_rows)
{
    __shared__ unsigned int red[16];
    pdl_launch_dependents();
    pdl_wait();    // X is the previous kernel's output; the pieces may still be read by the linear before that
    const unsigned int t = blockIdx.y, tid = threadIdx.x;
    if (t == 0 && pad_rows != 0)
    {
        // the rows between 3 M and the UMMA's N are zero, so that the tensor map covers whole boxes (a TMA box with rows
        // out of bounds is slow)
        const unsigned int k0 = blockIdx.x * NK_SPLIT_CHUNK + tid * 8;
        if (k0 < K)
        {
            for (unsigned int r = 3 * gridDim.y; r < 3 * gridDim.y + pad_rows; r++) { *reinterpret_cast<uint2*>(pieces + (size_t)r * K + k0) = make_uint2(0u, 0u); }
        }
    }
    const uint16_t* x = X + (size_t)t * ldx;
    unsigned int amax, bad;
    row_absmax_bits(x, K, red, amax, bad);
    const int s = e5m2_row_shift(amax);
    const float scale = __uint_as_float((unsigned int)(127 + s) << 23);
    if (blockIdx.x == 0 && tid == 0) { inv_scale[t] = __uint_as_float((unsigned int)(127 - s) << 23); }
    const unsigned int k0 = blockIdx.x * NK_SPLIT_CHUNK + tid * 8;
    if (k0 >= K) { return; }
    const uint4 va = *reinterpret_cast<const uint4*>(x + k0);
    const unsigned int w[4] = { va.x, va.y, va.z, va.w };
    unsigned int o0[2] = { 0, 0 }, o1[2] = { 0, 0 }, o2[2] = { 0, 0 };
#pragma unroll
    for (int q = 0; q < 8; q++)
    {
        unsigned int a, b, c;
        split_bf16_e5m2x3((q & 1) ? (w[q >> 1] >> 16) : (w[q >> 1] & 0xFFFFu), scale, a, b, c);
        const int sh = 8 * (q & 3);
        o0[q >> 2] |= a << sh;
        o1[q >> 2] |= b << sh;
        o2[q >> 2] |= c << sh;
    }
    uint8_t* p0 = pieces + (size_t)(3 * t) * K + k0;
    *reinterpret_cast<uint2*>(p0) = make_uint2(o0[0], o0[1]);
    *reinterpret_cast<uint2*>(p0 + K) = make_uint2(o1[0], o1[1]);
    *reinterpret_cast<uint2*>(p0 + 2 * (size_t)K) = make_uint2(o2[0], o2[1]);
}

// The parts of a tile that was cut across CTAs c_first .. c_last, added in that (k) order into v.  CTA c_first left its
// part in its second slot, the others in their first.  About 32 loads are issued together - every token of as many
// parts as that allows - so that the CTA that arrived last waits for memory once per batch, not once per value;
// absent parts add an exact 0.
template <int TOK>
__device__ __forceinline__ void nk_sum_parts(const float* __restrict__ partials, unsigned int M, unsigned int c_first, unsigned int c_last, unsigned int f,
    float (&v)[TOK])
{
    constexpr int PB = TOK >= 32 ? 1 : (32 / TOK > 8 ? 8 : 32 / TOK);
#pragma unroll
    for (int t = 0; t < TOK; t++) { v[t] = 0.f; }
    for (unsigned int c0 = c_first; c0 <= c_last; c0 += PB)
    {
        float tmp[PB][TOK];
#pragma unroll
        for (int i = 0; i < PB; i++)
        {
            const unsigned int c = c0 + i;
            const float* part = partials + (size_t)(2 * c + (c == c_first ? 1u : 0u)) * M * NK_BM;
#pragma unroll
            for (int t = 0; t < TOK; t++) { tmp[i][t] = (c <= c_last && (unsigned int)t < M) ? __ldcg(part + t * NK_BM + f) : 0.f; }
        }
#pragma unroll
        for (int i = 0; i < PB; i++)
        {
#pragma unroll
            for (int t = 0; t < TOK; t++) { v[t] += tmp[i][t]; }
        }
    }
}

// ---- the linear -------------------------------------------------------------------------------------------
// BNP = UMMA N = 3 * tokens rounded up to a multiple of 16 (the rows past 3 * M are zero: the TMA's fill, or written so).
// FUSED: no split kernel ran.  Four more warps read the BF16 activations themselves - first every token's whole row
// for its largest magnitude, then, one k block ahead of the UMMAs, the 128 activations of each token that the block
// needs - and write the three E5M2 rows into the stage's B tile in the layout the TMA would have produced.  One kernel
// less on the critical path between the previous kernel's activations and this one's outputs; taken for few tokens,
// where every CTA re-reading the rows costs little.
// PIECES = 3: BF16 activations as three E5M2 rows per token (W8A16).  PIECES = 1: the activations ARE FP8 (E4M3, one row
// per token, quantised with one scale for the whole tensor): the W8A8 linear of gemm_w8a8.cuh.
template <int WT, int BNP, bool FUSED, int PIECES = 3>
// (The bounds name 32 threads more than are launched: two CTAs then leave registers for a 256-thread block of the
// kernel that comes next on the stream - the split of the next linear's activations - to start beside them.)
__global__ void __launch_bounds__((FUSED ? NK_THREADS + 128 : NK_THREADS) + 32, 2) gemm_wq_native_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ StreamWMaps tmW, const NativeParams p)
{
    constexpr int STAGES = nk_stages(BNP);
    constexpr int STAGE_BYTES = nk_stage_bytes(BNP);
    constexpr int X_BYTES = nk_x_bytes(BNP);
    constexpr int TMEM_COLS = nk_tmem_cols(BNP);
    constexpr int TOK = BNP / PIECES;    // tokens one accumulator holds
    static_assert(PIECES == 3 || (PIECES == 1 && !FUSED), "pieces");
    constexpr int ACCS = nk_accs(BNP);
    static_assert(STAGES >= 2 && STAGES <= 8, "ring depth");
    static_assert(ACCS * BNP <= TMEM_COLS && (NK_BK / 32) % ACCS == 0, "accumulators");
    extern __shared__ unsigned char nk_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(nk_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + 8;
    uint64_t* acc_full = empty + 8;
    uint64_t* acc_empty = acc_full + 1;
    uint64_t* b_full = acc_empty + 1;        // [8], FUSED: the B tile of a stage has been written
    uint64_t* scale_ready = b_full + 8;      // FUSED: the tokens' 2^-s are in shared memory
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(scale_ready + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(tmem_base_slot + 1);
    volatile unsigned int* last_flag = abort_flag + 1;
    volatile unsigned int* go_flag = abort_flag + 2;
    float* inv_scale_s = reinterpret_cast<float*>(smem + 512);             // [TOK]
    unsigned int* row_max_s = reinterpret_cast<unsigned int*>(smem + 640);    // [TOK][4]
    unsigned char* stages = smem + NK_HEADER_BYTES;

    const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned long long U = (unsigned long long)p.tiles * p.nkb;
    const unsigned int G = gridDim.x;
    const unsigned int u0 = (unsigned int)((U * blockIdx.x) / G), u1 = (unsigned int)((U * (blockIdx.x + 1ull)) / G);
    const unsigned int n_units = u1 - u0;

    // which member of the group a tile belongs to
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
        mbar_expect_tx(full + s, NK_W_BYTES);
        tma_load_2d_hint(stages + s * STAGE_BYTES, &tmW.w[si], (int)(kb * NK_BK), (int)((tile - p.seg[si].tile0) * NK_BM), full + s, pol);
        if (FUSED) { mbar_arrive(full + s); }
    };
    const unsigned int pre = n_units < (unsigned int)STAGES ? n_units : (unsigned int)STAGES;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; s++)
        {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
            mbar_init(b_full + s, 4);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
        mbar_init(scale_ready, 1);
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The weights depend on nothing - not on the previous kernel, not on the rest of this CTA: the first ring of
        // stages is asked for before the CTA has even met (this thread is the TMA lane).
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
                mbar_expect_tx(full + s, X_BYTES);
                tma_load_2d(stages + s * STAGE_BYTES + NK_W_BYTES, &tmX, (int)(kb * NK_BK), 0, full + s);
                mbar_arrive(full + s);
            };
            if (!FUSED)
            {
                pdl_wait();
                for (unsigned int i = 0; i < pre; i++) { issue_acts(i); }
            }
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
                if (!FUSED) { issue_acts(i); }
                issued = i + 1;
            }
            // do not leave while copies are in flight: wait (bounded) for the stages still outstanding
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
        const uint32_t idesc = umma_idesc_f8(WT == DT_E5M2, PIECES == 3, NK_BM, BNP);
        unsigned int runs_done = 0;    // accumulations this CTA has handed to the epilogue
        bool ok = true;
        for (unsigned int i = 0; i < n_units && ok; i++)
        {
            const unsigned int kb = (u0 + i) % p.nkb, s = i % STAGES;
            const bool first = kb == 0 || i == 0;
            const bool last = kb + 1 == p.nkb || i + 1 == n_units;
            if (first && runs_done > 0 && (*abort_flag != 0 || !mbar_wait_bounded(acc_empty, (runs_done - 1) & 1u))) { ok = false; }
            if (ok && (*abort_flag != 0 || !mbar_wait_bounded(full + s, (i / STAGES) & 1u))) { ok = false; }
            if (FUSED && ok && !mbar_wait_bounded(b_full + s, (i / STAGES) & 1u)) { ok = false; }
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
                const uint32_t a_addr = smem_u32(stages + s * STAGE_BYTES), b_addr = a_addr + NK_W_BYTES;
#pragma unroll
                for (int k = 0; k < NK_BK / 32; k++)
                {
                    umma_f8(tmem_base + (k % ACCS) * BNP, umma_desc_kmajor_sw128(a_addr + k * 32), umma_desc_kmajor_sw128(b_addr + k * 32), idesc,
                        (first && k < ACCS) ? 0u : 1u);
                }
                umma_commit(empty + s);
                if (last) { umma_commit(acc_full); }
            }
            __syncwarp();
            if (last) { runs_done++; }
        }
    }
    else if (FUSED && warp >= 6)
    {
        // =========================== FUSED: the activations as three E5M2 rows (warps 6..9) ===========================
        const unsigned int ptid = threadIdx.x - 192;
        // rows past 3 M stay zero for the whole kernel
        for (int s = 0; s < STAGES; s++)
        {
            for (unsigned int i = ptid; i < (unsigned int)(X_BYTES / 16); i += 128) { sts128(smem_u32(stages + s * STAGE_BYTES + NK_W_BYTES) + i * 16, 0u, 0u, 0u, 0u); }
        }
        pdl_wait();    // the activations are the previous kernel's output
        // every token's largest finite magnitude, over its whole row
        float scale[TOK];
#pragma unroll
        for (int t = 0; t < TOK; t++)
        {
            scale[t] = 1.f;
            if ((unsigned int)t >= p.M) { continue; }
            const uint16_t* x = p.X + (size_t)t * p.ldx;
            unsigned int amax = 0;
            for (unsigned int k0 = ptid * 8; k0 < p.K; k0 += 128 * 8)
            {
                const uint4 v = *reinterpret_cast<const uint4*>(x + k0);
                const unsigned int w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
                for (int q = 0; q < 4; q++)
                {
                    const unsigned int lo = w[q] & 0x7FFFu, hi = (w[q] >> 16) & 0x7FFFu;
                    if (lo < 0x7F80u) { amax = max(amax, lo); }
                    if (hi < 0x7F80u) { amax = max(amax, hi); }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o)); }
            if (lane == 0) { row_max_s[t * 4 + (warp - 6)] = amax; }
        }
        bar_sync_named(2, 128);
#pragma unroll
        for (int t = 0; t < TOK; t++)
        {
            if ((unsigned int)t >= p.M) { continue; }
            const unsigned int amax = max(max(row_max_s[t * 4], row_max_s[t * 4 + 1]), max(row_max_s[t * 4 + 2], row_max_s[t * 4 + 3]));
            const int sh = e5m2_row_shift(amax);
            scale[t] = __uint_as_float((unsigned int)(127 + sh) << 23);
            if (ptid == (unsigned int)t) { inv_scale_s[t] = __uint_as_float((unsigned int)(127 - sh) << 23); }
        }
        bar_sync_named(2, 128);
        if (ptid == 0) { mbar_arrive(scale_ready); }
        // thread j writes byte j of the block's rows: k = 128 kb + j
        unsigned int nxt[TOK];
        auto fetch = [&](unsigned int i) {
            const uint16_t* xk = p.X + (size_t)((u0 + i) % p.nkb) * NK_BK + ptid;
#pragma unroll
            for (int t = 0; t < TOK; t++)
            {
                if ((unsigned int)t < p.M) { nxt[t] = __ldg(xk + (size_t)t * p.ldx); }
            }
        };
        if (n_units > 0) { fetch(0); }
        for (unsigned int i = 0; i < n_units; i++)
        {
            const unsigned int s = i % STAGES;
            unsigned int cur[TOK];
#pragma unroll
            for (int t = 0; t < TOK; t++) { cur[t] = nxt[t]; }
            if (i + 1 < n_units) { fetch(i + 1); }
            if (i >= (unsigned int)STAGES && (*abort_flag != 0 || !mbar_wait_bounded(empty + s, ((i / STAGES) - 1) & 1u)))
            {
                atomicMax(p.status, (unsigned int)ST_TIMEOUT_EMPTY);
                *abort_flag = 1;
                break;
            }
            const uint32_t b_tile = smem_u32(stages + s * STAGE_BYTES + NK_W_BYTES);
#pragma unroll
            for (int t = 0; t < TOK; t++)
            {
                if ((unsigned int)t >= p.M) { continue; }
                unsigned int pc[3];
                split_bf16_e5m2x3(cur[t], scale[t], pc[0], pc[1], pc[2]);
#pragma unroll
                for (int j = 0; j < 3; j++)
                {
                    // the 128-byte swizzle: 16-byte chunk index ^= row % 8
                    const unsigned int row = 3 * t + j;
                    const uint32_t addr = b_tile + row * 128 + ((((ptid >> 4) ^ row) & 7u) << 4) + (ptid & 15u);
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(pc[j]) : "memory");
                }
            }
            fence_proxy_async();    // the UMMA reads the tile through the async proxy
            __syncwarp();
            if (lane == 0) { mbar_arrive(b_full + s); }
        }
    }
    else
    {
        // =========================== epilogue (warps 2..5) ===========================
        const unsigned int quarter = warp & 3u;    // the TMEM lanes a warp may read: 32 (warp % 4) ..
        const unsigned int f = quarter * 32 + lane;
        const unsigned int etid = threadIdx.x - 64;
        pdl_wait();    // Y, the scales and the scratch memory belong to the stream's order
        if (FUSED && !mbar_wait_bounded(scale_ready, 0))
        {
            atomicMax(p.status, (unsigned int)ST_TIMEOUT_FULL);
            *abort_flag = 1;
        }
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
            // the four warps meet at named barriers below: they go on or stop TOGETHER, on one thread's reading of the flag
            bar_sync_named(1, 128);
            if (etid == 0) { *go_flag = *abort_flag == 0 ? 1u : 0u; }
            bar_sync_named(1, 128);
            if (*go_flag == 0) { break; }
            tc_fence_after();
            float v[TOK];
            {
                float acc[BNP];
#pragma unroll
                for (int a = 0; a < ACCS; a++)
                {
#pragma unroll
                    for (int c = 0; c < BNP; c += 16)
                    {
                        uint32_t r[16];
                        tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + a * BNP + c, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 16; q++) { acc[c + q] = a == 0 ? __uint_as_float(r[q]) : acc[c + q] + __uint_as_float(r[q]); }
                    }
                }
#pragma unroll
                for (int t = 0; t < TOK; t++) { v[t] = PIECES == 3 ? (acc[PIECES * t] + acc[PIECES * t + PIECES / 2]) + acc[PIECES * t + PIECES - 1] : acc[t]; }
            }
            // the accumulator is in registers: the MMA warp may start the next tile
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(acc_empty); }

            const unsigned int si = member_of(tile);
            const PrefillSeg& g = p.seg[si];
            const unsigned int n = (tile - g.tile0) * NK_BM + f;
            bool write_out = u == tile_begin && e == tile_end;
            if (!write_out)
            {
                // part of a tile: leave it in scratch memory; the last of the tile's CTAs to arrive adds the parts
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
                    if (is_last) { p.counters[c_first] = 0; }    // zero again for the next launch
                    *last_flag = is_last;
                }
                bar_sync_named(1, 128);
                write_out = *last_flag != 0;
                if (write_out)
                {
                    __threadfence();
                    nk_sum_parts<TOK>(p.partials, p.M, c_first, c_last, f, v);
                }
                bar_sync_named(1, 128);    // everybody has read last_flag before the next tile's writes it
            }
            if (write_out && n < g.N)
            {
#pragma unroll
                for (int t = 0; t < TOK; t++)
                {
                    if ((unsigned int)t >= p.M) { break; }
                    const long long yi = (long long)t * g.ldy_m + (long long)n * g.ldy_n;
                    float o = g.alpha * ((v[t] * (FUSED ? inv_scale_s[t] : __ldg(p.inv_scale + t))) * g.post_scale);
                    if (p.out_f32 == 1u)
                    {
                        float* y = reinterpret_cast<float*>(g.Y) + yi;
                        if (g.beta != 0.f) { o += g.beta * *y; }
                        *y = o;
                    }
                    else if (PIECES == 1 && p.out_f32 == 3u)
                    {
                        // E4M3 output of the W8A8 mode: the BF16 result re-encoded at scale 1 with the reference's encoder,
                        // beta ignored (cccc/cublas_real.h:787-834)
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
            u = e;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) { tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---- host side -----------------------------------------------------------------------------------------
// CTAs of a launch.  With more feature tiles than CTA slots: one CTA per slot, the units dealt out evenly (tiles are cut
// wherever a range ends; on such launches the exchange is a small share).  With fewer: every tile is cut into the same
// number of parts, as many as the slots allow (one part = the whole tile and no exchange between half the slots and all
// of them), so that no CTA works on two tiles and each meets the exchange once.  CTAs share HBM, not SMs: 192 whole-tile
// CTAs on 148 SMs finish together.
static inline unsigned int nk_grid(unsigned int tiles, unsigned int nkb, unsigned long long slots)
{
    if (tiles > slots) { return (unsigned int)slots; }
    unsigned long long parts = slots / tiles;
    if (parts > nkb) { parts = nkb; }
    return (unsigned int)(tiles * parts);
}

inline bool native_supported(int w_type, unsigned int N, unsigned int M, unsigned int K, unsigned int ldw, unsigned int ldx)
{
    if (w_type != DT_E4M3 && w_type != DT_E5M2) { return false; }
    return M >= 1 && M <= (unsigned int)NK_MAX_TOKENS && N > 0 && K > 0 && (K % NK_BK) == 0 && (ldx % 8) == 0 && (ldw % 16) == 0;
}

constexpr int NK_FUSED_MAX_TOKENS = 8;    // up to here every CTA splits the activations itself

template <int WT, int BNP, bool FUSED>
static int launch_native_bn(const void* X, unsigned int ldx, NativeParams& np, unsigned char* scratch, size_t scratch_bytes, unsigned int n_counters,
    int device, int sm_count, cudaStream_t stream, bool pdl)
{
    const unsigned long long U = (unsigned long long)np.tiles * np.nkb;
    if (U == 0 || U > 0x7FFFFFFFull) { return -2; }
    const unsigned int grid = nk_grid(np.tiles, np.nkb, 2ull * (unsigned)sm_count);
    // scratch memory: (the tokens' 2^-s and their pieces, when a kernel of its own writes them,) then two partial tiles per CTA
    const size_t piece_bytes = FUSED ? 0 : ((((size_t)BNP * np.K) + 1023) & ~(size_t)1023) + NK_SCALE_BYTES;
    const size_t part_bytes = (size_t)2 * grid * np.M * NK_BM * sizeof(float);
    if (piece_bytes + part_bytes > scratch_bytes || grid > n_counters || ((uintptr_t)scratch & 255u) != 0) { return -2; }
    float* inv_scale = reinterpret_cast<float*>(scratch);
    uint8_t* pieces = scratch + NK_SCALE_BYTES;
    np.inv_scale = inv_scale;
    np.partials = reinterpret_cast<float*>(scratch + piece_bytes);
    np.X = (const uint16_t*)X;
    np.ldx = ldx;

    CUtensorMap tmX;
    StreamWMaps tmW;
    memset(&tmX, 0, sizeof(tmX));
    memset(&tmW, 0, sizeof(tmW));
    bool ok = FUSED || make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pieces, np.K, (unsigned long long)BNP, np.K, NK_BK, BNP, true);
    for (unsigned int j = 0; j < (unsigned)PF_MAX_GROUP && ok; j++)
    {
        const PrefillSeg& g = np.seg[j < np.n_seg ? j : 0];
        ok = make_map_2d(&tmW.w[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.W, np.K, g.N, g.ldw, NK_BK, NK_BM, true);
    }
    if (!ok) { return -2; }
    auto kernel = gemm_wq_native_kernel<WT, BNP, FUSED>;
    static std::atomic<bool> attr_set[64];
    if (!attr_set[device].load(std::memory_order_acquire))
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, nk_smem_bytes(BNP)) != cudaSuccess)
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
    cfg.stream = stream;
    cfg.attrs = attr;
    if (!FUSED)
    {
        cfg.gridDim = dim3((np.K + NK_SPLIT_CHUNK - 1) / NK_SPLIT_CHUNK, np.M);
        cfg.blockDim = dim3(256);
        cfg.numAttrs = pdl ? 1 : 0;
        count_launch();
        if (cudaLaunchKernelEx(&cfg, split_activations_kernel, (const uint16_t*)X, ldx, np.K, pieces, inv_scale, (unsigned int)BNP - 3u * np.M) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16");
            return 1;
        }
    }
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(FUSED ? NK_THREADS + 128 : NK_THREADS);
    cfg.dynamicSmemBytes = nk_smem_bytes(BNP);
    // behind the split kernel the linear always launches early (its weight prefetch does not depend on it)
    cfg.numAttrs = (!FUSED || pdl) ? 1 : 0;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, kernel, tmX, tmW, np) != cudaSuccess)
    {
        report_launch("gemm_wq_bf16");
        return 1;
    }
    return 0;
}

// One launch (plus the split of the activations) for up to PF_MAX_GROUP linears that share X.  -2: not taken.
static int launch_native(int w_type, const GemvParams* items, unsigned int count, float* scratch, size_t scratch_bytes, unsigned int* counters,
    unsigned int n_counters, int device, int sm_count, cudaStream_t stream, bool pdl, bool own_split_kernel = false)
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
    np.nkb = np.K / NK_BK;
    for (unsigned int j = 0; j < count; j++)
    {
        if (!native_supported(w_type, items[j].N, items[j].M, items[j].K, items[j].ldw, items[j].ldx)) { return -2; }
        // a scale that is not a power of two is folded into the weights before their BF16 rounding by the
        // reference's conversion: only the kernels that dequantise can reproduce that
        if (!sk_al16(items[j].W) || !pf_is_pow2_scale(items[j].w_scale)) { return -2; }
        PrefillSeg& g = np.seg[j];
        g.W = items[j].W;
        g.Y = items[j].Y;
        g.N = items[j].N;
        g.ldw = items[j].ldw;
        g.ldy_m = items[j].ldy_m;
        g.ldy_n = items[j].ldy_n;
        g.alpha = items[j].alpha;
        g.beta = items[j].beta;
        g.w_scale = 1.0f;
        g.post_scale = items[j].w_scale;
        g.tile0 = np.tiles;
        np.tiles += (items[j].N + NK_BM - 1) / NK_BM;
    }
    if (!sk_al16(items[0].X)) { return -2; }
    const void* X = items[0].X;
    const unsigned int ldx = items[0].ldx;
    unsigned char* sc = reinterpret_cast<unsigned char*>(scratch);
#define NK_LAUNCH(WT_, BNP_, F_) launch_native_bn<WT_, BNP_, F_>(X, ldx, np, sc, scratch_bytes, n_counters, device, sm_count, stream, pdl)
    const bool fused = np.M <= (unsigned int)NK_FUSED_MAX_TOKENS && !own_split_kernel;
    if (w_type == DT_E5M2)
    {
        if (np.M <= 5) { return fused ? NK_LAUNCH(DT_E5M2, 16, true) : NK_LAUNCH(DT_E5M2, 16, false); }
        if (np.M <= 10) { return fused ? NK_LAUNCH(DT_E5M2, 32, true) : NK_LAUNCH(DT_E5M2, 32, false); }
        if (np.M <= 16) { return NK_LAUNCH(DT_E5M2, 48, false); }
        return NK_LAUNCH(DT_E5M2, 96, false);
    }
    if (np.M <= 5) { return fused ? NK_LAUNCH(DT_E4M3, 16, true) : NK_LAUNCH(DT_E4M3, 16, false); }
    if (np.M <= 10) { return fused ? NK_LAUNCH(DT_E4M3, 32, true) : NK_LAUNCH(DT_E4M3, 32, false); }
    if (np.M <= 16) { return NK_LAUNCH(DT_E4M3, 48, false); }
    return NK_LAUNCH(DT_E4M3, 96, false);
#undef NK_LAUNCH
}

}    // namespace b200
