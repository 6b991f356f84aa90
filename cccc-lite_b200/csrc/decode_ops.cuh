// Device code of the non-GEMM ops of an LLM decode layer, written so that a CTA-sized team of
// 256 threads can run them either as a kernel of their own (decode_ops.cu) or as one phase of a
// longer-running kernel: RMSNorm with the reference's summation order, half-rotate RoPE, the
// KV-cache append, and attention of one new token per sequence over a BF16 cache.
//
// Rounding points are the reference's: every tensor the reference materialises in BF16 (the
// normalised row, the rotated q and k, the scaled scores, the softmax probabilities, the attention
// output) is rounded to BF16 here at the same place, although nothing but the final output leaves
// the chip.
#pragma once

#include "common.cuh"
#include "gemv_decode.cuh"

#include <cooperative_groups.h>

namespace b200
{

constexpr int kTeam = 256;    // threads of a team; team barriers are bar.sync 1, 256

__device__ __forceinline__ void team_sync() { consumer_bar_sync<kTeam>(); }

__device__ __forceinline__ float bf16_round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ uint16_t bf16_bits(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }

// Sum of squares of `rows` rows of `inner` floats held in shared memory (xs[row * inner + i]), in
// the order of the reference's kernel (cccc-cuda/cuda_functions.cu:904-933, 256 threads per row):
// thread t accumulates x[t], x[t+256], ... with one fused multiply-add each, then the 256 partial
// sums are combined by a halving tree.  part: rows * 256 floats of shared memory.  On return
// part[row * 256] holds the sum of row `row`; all 256 threads of the team must call.
// The halving tree over the 256 per-thread partial sums of each row (part[row * 256 + thread]):
// p[t] += p[t + s] for s = 128, 64, ..., 1, exactly the additions of the reference's kernel.  The
// levels that cross warps go through shared memory; the last five stay inside warp 0, where
// p[t] += p[t + s] is a shuffle-down (lanes >= s compute values that are never used again).
__device__ __forceinline__ void team_tree_sum(float* part, unsigned int rows, unsigned int tid)
{
    team_sync();
    for (unsigned int s = kTeam / 2; s >= 32; s >>= 1)
    {
        if (tid < s)
        {
            for (unsigned int r = 0; r < rows; r++) { part[r * kTeam + tid] += part[r * kTeam + tid + s]; }
        }
        team_sync();
    }
    if (tid < 32)
    {
        for (unsigned int r = 0; r < rows; r++)
        {
            float v = part[r * kTeam + tid];
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) { v += __shfl_down_sync(0xFFFFFFFFu, v, s); }
            if (tid == 0) { part[r * kTeam] = v; }
        }
    }
    team_sync();
}
__device__ __forceinline__ void team_sum_squares(const float* xs, float* part, unsigned int rows, unsigned int inner, unsigned int tid)
{
    for (unsigned int r = 0; r < rows; r++)
    {
        float s = 0.f;
        for (unsigned int i = tid; i < inner; i += kTeam) { s = __fmaf_rn(xs[r * inner + i], xs[r * inner + i], s); }
        part[r * kTeam + tid] = s;
    }
    team_tree_sum(part, rows, tid);
}

// invstd of the reference: rsqrtf(sum / inner + eps).
__device__ __forceinline__ float rms_invstd(float sum, unsigned int inner, float eps) { return rsqrtf(sum / (float)inner + eps); }

// y = bf16((x * invstd) * scale), the reference's expression (two roundings-free float products).
__device__ __forceinline__ float rms_apply(float x, float invstd, float sc) { return bf16_round(__fmul_rn(__fmul_rn(x, invstd), sc)); }

// Half-rotate RoPE of one pair (cccc-cuda/cuda_functions.cu:1324-1344): one product rounded, the
// other fused into the add, then BF16.
__device__ __forceinline__ void rope_pair(float xl, float xr, float c, float s, float& yl, float& yr)
{
    yl = bf16_round(__fmaf_rn(xl, c, -__fmul_rn(xr, s)));
    yr = bf16_round(__fmaf_rn(xr, c, __fmul_rn(xl, s)));
}

// out = bf16( bf16( g * bf16(sigmoid(g)) ) * u ): the reference's silu (a BF16 sigmoid tensor times
// the input, MatrixEx.cpp:744-763) followed by elementMul (Matrix.cpp:1360-1386).
__device__ __forceinline__ float swiglu_one(float g, float u)
{
    const float s = bf16_round(1.0f / (1.0f + expf(-g)));
    return bf16_round(__fmul_rn(bf16_round(__fmul_rn(g, s)), u));
}

// 16-bit load that never comes from this SM's L1 (data another CTA of the same kernel may have written)
__device__ __forceinline__ float ld_bf16_cg(const uint16_t* p) { return bf16_bits_to_float(__ldcg(p)); }

// ---- attention of one new token per sequence ------------------------------------------------------
struct AttnDecodeParams
{
    const uint16_t* q;       // [B][ldq]: H heads of HD
    const uint16_t* k;       // [B][ldk]: Hkv heads of HD (the new token's key, before norm and RoPE)
    const uint16_t* v;       // [B][ldv]
    const uint16_t* q_norm;  // [HD] or nullptr
    const uint16_t* k_norm;  // [HD] or nullptr
    const uint16_t* cos_tab; // [rows][HD/2]
    const uint16_t* sin_tab;
    uint16_t* k_cache;       // [B][Hkv][T_max][HD]
    uint16_t* v_cache;
    const int* pos;          // [B]: where the new token goes = index of the newest valid row afterwards
    uint16_t* out;           // [B][ldo]: H heads of HD
    unsigned int ldq, ldk, ldv, ldo;
    unsigned int B, H, Hkv, T_max;
    float eps, scale;        // RMSNorm epsilon of the q/k norms; 1/sqrt(dk)
};

constexpr int kAttnRingK = 4;     // passes of 32 rows (8 KB at head_dim 128); even: the loop consumes two per turn
constexpr int kAttnRingV = 8;     // passes of 16 rows (4 KB at head_dim 128)
template <int HD>
__host__ __device__ constexpr size_t attn_ring_bytes()
{
    return (size_t)kTeam * 16 * ((kAttnRingK * (HD / 64)) > kAttnRingV ? (kAttnRingK * (HD / 64)) : kAttnRingV);
}

// floats of the region that serves as the K / V ring during the passes and as the cross-slot reduction buffer after them
template <int G, int HD>
__host__ __device__ constexpr size_t attn_red_floats()
{
    return (size_t)(kTeam / (HD / 8)) * G * HD > attn_ring_bytes<HD>() / 4 ? (size_t)(kTeam / (HD / 8)) * G * HD : attn_ring_bytes<HD>() / 4;
}

// Shared memory of one attention team (floats): see attn_smem_floats().
template <int G, int HD>
struct AttnSmem
{
    static constexpr int kSlots2 = kTeam / (HD / 8);    // token slots of the P*V pass
    float* qs;      // [G][HD]   rotated q, BF16-rounded
    float* kn;      // [HD]      rotated new k (owner split only)
    float* xin;     // [G+1][HD] raw q heads and the k head (norm input)
    float* part;    // [G+1][256] partial sums of the norms
    float* ml;      // [G][2]    this split's max and sum of exponentials
    float* gl;      // [G][2]    the sequence's max and 1/sum
    float* opart;   // [G][HD]   this split's partial output
    float* red;     // [kSlots2][G][HD]; the K / V ring (attn_ring_bytes) lives here while the passes run
    float* wq;      // [HD] q-norm weights, [HD] k-norm weights, [HD/2] cos row, [HD/2] sin row
    float* sc;      // [G][ts_cap] scores, then probabilities
    __device__ AttnSmem(float* base, unsigned int ts_cap)
    {
        qs = base;
        kn = qs + G * HD;
        xin = kn + HD;
        part = xin + (G + 1) * HD;
        ml = part + (G + 1) * kTeam;
        gl = ml + 2 * G;
        opart = gl + 2 * G;
        red = opart + G * HD;
        wq = red + attn_red_floats<G, HD>();
        sc = wq + 3 * HD;
        (void)ts_cap;
    }
};
template <int G, int HD>
__host__ __device__ constexpr size_t attn_smem_floats(unsigned int ts_cap)
{
    return (size_t)G * HD + HD + (size_t)(G + 1) * HD + (size_t)(G + 1) * kTeam + 4 * G + (size_t)G * HD
        + attn_red_floats<G, HD>() + 3 * HD + (size_t)G * ts_cap;
}

// 16-byte asynchronous copy global -> shared that bypasses L1 (cp.async.cg); `valid` false fills zeros without
// reading.  Each thread later reads back only what it copied itself, so cp.async.wait_group is all it needs.
__device__ __forceinline__ void cp_async16(uint4* smem_dst, const void* gmem_src, bool valid)
{
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const uint32_t bytes = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8])
{
    const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
    for (int i = 0; i < 4; i++)
    {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

// Prologue of a split: the G query heads of kv head `kvh` of sequence b are normalised (optional)
// and rotated into sm.qs; the split that owns row `pos` also normalises and rotates the new key,
// appends it and the new value to the caches (MatrixOp.cpp:237-276) and keeps the key in sm.kn.
// Every global input (q heads, k head, the two norm weights, the cos and sin rows of `pos`) is
// fetched in ONE round trip, one 16-byte piece per thread; q and k rows must be 16-byte aligned.
template <int G, int HD>
__device__ __forceinline__ void attn_prologue(const AttnDecodeParams& p, AttnSmem<G, HD>& sm, unsigned int b, unsigned int kvh,
    unsigned int pos, bool owner, unsigned int tid)
{
    constexpr int HALF = HD / 2;
    constexpr unsigned int NQ = (G + 1) * HD / 8, NW = HD / 8, NT = HALF / 8;
    static_assert(NQ + 2 * NW + 2 * NT <= kTeam, "one piece per thread");
    {
        const uint16_t* q = p.q + (size_t)b * p.ldq + (size_t)kvh * G * HD;
        const uint16_t* k = p.k + (size_t)b * p.ldk + (size_t)kvh * HD;
        const uint16_t* src = nullptr;
        float* dst = nullptr;
        bool fresh = false;    // written by the previous phase or kernel: not through this SM's L1
        unsigned int i = tid;
        if (i < NQ)
        {
            src = i < G * HD / 8 ? q + i * 8 : k + (i - G * HD / 8) * 8;
            dst = sm.xin + i * 8;
            fresh = true;
        }
        else if ((i -= NQ) < NW)
        {
            src = p.q_norm ? p.q_norm + i * 8 : nullptr;
            dst = sm.wq + i * 8;
        }
        else if ((i -= NW) < NW)
        {
            src = p.k_norm ? p.k_norm + i * 8 : nullptr;
            dst = sm.wq + HD + i * 8;
        }
        else if ((i -= NW) < NT)
        {
            src = p.cos_tab + (size_t)pos * HALF + i * 8;
            dst = sm.wq + 2 * HD + i * 8;
        }
        else if ((i -= NT) < NT)
        {
            src = p.sin_tab + (size_t)pos * HALF + i * 8;
            dst = sm.wq + 2 * HD + HALF + i * 8;
        }
        if (dst != nullptr)
        {
            float f[8];
            if (src != nullptr)
            {
                const uint4 v = fresh ? __ldcg(reinterpret_cast<const uint4*>(src)) : __ldg(reinterpret_cast<const uint4*>(src));
                unpack8(v, f);
            }
            else
            {
#pragma unroll
                for (int e = 0; e < 8; e++) { f[e] = 1.f; }
            }
#pragma unroll
            for (int e = 0; e < 8; e++) { dst[e] = f[e]; }
        }
    }
    team_sync();
    if (p.q_norm != nullptr || p.k_norm != nullptr) { team_sum_squares(sm.xin, sm.part, G + 1, HD, tid); }
    // normalise in place (BF16-rounded, as the reference's rmsNorm output tensor is)
    for (unsigned int i = tid; i < (G + 1) * HD; i += kTeam)
    {
        const unsigned int r = i / HD, d = i - r * HD;
        const bool has = r < G ? p.q_norm != nullptr : p.k_norm != nullptr;
        if (has) { sm.xin[i] = rms_apply(sm.xin[i], rms_invstd(sm.part[r * kTeam], HD, p.eps), sm.wq[(r < G ? 0 : HD) + d]); }
    }
    team_sync();
    for (unsigned int i = tid; i < (G + 1) * HALF; i += kTeam)
    {
        const unsigned int r = i / HALF, d = i - r * HALF;
        float yl, yr;
        rope_pair(sm.xin[r * HD + d], sm.xin[r * HD + HALF + d], sm.wq[2 * HD + d], sm.wq[2 * HD + HALF + d], yl, yr);
        float* dst = r < G ? sm.qs + r * HD : sm.kn;
        dst[d] = yl;
        dst[HALF + d] = yr;
    }
    team_sync();
    if (owner && pos < p.T_max)
    {
        uint16_t* kc = p.k_cache + (((size_t)b * p.Hkv + kvh) * p.T_max + pos) * HD;
        uint16_t* vc = p.v_cache + (((size_t)b * p.Hkv + kvh) * p.T_max + pos) * HD;
        const uint16_t* v = p.v + (size_t)b * p.ldv + (size_t)kvh * HD;
        for (unsigned int i = tid; i < HD; i += kTeam)
        {
            kc[i] = bf16_bits(sm.kn[i]);
            vc[i] = __ldcg(v + i);
        }
    }
}

// The end of a scores pass: the team's maximum per head, then the sum of exp(score - maximum), into sm.ml.
template <int G, int HD>
__device__ __forceinline__ void attn_scores_finish(AttnSmem<G, HD>& sm, unsigned int t0, unsigned int t1, unsigned int ts_cap, unsigned int tid,
    float (&mx)[G])
{
    // maximum over the team, then the sum of exponentials
#pragma unroll
    for (int g = 0; g < G; g++)
    {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { mx[g] = fmaxf(mx[g], __shfl_xor_sync(0xFFFFFFFFu, mx[g], o)); }
        if ((tid & 31u) == 0) { sm.red[g * 8 + (tid >> 5)] = mx[g]; }
    }
    team_sync();
    if (tid < G)
    {
        float m = sm.red[tid * 8];
        for (int w = 1; w < 8; w++) { m = fmaxf(m, sm.red[tid * 8 + w]); }
        sm.ml[2 * tid] = m;
    }
    team_sync();
    float ls[G];
    const unsigned int n_rows = t1 > t0 ? t1 - t0 : 0;
#pragma unroll
    for (int g = 0; g < G; g++)
    {
        ls[g] = 0.f;
        const float m = sm.ml[2 * g];
        for (unsigned int i = tid; i < n_rows; i += kTeam) { ls[g] += __expf(sm.sc[g * ts_cap + i] - m); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { ls[g] += __shfl_xor_sync(0xFFFFFFFFu, ls[g], o); }
    }
    team_sync();    // sm.red is reused
#pragma unroll
    for (int g = 0; g < G; g++)
    {
        if ((tid & 31u) == 0) { sm.red[g * 8 + (tid >> 5)] = ls[g]; }
    }
    team_sync();
    if (tid < G)
    {
        float l = 0.f;
        for (int w = 0; w < 8; w++) { l += sm.red[tid * 8 + w]; }
        sm.ml[2 * tid + 1] = l;
    }
    team_sync();
}

// The ring form of attn_scores: K rows travel global -> shared by cp.async into a ring of kAttnRingK passes (32
// rows each) that belongs to the threads piece by piece (every thread reads back only its own 16-byte pieces, so
// no barrier is involved), and the copy of pass i + kAttnRingK is issued right after pass i has been consumed:
// the DRAM latency of a pass overlaps the arithmetic of the passes before it, and no registers hold data in
// flight.  (With registers as the buffer a pass was requested and then waited for: 32 KB in flight per team only
// between the request and its use, 0.49 of the HBM rate at 32 sequences x 4096 rows.)
template <int G, int HD>
__device__ __forceinline__ void attn_scores_ring(const AttnDecodeParams& p, AttnSmem<G, HD>& sm, unsigned int b, unsigned int kvh,
    unsigned int t0, unsigned int t1, unsigned int ts_cap, unsigned int pos, bool owner, unsigned int tid, uint4* ring)
{
    constexpr int CPL = HD / 64;    // 16-byte pieces per lane
    constexpr int D = kAttnRingK;
    const unsigned int sub = tid & 7u, slot = tid >> 3;
    const uint16_t* Kb = p.k_cache + ((size_t)b * p.Hkv + kvh) * p.T_max * HD;
    const unsigned int n_pass = t1 > t0 ? (t1 - t0 + 31u) / 32u : 0u;
    auto issue = [&](unsigned int pass) {
        if (pass < n_pass)
        {
            const unsigned int t = t0 + pass * 32 + slot;
            const bool valid = t < t1 && !(owner && t == pos);
            const uint16_t* row = Kb + (size_t)(valid ? t : 0) * HD;
#pragma unroll
            for (int c = 0; c < CPL; c++) { cp_async16(ring + ((pass % D) * CPL + c) * kTeam + tid, reinterpret_cast<const uint4*>(row) + sub + 8 * c, valid); }
        }
        cp_async_commit();    // a group per pass, empty past the end, so that the wait below always counts the same
    };
#pragma unroll
    for (int d = 0; d < D; d++) { issue(d); }
    attn_prologue<G, HD>(p, sm, b, kvh, pos, owner, tid);
    float qf[G][CPL][8];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int c = 0; c < CPL; c++)
#pragma unroll
            for (int e = 0; e < 8; e++) { qf[g][c][e] = sm.qs[g * HD + (sub + 8 * c) * 8 + e]; }
    float mx[G];
#pragma unroll
    for (int g = 0; g < G; g++) { mx[g] = -INFINITY; }
    // Two passes per turn of the loop: their dot-product and shuffle chains are independent and interleave.
    for (unsigned int pass = 0; pass < n_pass; pass += 2)
    {
        cp_async_wait<D - 2>();    // the two oldest passes in flight have landed
        float acc[2][G];
#pragma unroll
        for (int u = 0; u < 2; u++)
        {
            const unsigned int t = t0 + (pass + u) * 32 + slot;
#pragma unroll
            for (int g = 0; g < G; g++) { acc[u][g] = 0.f; }
#pragma unroll
            for (int c = 0; c < CPL; c++)
            {
                float kf[8];
                if (owner && t == pos)
                {
                    // the row this call appends: taken from shared memory, not re-read from the cache
#pragma unroll
                    for (int e = 0; e < 8; e++) { kf[e] = sm.kn[(sub + 8 * c) * 8 + e]; }
                }
                else { unpack8(ring[(((pass + u) % D) * CPL + c) * kTeam + tid], kf); }
#pragma unroll
                for (int g = 0; g < G; g++)
#pragma unroll
                    for (int e = 0; e < 8; e++) { acc[u][g] = __fmaf_rn(kf[e], qf[g][c][e], acc[u][g]); }
            }
        }
        issue(pass + D);    // the two slots just read are free again
        issue(pass + D + 1);
        // The 2 G partial sums of the eight lanes of a row are reduce-scattered: each step halves what a lane
        // keeps and adds its partner's half (7 shuffles for 8 values where an all-reduce of each takes 24), so
        // that lane `sub` ends with the finished sum number `sub` (mod the count) and rounds, stores and tracks
        // the maximum of that one score only.
        constexpr int NV = 2 * G;
        float v[NV];
#pragma unroll
        for (int i = 0; i < NV; i++) { v[i] = acc[i / G][i % G]; }
        int idx = 0;    // index of v[0] among the original NV values
        int cnt = NV;   // compile-time after unrolling
#pragma unroll
        for (int step = 4; step >= 1; step >>= 1)
        {
            const bool upper = (sub & (unsigned)step) != 0;
            if (cnt > 1)
            {
                const int half = cnt / 2;
#pragma unroll
                for (int i = 0; i < NV / 2; i++)
                {
                    if (i < half)
                    {
                        const float send = upper ? v[i] : v[half + i];
                        const float recv = __shfl_xor_sync(0xFFFFFFFFu, send, step);
                        v[i] = (upper ? v[half + i] : v[i]) + recv;
                    }
                }
                idx += upper ? half : 0;
                cnt = half;
            }
            else { v[0] += __shfl_xor_sync(0xFFFFFFFFu, v[0], step); }
        }
#pragma unroll
        for (int i = 0; i < NV / 8 + (NV < 8 ? 1 : 0); i++)
        {
            if (i < cnt)
            {
                const int which = idx + i;    // (pass parity, head)
                const int u = which / G, g = which % G;
                const unsigned int t = t0 + (pass + u) * 32 + slot;
                if (t < t1)
                {
                    const float sc = bf16_round(__fmul_rn(p.scale, v[i]));
                    sm.sc[g * ts_cap + (t - t0)] = sc;
#pragma unroll
                    for (int gg = 0; gg < G; gg++)
                    {
                        if (gg == g) { mx[gg] = fmaxf(mx[gg], sc); }
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    team_sync();    // the ring shares its memory with sm.red, which the reductions below write
    attn_scores_finish<G, HD>(sm, t0, t1, ts_cap, tid, mx);
}

// Prologue and scores of the rows [t0, t1) of one kv head against the G rotated queries:
// sm.sc[g][t - t0] = bf16(scale * K[t] . q_g) (the reference's BF16 score tensor, MatrixEx.cpp:3056),
// and this split's maximum and sum of exp(score - maximum) per head in sm.ml.  Eight lanes share a
// row (two 16-byte pieces each for HD = 128), 32 rows per pass, UNROLL passes in flight.  The first
// batch of K rows is requested BEFORE the prologue runs: the cache does not depend on q, so the DRAM
// latency of the first batch and the prologue's own round trip overlap.
template <int G, int HD, int UNROLL = (G <= 4 ? 8 : 4), bool RING = false>
__device__ __forceinline__ void attn_scores(const AttnDecodeParams& p, AttnSmem<G, HD>& sm, unsigned int b, unsigned int kvh,
    unsigned int t0, unsigned int t1, unsigned int ts_cap, unsigned int pos, bool owner, unsigned int tid, uint4* ring = nullptr)
{
    // RING is a compile-time choice: a kernel carries only the form it uses (the stand-alone kernel runs its code
    // once per launch, and what bounds it at one sequence is instruction fetch)
    if constexpr (RING)
    {
        attn_scores_ring<G, HD>(p, sm, b, kvh, t0, t1, ts_cap, pos, owner, tid, ring);
        return;
    }
    else
    {
    constexpr int CPL = HD / 64;    // 16-byte pieces per lane
    const unsigned int sub = tid & 7u, slot = tid >> 3;
    const uint16_t* Kb = p.k_cache + ((size_t)b * p.Hkv + kvh) * p.T_max * HD;
    uint4 kv[UNROLL][CPL];
    auto fetch = [&](unsigned int tb) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
        {
            const unsigned int t = tb + u * 32 + slot;
#pragma unroll
            for (int c = 0; c < CPL; c++)
            {
                kv[u][c] = (t < t1 && !(owner && t == pos)) ? __ldcg(reinterpret_cast<const uint4*>(Kb + (size_t)t * HD) + sub + 8 * c)
                                                            : make_uint4(0, 0, 0, 0);
            }
        }
    };
    fetch(t0);
    attn_prologue<G, HD>(p, sm, b, kvh, pos, owner, tid);
    float qf[G][CPL][8];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int c = 0; c < CPL; c++)
#pragma unroll
            for (int e = 0; e < 8; e++) { qf[g][c][e] = sm.qs[g * HD + (sub + 8 * c) * 8 + e]; }
    float mx[G];
#pragma unroll
    for (int g = 0; g < G; g++) { mx[g] = -INFINITY; }
    for (unsigned int tb = t0; tb < t1; tb += 32 * UNROLL)
    {
        if (tb != t0) { fetch(tb); }
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
        {
            const unsigned int t = tb + u * 32 + slot;
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; g++) { acc[g] = 0.f; }
#pragma unroll
            for (int c = 0; c < CPL; c++)
            {
                float kf[8];
                if (owner && t == pos)
                {
                    // the row this call appends: taken from shared memory, not re-read from the cache
#pragma unroll
                    for (int e = 0; e < 8; e++) { kf[e] = sm.kn[(sub + 8 * c) * 8 + e]; }
                }
                else { unpack8(kv[u][c], kf); }
#pragma unroll
                for (int g = 0; g < G; g++)
#pragma unroll
                    for (int e = 0; e < 8; e++) { acc[g] = __fmaf_rn(kf[e], qf[g][c][e], acc[g]); }
            }
#pragma unroll
            for (int g = 0; g < G; g++)
            {
                acc[g] += __shfl_xor_sync(0xFFFFFFFFu, acc[g], 1);
                acc[g] += __shfl_xor_sync(0xFFFFFFFFu, acc[g], 2);
                acc[g] += __shfl_xor_sync(0xFFFFFFFFu, acc[g], 4);
                if (t < t1)
                {
                    const float s = bf16_round(__fmul_rn(p.scale, acc[g]));
                    if (sub == 0) { sm.sc[g * ts_cap + (t - t0)] = s; }
                    mx[g] = fmaxf(mx[g], s);
                }
            }
        }
    }
    attn_scores_finish<G, HD>(sm, t0, t1, ts_cap, tid, mx);
    }
}

// Probabilities and P*V for the rows [t0, t1): p = bf16(exp(score - max) / sum) with the
// sequence-wide max and 1/sum (the reference's BF16 softmax tensor, MatrixEx.cpp:3091), then
// opart[g][d] = sum_t V[t][d] * p[g][t] in FP32.  HD/8 lanes share a row (16 bytes each).
// `stats` produces the sequence-wide (max, 1/sum) into sm.gl; it runs AFTER the first batch of V
// rows has been requested, because V does not depend on it.
template <int G, int HD, bool RING = false, class Stats>
__device__ __forceinline__ void attn_pv(const AttnDecodeParams& p, AttnSmem<G, HD>& sm, unsigned int b, unsigned int kvh,
    unsigned int t0, unsigned int t1, unsigned int ts_cap, unsigned int pos_row, unsigned int tid, Stats stats, uint4* ring = nullptr)
{
    constexpr int LPR = HD / 8;             // lanes per row
    constexpr int SLOTS = kTeam / LPR;      // rows per pass
    constexpr int UNROLL = 8;
    const unsigned int n = t1 > t0 ? t1 - t0 : 0;
    const unsigned int sub = tid % LPR, slot = tid / LPR;
    const uint16_t* Vb = p.v_cache + ((size_t)b * p.Hkv + kvh) * p.T_max * HD;
    if constexpr (RING)
    {
        // The ring form (see attn_scores_ring): V rows by cp.async, kAttnRingV passes of SLOTS rows in flight, the first
        // ones requested before the statistics are exchanged.
        constexpr int D = kAttnRingV;
        const unsigned int n_pass = (n + SLOTS - 1) / SLOTS;
        auto issue = [&](unsigned int pass) {
            if (pass < n_pass)
            {
                const unsigned int t = t0 + pass * SLOTS + slot;
                const bool valid = t < t1;
                // the row this call appended comes from the projection output, not back from the cache
                const uint16_t* vrow = t == pos_row ? p.v + (size_t)b * p.ldv + (size_t)kvh * HD : Vb + (size_t)(valid ? t : 0) * HD;
                cp_async16(ring + (pass % D) * kTeam + tid, reinterpret_cast<const uint4*>(vrow) + sub, valid);
            }
            cp_async_commit();
        };
#pragma unroll
        for (int d = 0; d < D; d++) { issue(d); }
        stats();
        team_sync();
#pragma unroll
        for (int g = 0; g < G; g++)
        {
            const float m = sm.gl[2 * g], inv = sm.gl[2 * g + 1];
            for (unsigned int i = tid; i < n; i += kTeam)
            {
                sm.sc[g * ts_cap + i] = bf16_round(__fmul_rn(__expf(sm.sc[g * ts_cap + i] - m), inv));
            }
        }
        team_sync();
        float acc[G][8];
#pragma unroll
        for (int g = 0; g < G; g++)
#pragma unroll
            for (int e = 0; e < 8; e++) { acc[g][e] = 0.f; }
        for (unsigned int pass = 0; pass < n_pass; pass += 2)
        {
            cp_async_wait<D - 2>();
#pragma unroll
            for (int u = 0; u < 2; u++)
            {
                const unsigned int t = t0 + (pass + u) * SLOTS + slot;
                if (t < t1)
                {
                    float vf[8];
                    unpack8(ring[((pass + u) % D) * kTeam + tid], vf);
#pragma unroll
                    for (int g = 0; g < G; g++)
                    {
                        const float pr = sm.sc[g * ts_cap + (t - t0)];
#pragma unroll
                        for (int e = 0; e < 8; e++) { acc[g][e] = __fmaf_rn(vf[e], pr, acc[g][e]); }
                    }
                }
            }
            issue(pass + D);
            issue(pass + D + 1);
        }
        cp_async_wait<0>();
        team_sync();    // every thread has read its last ring slot before sm.red (the same memory) is written
#pragma unroll
        for (int g = 0; g < G; g++)
#pragma unroll
            for (int e = 0; e < 8; e++) { sm.red[(slot * G + g) * HD + sub * 8 + e] = acc[g][e]; }
        team_sync();
        for (unsigned int i = tid; i < G * HD; i += kTeam)
        {
            float sacc = 0.f;
            for (int sl = 0; sl < SLOTS; sl++) { sacc += sm.red[sl * G * HD + i]; }
            sm.opart[i] = sacc;
        }
        team_sync();
        return;
    }
    else
    {
    uint4 vv[UNROLL];
    auto fetch = [&](unsigned int tb) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
        {
            const unsigned int t = tb + u * SLOTS + slot;
            // the row this call appended comes from the projection output, not back from the cache
            const uint16_t* vrow = t == pos_row ? p.v + (size_t)b * p.ldv + (size_t)kvh * HD : Vb + (size_t)t * HD;
            vv[u] = t < t1 ? __ldcg(reinterpret_cast<const uint4*>(vrow) + sub) : make_uint4(0, 0, 0, 0);
        }
    };
    fetch(t0);
    stats();
    team_sync();
#pragma unroll
    for (int g = 0; g < G; g++)
    {
        const float m = sm.gl[2 * g], inv = sm.gl[2 * g + 1];
        for (unsigned int i = tid; i < n; i += kTeam)
        {
            sm.sc[g * ts_cap + i] = bf16_round(__fmul_rn(__expf(sm.sc[g * ts_cap + i] - m), inv));
        }
    }
    team_sync();
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int e = 0; e < 8; e++) { acc[g][e] = 0.f; }
    for (unsigned int tb = t0; tb < t1; tb += SLOTS * UNROLL)
    {
        if (tb != t0) { fetch(tb); }
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
        {
            const unsigned int t = tb + u * SLOTS + slot;
            if (t < t1)
            {
                float vf[8];
                unpack8(vv[u], vf);
#pragma unroll
                for (int g = 0; g < G; g++)
                {
                    const float pr = sm.sc[g * ts_cap + (t - t0)];
#pragma unroll
                    for (int e = 0; e < 8; e++) { acc[g][e] = __fmaf_rn(vf[e], pr, acc[g][e]); }
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int e = 0; e < 8; e++) { sm.red[(slot * G + g) * HD + sub * 8 + e] = acc[g][e]; }
    team_sync();
    for (unsigned int i = tid; i < G * HD; i += kTeam)
    {
        float s = 0.f;
        for (int sl = 0; sl < SLOTS; sl++) { s += sm.red[sl * G * HD + i]; }
        sm.opart[i] = s;
    }
    team_sync();
    }
}

}    // namespace b200
