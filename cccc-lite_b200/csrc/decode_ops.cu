// C-ABI of the non-GEMM ops of a decode layer: RMSNorm (with the residual add that precedes it),
// RoPE, embedding gather, SwiGLU, and attention of one new token per sequence over a BF16 KV cache
// with the q/k norms, RoPE and the cache append folded into its prologue.
#include "common.cuh"
#include "decode_ops.cuh"
#include "../../include/cccc_cuda_b200.h"

#include <atomic>

namespace cg = cooperative_groups;

namespace b200
{

// ---- RMSNorm ------------------------------------------------------------------------------------
// One CTA per row.  With a residual: s = bf16(x + r) is stored (the reference's add tensor,
// R1 = X + O_out) and normalised.  Shared memory: the row as floats + 256 partial sums.
__global__ void __launch_bounds__(kTeam) rms_norm_bf16_kernel(const uint16_t* __restrict__ X, const uint16_t* __restrict__ R,
    uint16_t* __restrict__ S, uint16_t* __restrict__ Y, const uint16_t* __restrict__ scale, unsigned int inner, float eps)
{
    extern __shared__ __align__(16) float rn_smem[];
    float* xs = rn_smem;
    float* part = rn_smem + inner;
    const unsigned int tid = threadIdx.x;
    const size_t row = (size_t)blockIdx.x * inner;
    pdl_launch_dependents();
    pdl_wait();
    for (unsigned int i = tid; i < inner; i += kTeam)
    {
        float v = bf16_bits_to_float(X[row + i]);
        if (R != nullptr)
        {
            v = bf16_round(__fadd_rn(v, bf16_bits_to_float(R[row + i])));
            if (S != nullptr) { S[row + i] = bf16_bits(v); }
        }
        xs[i] = v;
    }
    team_sync();
    team_sum_squares(xs, part, 1, inner, tid);
    const float invstd = rms_invstd(part[0], inner, eps);
    for (unsigned int i = tid; i < inner; i += kTeam)
    {
        Y[row + i] = bf16_bits(rms_apply(xs[i], invstd, scale ? bf16_bits_to_float(scale[i]) : 1.f));
    }
}

// ---- RoPE (standalone) ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_bf16_kernel(const uint16_t* __restrict__ X, uint16_t* __restrict__ Y,
    const uint16_t* __restrict__ cos_tab, const uint16_t* __restrict__ sin_tab, unsigned int D, unsigned int T, unsigned long long total,
    unsigned int pos_offset)
{
    const unsigned int half = D / 2;
    pdl_launch_dependents();
    pdl_wait();
    for (unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (unsigned long long)gridDim.x * blockDim.x)
    {
        const unsigned int i = (unsigned int)(idx % half);
        const unsigned long long bt = idx / half;
        const unsigned int t = (unsigned int)(bt % T);
        const size_t base = (size_t)bt * D;
        const size_t tab = (size_t)(t + pos_offset) * half + i;
        float yl, yr;
        rope_pair(bf16_bits_to_float(X[base + i]), bf16_bits_to_float(X[base + half + i]), bf16_bits_to_float(cos_tab[tab]),
            bf16_bits_to_float(sin_tab[tab]), yl, yr);
        Y[base + i] = bf16_bits(yl);
        Y[base + half + i] = bf16_bits(yr);
    }
}

// ---- embedding gather ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_bf16_kernel(const int* __restrict__ ids, const uint16_t* __restrict__ W,
    uint16_t* __restrict__ Y, unsigned int D, unsigned int vocab)
{
    pdl_launch_dependents();
    pdl_wait();
    const int id = ids[blockIdx.x];
    const bool ok = id >= 0 && (unsigned int)id < vocab;
    const uint16_t* src = W + (size_t)(ok ? id : 0) * D;
    uint16_t* dst = Y + (size_t)blockIdx.x * D;
    if ((D % 8) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0)
    {
        for (unsigned int i = threadIdx.x; i < D / 8; i += blockDim.x)
        {
            reinterpret_cast<uint4*>(dst)[i] = ok ? reinterpret_cast<const uint4*>(src)[i] : make_uint4(0, 0, 0, 0);
        }
    }
    else
    {
        for (unsigned int i = threadIdx.x; i < D; i += blockDim.x) { dst[i] = ok ? src[i] : (uint16_t)0; }
    }
}

// ---- SwiGLU ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_bf16_kernel(const uint16_t* __restrict__ G, const uint16_t* __restrict__ U,
    uint16_t* __restrict__ O, unsigned int cols, unsigned int ldg, unsigned int ldu, unsigned int ldo)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.y;
    for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < cols; i += gridDim.x * blockDim.x)
    {
        O[row * ldo + i] = bf16_bits(swiglu_one(bf16_bits_to_float(G[row * ldg + i]), bf16_bits_to_float(U[row * ldu + i])));
    }
}

// ---- attention ---------------------------------------------------------------------------------------
// Grid (S, Hkv, B), clusters of S CTAs along x: the S splits of one (sequence, kv head) exchange
// their softmax statistics and partial outputs through distributed shared memory.
template <int G, int HD>
__global__ void __launch_bounds__(kTeam, (G <= 4 ? 2 : 1)) attn_decode_kernel(const AttnDecodeParams p, unsigned int ts_cap)
{
    extern __shared__ __align__(16) float at_smem[];
    cg::cluster_group cluster = cg::this_cluster();
    AttnSmem<G, HD> sm(at_smem, ts_cap);
    uint4* ring = reinterpret_cast<uint4*>(sm.red);    // the reduction buffer is idle while the K and V passes run
    const unsigned int tid = threadIdx.x;
    const unsigned int S = gridDim.x, rank = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();
    const int pos_i = p.pos[b];
    const unsigned int pos = pos_i < 0 ? 0u : (unsigned int)pos_i;
    const unsigned int T = min(pos + 1u, p.T_max);
    unsigned int ts = (T + S - 1) / S;
    ts = (ts + 31u) & ~31u;
    const unsigned int t0 = min(rank * ts, T), t1 = min(t0 + ts, T);
    const bool owner = pos >= t0 && pos < t1;
    attn_scores<G, HD, 4, true>(p, sm, b, kvh, t0, t1, ts_cap, pos, owner, tid, ring);    // (runs the prologue too)
    cluster.sync();
    attn_pv<G, HD, true>(p, sm, b, kvh, t0, t1, ts_cap, owner ? pos : 0xFFFFFFFFu, tid, [&]() {
        // One thread per (head, split) fetches that split's (max, sum) over distributed shared memory in a single
        // round trip; the S lanes of a head then pass their pairs to the head's first lane, which combines them in
        // split order (the order a serial loop over the splits would use, so the bits do not depend on S's layout).
        const unsigned int lanes = G * S;    // <= 128: G <= 8, S <= 16
        if (tid < ((lanes + 31u) & ~31u))
        {
            const unsigned int g = tid / S, r = tid % S;
            float m = -INFINITY, l = 0.f;
            if (tid < lanes)
            {
                const float* ml = cluster.map_shared_rank(sm.ml, r);
                m = ml[2 * g];
                l = ml[2 * g + 1];
            }
            float gmax = -INFINITY, L = 0.f;
            const unsigned int lane = tid & 31u, first = lane - r;    // S divides 32, so a head's lanes share a warp
            for (unsigned int j = 0; j < S; j++) { gmax = fmaxf(gmax, __shfl_sync(0xFFFFFFFFu, m, first + j)); }
            for (unsigned int j = 0; j < S; j++)
            {
                const float mj = __shfl_sync(0xFFFFFFFFu, m, first + j), lj = __shfl_sync(0xFFFFFFFFu, l, first + j);
                if (lj > 0.f) { L += lj * __expf(mj - gmax); }
            }
            if (tid < lanes && r == 0)
            {
                sm.gl[2 * g] = gmax;
                sm.gl[2 * g + 1] = 1.0f / L;
            }
        }
    }, ring);
    cluster.sync();
    if (rank == 0)
    {
        uint16_t* o = p.out + (size_t)b * p.ldo + (size_t)kvh * G * HD;
        for (unsigned int i = tid; i < G * HD; i += kTeam)
        {
            float s = 0.f;
            for (unsigned int r = 0; r < S; r++) { s += cluster.map_shared_rank(sm.opart, r)[i]; }
            o[i] = bf16_bits(s);
        }
    }
    cluster.sync();    // the other splits keep their shared memory alive until split 0 has read it
}

static unsigned int attn_ts_cap(unsigned int T_max, unsigned int S) { return (((T_max + S - 1) / S) + 31u) & ~31u; }

template <int G, int HD>
static int launch_attn(const AttnDecodeParams& p, int sm_count, int max_smem, cudaStream_t stream, bool pdl)
{
    auto kernel = attn_decode_kernel<G, HD>;
    // Splits per (sequence, kv head): a power of two <= 16 with at least 64 rows per split.  Two CTAs share an SM, and an
    // SM streams fastest with both (36 against 24 GB/s), so the splits grow while the CTAs still fit two per SM
    // (measured at 4096 rows: 4 / 8 / 16 sequences 35 -> 25, 59 -> 38, 107 -> 65 us with 256 CTAs instead of 128);
    // between one and 1.3 CTAs per SM one more doubling of a small cluster still gains (12 / 24 sequences: 95 -> 63,
    // 120 -> 107 us), but clusters of 16 only pay while 8 would leave half the SMs empty (2 sequences: 24 us with
    // 8 splits, 32 with 16).
    const unsigned long long units = (unsigned long long)p.B * p.Hkv;
    unsigned int S = 1;
    while (S < 8 && units * S * 2 <= 2ull * (unsigned long long)sm_count && p.T_max / (S * 2) >= 64) { S *= 2; }
    if (S == 8 && units * S * 2 <= (unsigned long long)sm_count + 20 && p.T_max / (S * 2) >= 64) { S = 16; }
    if (S <= 2 && units * S * 10 <= 13ull * (unsigned long long)sm_count && p.T_max / (S * 2) >= 64) { S *= 2; }
    auto smem_bytes = [](unsigned int ts_cap) { return attn_smem_floats<G, HD>(ts_cap) * sizeof(float); };
    while (S < 16 && smem_bytes(attn_ts_cap(p.T_max, S)) > (size_t)max_smem) { S *= 2; }
    static std::atomic<int> max_cluster{ 0 };    // largest cluster size this kernel can be scheduled with (0 = not probed)
    for (;;)
    {
        const unsigned int ts_cap = attn_ts_cap(p.T_max, S);
        const size_t smem = smem_bytes(ts_cap);
        if (smem > (size_t)max_smem) { return -1; }
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess
            || (S > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess))
        {
            cudaGetLastError();
            if (S > 8)
            {
                S = 8;
                continue;
            }
            return report_launch("attn_decode_bf16") ? 1 : 1;
        }
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(S, p.Hkv, p.B);
        cfg.blockDim = dim3(kTeam);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = S;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 2 : 1;
        if (S > 8 && max_cluster.load(std::memory_order_relaxed) == 0)
        {
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1)
            {
                cudaGetLastError();
                max_cluster.store(8, std::memory_order_relaxed);
            }
            else { max_cluster.store(16, std::memory_order_relaxed); }
        }
        if (S > 8 && max_cluster.load(std::memory_order_relaxed) == 8)
        {
            S = 8;
            continue;
        }
        count_launch();
        if (cudaLaunchKernelEx(&cfg, kernel, p, ts_cap) != cudaSuccess) { return report_launch("attn_decode_bf16") ? 1 : 1; }
        return 0;
    }
}

struct DeviceFacts
{
    std::atomic<int> ready{ 0 };
    int sm_count = 0, max_smem = 0;
};
static DeviceFacts g_facts[64];
static const DeviceFacts* device_facts()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { return nullptr; }
    DeviceFacts& f = g_facts[dev];
    if (f.ready.load(std::memory_order_acquire) == 0)
    {
        int a = 0, b = 0;
        if (cudaDeviceGetAttribute(&a, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess
            || cudaDeviceGetAttribute(&b, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
        {
            return nullptr;
        }
        f.sm_count = a;    // two threads may both write the same values: harmless
        f.max_smem = b;
        f.ready.store(1, std::memory_order_release);
    }
    return &f;
}

template <class K, class... Args>
static int launch_simple(const char* label, K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, Args... args)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, kernel, args...) != cudaSuccess)
    {
        report_launch(label);
        return 1;
    }
    return 0;
}

}    // namespace b200

using namespace b200;

C_EXPORT int cuda_rms_norm_bf16(const void* X, const void* residual, void* sum_out, void* Y, const void* scale, unsigned int rows,
    unsigned int inner, float epsilon, void* stream, unsigned int flags)
{
    if (rows == 0 || inner == 0) { return 0; }
    if (!X || !Y) { return -1; }
    const size_t smem = ((size_t)inner + kTeam) * sizeof(float);
    const DeviceFacts* f = device_facts();
    if (!f) { return 1; }
    if (smem > (size_t)f->max_smem) { return -1; }
    if (smem > 48 * 1024 && cudaFuncSetAttribute(rms_norm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    {
        return report_launch("rms_norm_bf16") ? 1 : 1;
    }
    return launch_simple("rms_norm_bf16", rms_norm_bf16_kernel, dim3(rows), dim3(kTeam), smem, (cudaStream_t)stream, (flags & 1u) != 0,
        (const uint16_t*)X, (const uint16_t*)residual, (uint16_t*)sum_out, (uint16_t*)Y, (const uint16_t*)scale, inner, epsilon);
}

C_EXPORT int cuda_rope_bf16(const void* X, void* Y, const void* cos_tab, const void* sin_tab, unsigned int D, unsigned int T,
    unsigned int B, unsigned int pos_offset, void* stream, unsigned int flags)
{
    const unsigned long long total = (unsigned long long)(D / 2) * T * B;
    if (total == 0) { return 0; }
    if (!X || !Y || !cos_tab || !sin_tab || (D & 1u)) { return -1; }
    const unsigned int grid = (unsigned int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    return launch_simple("rope_bf16", rope_bf16_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (flags & 1u) != 0, (const uint16_t*)X,
        (uint16_t*)Y, (const uint16_t*)cos_tab, (const uint16_t*)sin_tab, D, T, total, pos_offset);
}

C_EXPORT int cuda_embed_bf16(const void* ids, const void* W, void* Y, unsigned int D, unsigned int n_tokens, unsigned int vocab,
    void* stream, unsigned int flags)
{
    if (n_tokens == 0 || D == 0) { return 0; }
    if (!ids || !W || !Y) { return -1; }
    return launch_simple("embed_bf16", embed_bf16_kernel, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, (flags & 1u) != 0, (const int*)ids,
        (const uint16_t*)W, (uint16_t*)Y, D, vocab);
}

C_EXPORT int cuda_swiglu_bf16(const void* gate, const void* up, void* out, unsigned int rows, unsigned int cols, unsigned int ld_gate,
    unsigned int ld_up, unsigned int ld_out, void* stream, unsigned int flags)
{
    if (rows == 0 || cols == 0) { return 0; }
    if (!gate || !up || !out || rows > 65535u) { return -1; }
    const unsigned int gx = (cols + 255) / 256 < 64 ? (cols + 255) / 256 : 64;
    return launch_simple("swiglu_bf16", swiglu_bf16_kernel, dim3(gx, rows), dim3(256), 0, (cudaStream_t)stream, (flags & 1u) != 0,
        (const uint16_t*)gate, (const uint16_t*)up, (uint16_t*)out, cols, ld_gate, ld_up, ld_out);
}

C_EXPORT int cuda_attn_decode_bf16(const cuda_attn_decode* a, void* stream, unsigned int flags)
{
    if (!a) { return -1; }
    if (a->B == 0 || a->H == 0) { return 0; }
    if (!a->q || !a->k || !a->v || !a->cos_tab || !a->sin_tab || !a->k_cache || !a->v_cache || !a->pos || !a->out) { return -1; }
    if (a->Hkv == 0 || (a->H % a->Hkv) != 0 || a->T_max == 0 || a->B > 65535u || a->Hkv > 65535u) { return -1; }
    auto misaligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) != 0; };
    if ((a->ldq % 8) != 0 || (a->ldk % 8) != 0 || (a->ldv % 8) != 0 || misaligned(a->q) || misaligned(a->k) || misaligned(a->v)
        || misaligned(a->k_cache) || misaligned(a->v_cache) || misaligned(a->cos_tab) || misaligned(a->sin_tab)
        || (a->q_norm && misaligned(a->q_norm)) || (a->k_norm && misaligned(a->k_norm)))
    {
        return -1;
    }
    const DeviceFacts* f = device_facts();
    if (!f) { return 1; }
    AttnDecodeParams p;
    p.q = (const uint16_t*)a->q;
    p.k = (const uint16_t*)a->k;
    p.v = (const uint16_t*)a->v;
    p.q_norm = (const uint16_t*)a->q_norm;
    p.k_norm = (const uint16_t*)a->k_norm;
    p.cos_tab = (const uint16_t*)a->cos_tab;
    p.sin_tab = (const uint16_t*)a->sin_tab;
    p.k_cache = (uint16_t*)a->k_cache;
    p.v_cache = (uint16_t*)a->v_cache;
    p.pos = (const int*)a->pos;
    p.out = (uint16_t*)a->out;
    p.ldq = a->ldq;
    p.ldk = a->ldk;
    p.ldv = a->ldv;
    p.ldo = a->ldo;
    p.B = a->B;
    p.H = a->H;
    p.Hkv = a->Hkv;
    p.T_max = a->T_max;
    p.eps = a->epsilon;
    p.scale = 1.0f / sqrtf(a->dk > 0.f ? a->dk : (float)a->head_dim);
    const unsigned int G = a->H / a->Hkv;
    const bool pdl = (flags & 1u) != 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->head_dim == 128)
    {
        switch (G)
        {
        case 1: return launch_attn<1, 128>(p, f->sm_count, f->max_smem, st, pdl);
        case 2: return launch_attn<2, 128>(p, f->sm_count, f->max_smem, st, pdl);
        case 4: return launch_attn<4, 128>(p, f->sm_count, f->max_smem, st, pdl);
        case 8: return launch_attn<8, 128>(p, f->sm_count, f->max_smem, st, pdl);
        default: return -1;
        }
    }
    if (a->head_dim == 64)
    {
        switch (G)
        {
        case 1: return launch_attn<1, 64>(p, f->sm_count, f->max_smem, st, pdl);
        case 2: return launch_attn<2, 64>(p, f->sm_count, f->max_smem, st, pdl);
        case 4: return launch_attn<4, 64>(p, f->sm_count, f->max_smem, st, pdl);
        case 8: return launch_attn<8, 64>(p, f->sm_count, f->max_smem, st, pdl);
        default: return -1;
        }
    }
    return -1;
}
