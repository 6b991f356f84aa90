// Host side of the persistent decode-step kernel: a "program" is recorded once (linears with their
// inputs, attention), finalised (tensor maps, phase list and scratch go to the device; the only place
// that allocates) and then launched as ONE cooperative kernel per step, as often as wanted.
#include "common.cuh"
#include "decode_program.cuh"
#include "tensor_map.cuh"
#include "../../include/cccc_cuda_b200.h"

#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>
#include <vector>

namespace b200
{
void register_reset_hook(void (*fn)(int device));    // api.cu: run when a bounded wait ran out

static bool chain_pow2_scale(float s)
{
    if (!(s > 0.f) || std::isinf(s)) { return false; }
    int e = 0;
    return std::frexp(s, &e) == 0.5f && e >= -39 && e <= 41;
}
}    // namespace b200

using namespace b200;

struct cuda_decode_program
{
    int w_type = 0;
    unsigned int M = 0;
    int device = 0, sm_count = 0, max_smem = 0;
    std::vector<ProgPhase> phases;
    std::vector<CUtensorMap> maps;
    std::vector<float> inv_scales;    // per segment, in phase order (the split into w_scale / post_scale is made at finalise)
    bool any_unscalable = false;      // an FP8 scale that is not a power of two
    bool fma = false;                 // CUDA-core k steps (no per-weight multiplier needed): decided at finalise
    unsigned int max_K = 0;
    unsigned int attn_items = 0, attn_heads = 0;
    size_t attn_smem = 0;
    // device side
    ProgPhase* d_phases = nullptr;
    CUtensorMap* d_maps = nullptr;
    float* d_partials = nullptr;
    unsigned int* d_words = nullptr;    // [0..63] sync, [64..] stream-K counters, then attention counters
    float* d_attn_stats = nullptr;
    float* d_attn_partial = nullptr;
    size_t words = 0;
    ProgHeader hd;
    size_t smem = 0;
    bool finalized = false;
};

namespace
{
std::mutex g_prog_mutex;
std::vector<cuda_decode_program*> g_programs;

// After a bounded wait ran out a launch may have left arrival counters behind: start clean again.
void reset_programs(int device)
{
    std::lock_guard<std::mutex> lock(g_prog_mutex);
    for (cuda_decode_program* p : g_programs)
    {
        if (p->device == device && p->d_words)
        {
            cudaMemset(p->d_words, 0, p->words * sizeof(unsigned int));
            p->hd.epoch = 0;
        }
    }
}

template <int WT, bool SCALED, bool FMA>
int launch_program(cuda_decode_program* p, cudaStream_t stream)
{
    auto kernel = decode_program_kernel<WT, SCALED, 4, FMA>;
    static std::atomic<bool> attr_set[64];
    if (!attr_set[p->device].load(std::memory_order_acquire))
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, p->max_smem) != cudaSuccess)
        {
            report_launch("decode_program");
            return 1;
        }
        attr_set[p->device].store(true, std::memory_order_release);
    }
    void* args[] = { &p->hd };
    count_launch();
    if (cudaLaunchCooperativeKernel((void*)kernel, dim3(p->sm_count), dim3(kChainThreads), args, p->smem, stream) != cudaSuccess)
    {
        report_launch("decode_program");
        return 1;
    }
    p->hd.epoch++;    // the kernel's arrival targets are relative to the launches before it
    return 0;
}
}    // namespace

C_EXPORT int cuda_decode_program_create(cuda_decode_program** out, int w_type, unsigned int M_tokens)
{
    if (!out || (w_type != DT_E4M3 && w_type != DT_E5M2 && w_type != DT_FP4) || M_tokens == 0 || M_tokens > (unsigned)kChainMaxTokens)
    {
        return -1;
    }
    cuda_decode_program* p = new cuda_decode_program();
    p->w_type = w_type;
    p->M = M_tokens;
    if (cudaGetDevice(&p->device) != cudaSuccess || p->device < 0 || p->device >= 64
        || cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, p->device) != cudaSuccess
        || cudaDeviceGetAttribute(&p->max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, p->device) != cudaSuccess)
    {
        delete p;
        return 1;
    }
    *out = p;
    return 0;
}

C_EXPORT int cuda_decode_program_add_linears(cuda_decode_program* p, unsigned int count, const cuda_wq_linear* lin,
    const cuda_decode_input* in, unsigned int K, unsigned int flags)
{
    if (!p || p->finalized || !lin || !in || count == 0 || count > (unsigned)kMaxGroup || K == 0) { return -1; }
    const bool fp4 = p->w_type == DT_FP4;
    if (in->mode < 0 || in->mode > 2 || !in->x || (in->mode == (int)XM_SWIGLU && !in->x2)) { return -1; }
    // what the TMA-fed kernel takes: whole k steps, 16-byte aligned rows
    if ((K % (fp4 ? 256u : 64u)) != 0 || K > 16384u) { return -1; }
    // the team reads its inputs with 16-byte loads
    if (((uintptr_t)in->x & 15u) != 0 || (in->ldx % 8) != 0) { return -1; }
    if (in->mode == (int)XM_SWIGLU && (((uintptr_t)in->x2 & 15u) != 0 || (in->ldx2 % 8) != 0)) { return -1; }
    using Cfg = ChainCfg<DT_E5M2>;
    ProgPhase ph;
    memset(&ph, 0, sizeof(ph));
    ph.kind = PH_LINEAR;
    ph.n_seg = count;
    ph.K = K;
    ph.x_mode = (unsigned)in->mode;
    ph.out_mode = (flags & 4u) ? 1u : ((flags & 8u) ? 2u : 0u);
    ph.paired = (flags & 16u) ? 1u : 0u;
    if (ph.paired
        && (count != 2 || lin[0].N_out != lin[1].N_out || (lin[0].N_out % 16) != 0 || lin[0].beta != 0.f || lin[1].beta != 0.f || ph.out_mode != 0))
    {
        return -1;
    }
    const unsigned int box_rows = ph.paired ? 16u : (unsigned)ChainCfg<DT_E5M2>::R;
    ph.x_src = (const uint16_t*)in->x;
    ph.x_src2 = (const uint16_t*)in->x2;
    ph.norm_w = (const uint16_t*)in->norm_weight;
    ph.ldx = in->ldx;
    ph.ldx2 = in->ldx2;
    ph.eps = in->epsilon;
    ph.map_base = (unsigned)p->maps.size();
    const unsigned int SKS = Cfg::SKS;    // the same for every weight type
    const unsigned long long kbytes = fp4 ? K / 2 : K;
    for (unsigned int j = 0; j < (unsigned)kMaxGroup; j++)
    {
        GemvSeg& g = ph.seg[j];
        if (j >= count)
        {
            g.rb_begin = 0xFFFFFFFFu;
            continue;
        }
        const cuda_wq_linear& L = lin[j];
        if (!L.W || (!L.Y && !(ph.paired && j == 1)) || L.N_out == 0 || ((uintptr_t)L.W & 15u) != 0 || (L.ldw % (fp4 ? 256u : 16u)) != 0)
        {
            return -1;
        }
        if (fp4 && (!L.blk_scales || ((uintptr_t)L.blk_scales & 15u) != 0)) { return -1; }
        g.W = (const uint8_t*)L.W;
        g.blk = fp4 ? (const uint8_t*)L.blk_scales : nullptr;
        g.Y = (uint16_t*)L.Y;
        g.N = L.N_out;
        g.ldw = L.ldw;
        g.ldy_m = L.ldy_m;
        g.ldy_n = L.ldy_n;
        g.alpha = L.alpha;
        g.beta = L.beta;
        if (ph.paired)
        {
            g.rb_begin = j == 0 ? 0u : 0xFFFFFFFFu;    // one list of row blocks: 16 gate rows + the same 16 up rows each
            if (j == 0) { ph.n_row_blocks = L.N_out / 16; }
        }
        else
        {
            g.rb_begin = ph.n_row_blocks;
            ph.n_row_blocks += (L.N_out + Cfg::R - 1) / Cfg::R;
        }
        if (!fp4 && !chain_pow2_scale(L.inv_scale)) { p->any_unscalable = true; }
        CUtensorMap mw, ms;
        const unsigned long long ldw_bytes = fp4 ? L.ldw / 2 : L.ldw;
        if (!make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, L.W, 64, L.N_out, kbytes / 64, ldw_bytes, box_rows, SKS, false)) { return -1; }
        ms = mw;
        if (fp4 && !make_map(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, L.blk_scales, 16, L.N_out, K / 256, L.ldw / 16, box_rows, SKS / 2, false))
        {
            return -1;
        }
        p->maps.push_back(mw);
        p->maps.push_back(ms);
        p->inv_scales.push_back(L.inv_scale);
    }
    const unsigned int ske = (fp4 ? 128u : 64u) * SKS;
    ph.n_kstages = (K + ske - 1) / ske;
    const unsigned long long total = (unsigned long long)ph.n_row_blocks * ph.n_kstages;
    if (total == 0 || total > 0x7FFFFFFFull) { return -1; }
    ph.total_items = (unsigned)total;
    if (K > p->max_K) { p->max_K = K; }
    p->phases.push_back(ph);
    return 0;
}

C_EXPORT int cuda_decode_program_add_attention(cuda_decode_program* p, const cuda_attn_decode* a)
{
    if (!p || p->finalized || !a) { return -1; }
    if (!a->q || !a->k || !a->v || !a->cos_tab || !a->sin_tab || !a->k_cache || !a->v_cache || !a->pos || !a->out) { return -1; }
    if (a->B != p->M || a->Hkv == 0 || a->H != 4 * a->Hkv || a->head_dim != 128 || a->T_max == 0) { return -1; }
    auto misaligned = [](const void* ptr) { return ((uintptr_t)ptr & 15u) != 0; };
    if ((a->ldq % 8) != 0 || (a->ldk % 8) != 0 || (a->ldv % 8) != 0 || misaligned(a->q) || misaligned(a->k) || misaligned(a->v)
        || misaligned(a->k_cache) || misaligned(a->v_cache) || misaligned(a->cos_tab) || misaligned(a->sin_tab)
        || (a->q_norm && misaligned(a->q_norm)) || (a->k_norm && misaligned(a->k_norm)))
    {
        return -1;
    }
    const unsigned int heads = a->B * a->Hkv;
    if (heads > (unsigned)p->sm_count) { return -1; }
    unsigned int S = 1;
    while (S < 16 && heads * S * 2 <= (unsigned)p->sm_count && a->T_max / (S * 2) >= 32) { S *= 2; }
    ProgPhase ph;
    memset(&ph, 0, sizeof(ph));
    AttnDecodeParams& A = ph.attn;
    A.q = (const uint16_t*)a->q;
    A.k = (const uint16_t*)a->k;
    A.v = (const uint16_t*)a->v;
    A.q_norm = (const uint16_t*)a->q_norm;
    A.k_norm = (const uint16_t*)a->k_norm;
    A.cos_tab = (const uint16_t*)a->cos_tab;
    A.sin_tab = (const uint16_t*)a->sin_tab;
    A.k_cache = (uint16_t*)a->k_cache;
    A.v_cache = (uint16_t*)a->v_cache;
    A.pos = (const int*)a->pos;
    A.out = (uint16_t*)a->out;
    A.ldq = a->ldq;
    A.ldk = a->ldk;
    A.ldv = a->ldv;
    A.ldo = a->ldo;
    A.B = a->B;
    A.H = a->H;
    A.Hkv = a->Hkv;
    A.T_max = a->T_max;
    A.eps = a->epsilon;
    A.scale = 1.0f / sqrtf(a->dk > 0.f ? a->dk : (float)a->head_dim);
    ph.attn_S = S;
    ph.attn_ts_cap = (((a->T_max + S - 1) / S) + 31u) & ~31u;
    const size_t smem = attn_smem_floats<4, 128>(ph.attn_ts_cap) * sizeof(float);
    if (smem > p->attn_smem) { p->attn_smem = smem; }
    if (heads * S > p->attn_items) { p->attn_items = heads * S; }
    if (heads > p->attn_heads) { p->attn_heads = heads; }
    ph.kind = PH_ATTN_SCORES;
    p->phases.push_back(ph);
    ph.kind = PH_ATTN_PV;
    p->phases.push_back(ph);
    return 0;
}

C_EXPORT int cuda_decode_program_finalize(cuda_decode_program* p)
{
    if (!p || p->finalized || p->phases.empty()) { return -1; }
    using Cfg = ChainCfg<DT_E5M2>;
    const bool fp4 = p->w_type == DT_FP4;
    const unsigned int grid = (unsigned)p->sm_count;
    const size_t stage = fp4 ? ((ChainCfg<DT_FP4>::W_BYTES + ChainCfg<DT_FP4>::S_BYTES + 1023) / 1024) * 1024 : (size_t)Cfg::W_BYTES;
    const size_t red_bytes = (size_t)Cfg::WK * Cfg::R * 8 * Cfg::MT * sizeof(float);
    const size_t xbuf = (((size_t)kChainMaxTokens * p->max_K * 2) + 1023) / 1024 * 1024;
    size_t u_bytes = xbuf + red_bytes;
    if (p->attn_smem > u_bytes) { u_bytes = p->attn_smem; }
    u_bytes = (u_bytes + 1023) / 1024 * 1024;
    if ((size_t)p->max_smem < Cfg::HEADER_BYTES + u_bytes + 2 * stage) { return -1; }
    size_t ns = ((size_t)p->max_smem - Cfg::HEADER_BYTES - u_bytes) / stage;
    if (ns > (size_t)Cfg::kMaxStages) { ns = Cfg::kMaxStages; }
    p->smem = Cfg::HEADER_BYTES + ns * stage + u_bytes;

    // Weights that need no per-weight multiplier (FP4 block scales; FP8 with power-of-two scales) take the
    // CUDA-core k steps, which outrun the legacy tensor-core path at one or two tokens.
    p->fma = fp4 || !p->any_unscalable;
    // the split of each dequant multiplier into what is applied per weight and what after the sums, and
    // the schedule of each linear phase
    size_t si = 0;
    for (ProgPhase& ph : p->phases)
    {
        if (ph.kind != PH_LINEAR) { continue; }
        for (unsigned int j = 0; j < ph.n_seg; j++, si++)
        {
            const float inv = p->inv_scales[si];
            if (fp4)
            {
                ph.seg[j].w_scale = 1.0f;
                ph.seg[j].post_scale = p->fma ? 1.0f : 65536.0f;    // the tensor-core FP4 dequantiser leaves 2^-16 in every weight
            }
            else if (p->any_unscalable)
            {
                ph.seg[j].w_scale = inv;
                ph.seg[j].post_scale = 1.0f;
            }
            else
            {
                ph.seg[j].w_scale = 1.0f;    // a power of two commutes exactly with the rounding and the sums
                ph.seg[j].post_scale = inv;
            }
        }
        // whole row blocks per CTA unless that leaves most SMs idle for long; then (row block, k stage) items
        // in equal runs with the FP32 fix-up, whose store / fence / atomic / reload chains cost about 4 us of a phase
        const double block_bytes = (double)Cfg::R * (double)(fp4 ? ph.K / 2 + ph.K / 16 : ph.K);
        const double rounds = (double)((ph.n_row_blocks + grid - 1) / grid);
        const double t_whole = rounds * block_bytes / 45e9;
        const double t_split = 4.0e-6 + (double)ph.n_row_blocks * block_bytes / ((double)grid * 42e9);
        ph.gran = (t_whole <= t_split) ? ph.n_kstages : 1u;
    }

    unsigned int* status = cuda_b200_status_word();
    if (!status) { return 1; }
    const size_t tile = (size_t)Cfg::R * 8 * Cfg::MT;
    p->words = 64 + grid + (p->attn_heads ? p->attn_heads : 1);
    bool ok = cudaMalloc((void**)&p->d_phases, p->phases.size() * sizeof(ProgPhase)) == cudaSuccess
        && cudaMalloc((void**)&p->d_maps, (p->maps.empty() ? 1 : p->maps.size()) * sizeof(CUtensorMap)) == cudaSuccess
        && cudaMalloc((void**)&p->d_partials, (size_t)grid * 2 * tile * sizeof(float)) == cudaSuccess
        && cudaMalloc((void**)&p->d_words, p->words * sizeof(unsigned int)) == cudaSuccess
        && cudaMemset(p->d_words, 0, p->words * sizeof(unsigned int)) == cudaSuccess;
    if (ok && p->attn_items)
    {
        ok = cudaMalloc((void**)&p->d_attn_stats, (size_t)p->attn_items * 8 * sizeof(float)) == cudaSuccess
            && cudaMalloc((void**)&p->d_attn_partial, (size_t)p->attn_items * 4 * 128 * sizeof(float)) == cudaSuccess;
    }
    if (ok)
    {
        for (ProgPhase& ph : p->phases)
        {
            if (ph.kind == PH_LINEAR) { continue; }
            ph.attn_stats = p->d_attn_stats;
            ph.attn_partial = p->d_attn_partial;
            ph.attn_counters = p->d_words + 64 + grid;
        }
        ok = cudaMemcpy(p->d_phases, p->phases.data(), p->phases.size() * sizeof(ProgPhase), cudaMemcpyHostToDevice) == cudaSuccess
            && (p->maps.empty() || cudaMemcpy(p->d_maps, p->maps.data(), p->maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) == cudaSuccess);
    }
    if (!ok)
    {
        report_launch("decode_program_finalize");
        return 1;
    }
    ProgHeader& h = p->hd;
    h.phases = p->d_phases;
    h.maps = p->d_maps;
    h.partials = p->d_partials;
    h.counters = p->d_words + 64;
    h.status = status;
    h.sync = p->d_words;
    h.n_phases = (unsigned)p->phases.size();
    h.M = p->M;
    h.n_stages = (unsigned)ns;
    h.epoch = 0;
    h.xbuf_bytes = (unsigned)xbuf;
    p->finalized = true;
    {
        std::lock_guard<std::mutex> lock(g_prog_mutex);
        if (g_programs.empty()) { register_reset_hook(reset_programs); }
        g_programs.push_back(p);
    }
    return 0;
}

C_EXPORT int cuda_decode_program_launch(cuda_decode_program* p, void* stream)
{
    if (!p || !p->finalized) { return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    // no per-weight multiplier (FP4 block scales; power-of-two FP8 scales): CUDA-core k steps; else tensor-core k steps
    if (p->w_type == DT_FP4) { return launch_program<DT_FP4, false, true>(p, st); }
    if (p->w_type == DT_E5M2) { return p->fma ? launch_program<DT_E5M2, false, true>(p, st) : launch_program<DT_E5M2, true, false>(p, st); }
    return p->fma ? launch_program<DT_E4M3, false, true>(p, st) : launch_program<DT_E4M3, true, false>(p, st);
}

C_EXPORT unsigned int cuda_decode_program_phases(const cuda_decode_program* p) { return p ? (unsigned)p->phases.size() : 0u; }

C_EXPORT void cuda_decode_program_destroy(cuda_decode_program* p)
{
    if (!p) { return; }
    {
        std::lock_guard<std::mutex> lock(g_prog_mutex);
        for (size_t i = 0; i < g_programs.size(); i++)
        {
            if (g_programs[i] == p)
            {
                g_programs.erase(g_programs.begin() + i);
                break;
            }
        }
    }
    cudaFree(p->d_phases);
    cudaFree(p->d_maps);
    cudaFree(p->d_partials);
    cudaFree(p->d_words);
    cudaFree(p->d_attn_stats);
    cudaFree(p->d_attn_partial);
    delete p;
}

