// C-ABI of the fused quantized-weight linear and the library's host bookkeeping.
#include "common.cuh"
#include "gemv_decode.cuh"
#include "gemm_prefill.cuh"
#include "../../include/cccc_cuda_b200.h"

#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>

namespace b200
{

static std::atomic<unsigned long long> g_launches{ 0 };
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

constexpr int kMaxDevices = 64;

// ---- per-device workspace ------------------------------------------------------------------------
// [0, 256)            status word (+ padding)
// [256, 256 + 4 KB)   stream-K arrival counters, zero between launches
// [8 KB, ...)         FP32 partial tiles
struct Workspace
{
    unsigned char* base = nullptr;
    size_t bytes = 0;
    int device = 0;
    int sm_count = 0;
    int max_smem = 0;
    bool tried = false;
    unsigned int* status() const { return reinterpret_cast<unsigned int*>(base); }
    unsigned int* counters() const { return reinterpret_cast<unsigned int*>(base + 256); }
    float* partials() const { return reinterpret_cast<float*>(base + 8192); }
};
constexpr size_t kPartialBytes = 8u << 20;
static Workspace g_ws[kMaxDevices];
static std::mutex g_ws_mutex;

static Workspace* workspace()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { return nullptr; }
    Workspace& w = g_ws[dev];
    if (w.base) { return &w; }
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (w.base) { return &w; }
    if (w.tried) { return nullptr; }
    w.tried = true;
    w.device = dev;
    cudaDeviceGetAttribute(&w.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&w.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const size_t bytes = 8192 + kPartialBytes;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { return nullptr; }
    if (cudaMemset(p, 0, 8192) != cudaSuccess)
    {
        cudaFree(p);
        return nullptr;
    }
    w.bytes = bytes;
    w.base = (unsigned char*)p;
    return &w;
}

int report_launch(const char* label)
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        fprintf(stderr, "%s kernel launch failed: %s\n", label, cudaGetErrorString(e));
        return 1;
    }
    return 0;
}

// Device sync, then the pending CUDA error (the sync's or the last launch's), then this
// library's own status word, in the reference's report format (cuda_functions.cu:26-40).
int sync_and_report(const char* label)
{
    const cudaError_t sync_status = cudaDeviceSynchronize();
    const cudaError_t last_status = cudaGetLastError();
    const cudaError_t report = (sync_status != cudaSuccess) ? sync_status : last_status;
    if (report != cudaSuccess)
    {
        fprintf(stderr, "%s kernel launch failed: %s\n", label, cudaGetErrorString(report));
        return 1;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_ws[dev].base)
    {
        unsigned int st = 0;
        if (cudaMemcpy(&st, g_ws[dev].status(), sizeof(st), cudaMemcpyDeviceToHost) == cudaSuccess && st != 0)
        {
            fprintf(stderr, "%s kernel launch failed: a bounded wait ran out (status %u)\n", label, st);
            // A run that gave up may have left arrival counters behind: start clean again.
            cudaMemset(g_ws[dev].base, 0, 8192);
            return 1;
        }
    }
    return 0;
}

// ---- launch helpers ---------------------------------------------------------------------------------
template <class Kernel>
static cudaError_t launch(Kernel k, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, const GemvParams& p)
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
    return cudaLaunchKernelEx(&cfg, k, p);
}

static bool is_pow2_scale(float s)
{
    if (!(s > 0.f) || std::isinf(s)) { return false; }
    int e = 0;
    const float m = std::frexp(s, &e);
    return m == 0.5f && e >= -39 && e <= 41;    // 2^-40 .. 2^40
}

template <class Cfg, bool SCALED>
static int launch_gemv_cfg(GemvParams p, Workspace* ws, cudaStream_t stream, bool pdl)
{
    const int header = Cfg::HEADER_BYTES + Cfg::RED_BYTES;
    const int stage = Cfg::stage_bytes((int)p.M);
    int ns = (ws->max_smem - header) / stage;
    if (ns > Cfg::kMaxStages) { ns = Cfg::kMaxStages; }
    if (ns < 2) { return -2; }
    p.n_row_blocks = (p.N + Cfg::R - 1) / Cfg::R;
    p.n_kstages = (p.K + Cfg::SKE - 1) / Cfg::SKE;
    const unsigned long long total = (unsigned long long)p.n_row_blocks * p.n_kstages;
    if (total == 0 || total > 0x7FFFFFFFull) { return -2; }
    p.total_items = (unsigned int)total;
    p.n_stages = (unsigned int)ns;
    const unsigned int grid = (unsigned int)(total < (unsigned long long)ws->sm_count ? total : ws->sm_count);
    if ((size_t)grid * 2 * Cfg::R * 8 * Cfg::MT * sizeof(float) > kPartialBytes || grid * sizeof(unsigned int) > 4096) { return -2; }
    const size_t smem = (size_t)header + (size_t)ns * stage;
    auto kernel = gemv_wq_kernel<Cfg, SCALED>;
    static bool attr_set[kMaxDevices] = {};    // per instantiation, per device
    if (!attr_set[ws->device])
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ws->max_smem) != cudaSuccess)
        {
            return report_launch("gemm_wq_bf16") ? 1 : 1;
        }
        attr_set[ws->device] = true;
    }
    if (launch(kernel, dim3(grid), dim3(kGemvThreads), smem, stream, pdl, p) != cudaSuccess)
    {
        report_launch("gemm_wq_bf16");
        return 1;
    }
    return 0;
}

template <int WT, bool SCALED>
static int launch_gemv(const GemvParams& p, Workspace* ws, cudaStream_t stream, bool pdl)
{
    if (p.M <= 2) { return launch_gemv_cfg<GemvCfg<WT, 1, 1, 1, 16>, SCALED>(p, ws, stream, pdl); }
    if (p.M <= 8) { return launch_gemv_cfg<GemvCfg<WT, 1, 2, 1, 8>, SCALED>(p, ws, stream, pdl); }
    if (p.M <= 16) { return launch_gemv_cfg<GemvCfg<WT, 2, 2, 2, 4>, SCALED>(p, ws, stream, pdl); }
    return launch_gemv_cfg<GemvCfg<WT, 4, 2, 4, 4>, SCALED>(p, ws, stream, pdl);
}

template <int WT>
static int launch_plain(const GemvParams& p, cudaStream_t stream)
{
    const unsigned int grid = (p.N + 7) / 8;
    linear_wq_plain_kernel<WT><<<grid, 256, 0, stream>>>(p);
    count_launch();
    return report_launch("gemm_wq_bf16");
}

enum
{
    PLAN_PLAIN = 0,
    PLAN_DECODE = 1,
    PLAN_PREFILL = 2
};

static inline bool al16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

static int plan_for(int w_type, const void* W, const void* blk, const void* X, const void* Y, unsigned int N, unsigned int M,
    unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m, unsigned int ldy_n)
{
    (void)Y;
    (void)ldy_m;
    (void)ldy_n;
    if (N == 0 || M == 0 || K == 0) { return PLAN_PLAIN; }
    if (!al16(W) || !al16(X) || (ldx % 8) != 0) { return PLAN_PLAIN; }
    if (w_type == DT_FP4)
    {
        if (!blk || !al16(blk) || (K % 256) != 0 || (ldw % 256) != 0) { return PLAN_PLAIN; }
    }
    else
    {
        if ((K % 64) != 0 || (ldw % 16) != 0) { return PLAN_PLAIN; }
    }
    if (M <= 32) { return PLAN_DECODE; }
    if (prefill_supported(w_type, N, M, K, ldw, ldx, ldy_m, ldy_n)) { return PLAN_PREFILL; }
    return PLAN_PLAIN;
}

}    // namespace b200

using namespace b200;

C_EXPORT int cuda_gemm_wq_bf16(int w_type, const void* W, const void* blk_scales, float inv_scale, const void* X, void* Y,
    unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m,
    unsigned int ldy_n, float alpha, float beta, void* stream, unsigned int flags)
{
    if (w_type != DT_E4M3 && w_type != DT_E5M2 && w_type != DT_FP4) { return -1; }
    if (N_out == 0 || M_tokens == 0) { return 0; }
    if (!W || !X || !Y) { return -1; }
    Workspace* ws = workspace();
    if (!ws)
    {
        fprintf(stderr, "gemm_wq_bf16 kernel launch failed: no workspace on this device\n");
        return 1;
    }
    cudaStream_t st = (cudaStream_t)stream;
    GemvParams p;
    memset(&p, 0, sizeof(p));
    p.W = (const uint8_t*)W;
    p.blk = (w_type == DT_FP4) ? (const uint8_t*)blk_scales : nullptr;
    p.X = (const uint16_t*)X;
    p.Y = (uint16_t*)Y;
    p.partials = ws->partials();
    p.counters = ws->counters();
    p.status = ws->status();
    p.N = N_out;
    p.M = M_tokens;
    p.K = K;
    p.ldw = ldw;
    p.ldx = ldx;
    p.ldy_m = ldy_m;
    p.ldy_n = ldy_n;
    p.w_scale = inv_scale;
    p.alpha = alpha;
    p.beta = beta;
    p.post_scale = 1.0f;
    const bool pdl = (flags & 1u) != 0;

    int plan = plan_for(w_type, W, blk_scales, X, Y, N_out, M_tokens, K, ldw, ldx, ldy_m, ldy_n);
    if (plan == PLAN_DECODE)
    {
        int r;
        if (w_type == DT_FP4)
        {
            p.post_scale = 65536.0f;    // the FP4 dequantiser leaves 2^-16 in every weight
            r = launch_gemv<DT_FP4, false>(p, ws, st, pdl);
        }
        else if (is_pow2_scale(inv_scale))
        {
            // A power-of-two multiplier commutes exactly with the BF16 rounding and the FP32 sums.
            p.post_scale = inv_scale;
            p.w_scale = 1.0f;
            r = (w_type == DT_E5M2) ? launch_gemv<DT_E5M2, false>(p, ws, st, pdl) : launch_gemv<DT_E4M3, false>(p, ws, st, pdl);
        }
        else { r = (w_type == DT_E5M2) ? launch_gemv<DT_E5M2, true>(p, ws, st, pdl) : launch_gemv<DT_E4M3, true>(p, ws, st, pdl); }
        if (r != -2) { return r; }
        p.post_scale = 1.0f;
        p.w_scale = inv_scale;
        plan = PLAN_PLAIN;
    }
    if (plan == PLAN_PREFILL)
    {
        const int r = launch_prefill(w_type, p, ws->sm_count, ws->max_smem, st);
        if (r != -2) { return r; }
        plan = PLAN_PLAIN;
    }
    if (K == 0)
    {
        // Nothing to sum: Y = beta * Y, which the plain kernel computes with an empty k loop.
    }
    switch (w_type)
    {
    case DT_E4M3: return launch_plain<DT_E4M3>(p, st);
    case DT_E5M2: return launch_plain<DT_E5M2>(p, st);
    default: return launch_plain<DT_FP4>(p, st);
    }
}

C_EXPORT int cuda_gemm_wq_bf16_plan(int w_type, const void* W, const void* blk_scales, const void* X, const void* Y,
    unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m,
    unsigned int ldy_n)
{
    if (w_type != DT_E4M3 && w_type != DT_E5M2 && w_type != DT_FP4) { return -1; }
    return plan_for(w_type, W, blk_scales, X, Y, N_out, M_tokens, K, ldw, ldx, ldy_m, ldy_n);
}

C_EXPORT int cuda_check_error(const char* label) { return sync_and_report(label ? label : "cuda"); }

C_EXPORT void cuda_clear_last_error(void) { cudaGetLastError(); }

C_EXPORT unsigned long long cuda_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

C_EXPORT const char* cuda_b200_version(void) { return "cccc-cuda-b200 0.1 sm_100a"; }
