// C-ABI of the fused quantized-weight linear and the library's host bookkeeping.
#include "common.cuh"
#include "gemv_launch.cuh"
#include "gemm_w8a8.cuh"
#include "../../include/cccc_cuda_b200.h"

#include <atomic>
#include <mutex>
#include <vector>

namespace b200
{

static std::atomic<unsigned long long> g_launches{ 0 };
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---- per-device workspace ------------------------------------------------------------------------
// [0, 256)            status word (+ padding)
// [256, 256 + 4 KB)   stream-K arrival counters, zero between launches
// [8 KB, ...)         FP32 partial tiles; the native kernels' activation pieces; the W8A8 mode's quantised activations
//                     (tokens x K bytes: 64 MB hold 4096 tokens of K = 16384)
struct Workspace
{
    std::atomic<unsigned char*> base{ nullptr };    // published last (release) once `scratch` is complete
    size_t bytes = 0;
    bool tried = false;
    GemvScratch scratch;
    unsigned int* status() const { return reinterpret_cast<unsigned int*>(base.load(std::memory_order_acquire)); }
};
constexpr size_t kPartialBytes = 64u << 20;
static Workspace g_ws[kMaxDevices];
static std::mutex g_ws_mutex;

static Workspace* workspace()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { return nullptr; }
    Workspace& w = g_ws[dev];
    if (w.base.load(std::memory_order_acquire)) { return &w; }
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    if (w.base.load(std::memory_order_relaxed)) { return &w; }
    if (w.tried) { return nullptr; }
    w.tried = true;
    w.scratch.device = dev;
    cudaDeviceGetAttribute(&w.scratch.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&w.scratch.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&w.scratch.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    const size_t bytes = 8192 + kPartialBytes;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { return nullptr; }
    if (cudaMemset(p, 0, 8192) != cudaSuccess)
    {
        cudaFree(p);
        return nullptr;
    }
    w.bytes = bytes;
    w.scratch.status = reinterpret_cast<unsigned int*>(p);
    w.scratch.counters = reinterpret_cast<unsigned int*>((unsigned char*)p + 256);
    w.scratch.n_counters = 1024;
    w.scratch.partials = reinterpret_cast<float*>((unsigned char*)p + 8192);
    w.scratch.partial_bytes = kPartialBytes;
    w.base.store((unsigned char*)p, std::memory_order_release);
    return &w;
}

unsigned int* cuda_b200_status_word()
{
    Workspace* ws = workspace();
    return ws ? ws->scratch.status : nullptr;
}

// Functions to run when one of the library's bounded waits ran out (they put device-side counters of
// longer-lived objects back to zero).
static std::mutex g_hook_mutex;
static std::vector<void (*)(int)> g_reset_hooks;
void register_reset_hook(void (*fn)(int device))
{
    std::lock_guard<std::mutex> lock(g_hook_mutex);
    g_reset_hooks.push_back(fn);
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
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_ws[dev].base.load(std::memory_order_acquire))
    {
        unsigned int st = 0;
        if (cudaMemcpy(&st, g_ws[dev].status(), sizeof(st), cudaMemcpyDeviceToHost) == cudaSuccess && st != 0)
        {
            fprintf(stderr, "%s kernel launch failed: a bounded wait ran out (status %u)\n", label, st);
            // A run that gave up may have left arrival counters behind: start clean again.
            cudaMemset(g_ws[dev].base.load(std::memory_order_acquire), 0, 8192);
            std::vector<void (*)(int)> hooks;
            {
                std::lock_guard<std::mutex> lock(g_hook_mutex);
                hooks = g_reset_hooks;
            }
            for (auto fn : hooks) { fn(dev); }
            return 1;
        }
    }
    return 0;
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
    return run_linear_wq(&ws->scratch, w_type, W, blk_scales, inv_scale, X, Y, N_out, M_tokens, K, ldw, ldx, ldy_m, ldy_n, alpha,
        beta, (cudaStream_t)stream, flags);
}

C_EXPORT int cuda_gemm_w8a8_bf16(const void* W, float w_inv_scale, const void* X, float act_scale, void* Y, unsigned int N_out,
    unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m, unsigned int ldy_n, float alpha, float beta,
    void* stream, unsigned int flags)
{
    if (N_out == 0 || M_tokens == 0) { return 0; }
    if (!W || !X || !Y) { return -1; }
    Workspace* ws = workspace();
    if (!ws)
    {
        fprintf(stderr, "gemm_w8a8_bf16 kernel launch failed: no workspace on this device\n");
        return 1;
    }
    const W8A8Member m = { W, Y, w_inv_scale, alpha, beta, N_out, ldw, ldy_m, ldy_n };
    return launch_w8a8(&ws->scratch, &m, 1, X, act_scale, M_tokens, K, ldx, (cudaStream_t)stream, flags, false, false, (flags >> 8) & 3u);
}

C_EXPORT int cuda_gemm_w8a8_bf16_group(unsigned int count, const cuda_wq_linear* linears, const void* X, float act_scale, unsigned int M_tokens,
    unsigned int K, unsigned int ldx, void* stream, unsigned int flags)
{
    if (count == 0 || M_tokens == 0) { return 0; }
    if (!linears || !X || count > (unsigned int)PF_MAX_GROUP) { return -1; }
    Workspace* ws = workspace();
    if (!ws)
    {
        fprintf(stderr, "gemm_w8a8_bf16 kernel launch failed: no workspace on this device\n");
        return 1;
    }
    W8A8Member m[PF_MAX_GROUP];
    for (unsigned int j = 0; j < count; j++)
    {
        if (linears[j].N_out == 0) { return -1; }
        m[j] = { linears[j].W, linears[j].Y, linears[j].inv_scale, linears[j].alpha, linears[j].beta, linears[j].N_out, linears[j].ldw,
            linears[j].ldy_m, linears[j].ldy_n };
    }
    return launch_w8a8(&ws->scratch, m, count, X, act_scale, M_tokens, K, ldx, (cudaStream_t)stream, flags, false, false, (flags >> 8) & 3u);
}

C_EXPORT int cuda_gemm_fp8_fp8(const void* W, float w_inv_scale, const void* X_fp8, float x_inv_scale, void* Y, int y_type, unsigned int N_out,
    unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m, unsigned int ldy_n, float alpha, float beta,
    void* stream, unsigned int flags)
{
    if (y_type != DT_BF16 && y_type != DT_E4M3) { return -1; }
    if (N_out == 0 || M_tokens == 0) { return 0; }
    if (!W || !X_fp8 || !Y) { return -1; }
    Workspace* ws = workspace();
    if (!ws)
    {
        fprintf(stderr, "gemm_fp8_fp8 kernel launch failed: no workspace on this device\n");
        return 1;
    }
    const W8A8Member m = { W, Y, w_inv_scale, alpha, beta, N_out, ldw, ldy_m, ldy_n };
    return launch_w8a8(&ws->scratch, &m, 1, X_fp8, x_inv_scale, M_tokens, K, ldx, (cudaStream_t)stream, flags & 1u, true, y_type == DT_E4M3, (flags >> 8) & 3u);
}

C_EXPORT int cuda_bf16_to_fp8e4m3_dynamic(const void* src, void* dst_fp8, unsigned int n, void* d_absmax_tmp, void* d_inv_scale_out)
{
    if (n == 0) { return 0; }
    if (!src || !dst_fp8 || !d_absmax_tmp || !d_inv_scale_out) { return -1; }
    if (cudaMemsetAsync(d_absmax_tmp, 0, sizeof(float), 0) != cudaSuccess) { return report_launch("bf162fp8e4m3_dynamic") ? 1 : 0; }
    unsigned int gx = (n + 255u) / 256u;
    count_launch();
    absmax_bf16_rows_kernel<<<dim3(gx > 1024u ? 1024u : gx, 1), 256>>>((const uint16_t*)src, n, n, 1, (float*)d_absmax_tmp);
    count_launch();
    quantise_activations_kernel<<<dim3(gx, 1), 256>>>((const uint16_t*)src, n, n, 1, (uint8_t*)dst_fp8, n, (const float*)d_absmax_tmp, 0.f, 0.f,
        (float*)d_inv_scale_out, 1, false, false);
    return report_launch("bf162fp8e4m3_dynamic");
}

C_EXPORT int cuda_gemm_wq_bf16_group(int w_type, unsigned int count, const cuda_wq_linear* linears, const void* X,
    unsigned int M_tokens, unsigned int K, unsigned int ldx, void* stream, unsigned int flags)
{
    if (w_type != DT_E4M3 && w_type != DT_E5M2 && w_type != DT_FP4) { return -1; }
    if (count == 0 || M_tokens == 0) { return 0; }
    if (!linears || !X) { return -1; }
    for (unsigned int j = 0; j < count; j++)
    {
        if (linears[j].N_out != 0 && (!linears[j].W || !linears[j].Y)) { return -1; }
    }
    Workspace* ws = workspace();
    if (!ws)
    {
        fprintf(stderr, "gemm_wq_bf16 kernel launch failed: no workspace on this device\n");
        return 1;
    }
    static_assert(sizeof(GroupItem) == sizeof(cuda_wq_linear), "GroupItem mirrors cuda_wq_linear");
    return run_linear_wq_group(&ws->scratch, w_type, count, reinterpret_cast<const GroupItem*>(linears), X, M_tokens, K, ldx,
        (cudaStream_t)stream, flags);
}

C_EXPORT int cuda_gemm_wq_bf16_allreduce(int w_type, const void* W, const void* blk_scales, float inv_scale, const void* X, void* Y,
    unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m,
    unsigned int ldy_n, float alpha, const unsigned long long* peer_recv_ptrs, const unsigned long long* peer_flag_ptrs,
    void* seq_counters, unsigned int n_max, int rank, int world, void* stream, unsigned int flags)
{
    if (w_type != DT_E4M3 && w_type != DT_E5M2 && w_type != DT_FP4) { return -1; }
    if (!W || !X || !Y || N_out == 0 || M_tokens == 0 || K == 0) { return -1; }
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) { return -1; }
    if (world > 1 && (!peer_recv_ptrs || !peer_flag_ptrs || !seq_counters)) { return -1; }
    Workspace* ws = workspace();
    if (!ws)
    {
        fprintf(stderr, "gemm_wq_bf16 kernel launch failed: no workspace on this device\n");
        return 1;
    }
    GemvAllReduce ar;
    memset(&ar, 0, sizeof(ar));
    for (int r = 0; r < world && world > 1; r++)
    {
        ar.peer_recv[r] = reinterpret_cast<float*>(peer_recv_ptrs[r]);
        ar.peer_flag[r] = reinterpret_cast<unsigned int*>(peer_flag_ptrs[r]);
    }
    ar.seq = reinterpret_cast<unsigned int*>(seq_counters);
    ar.n_max = n_max;
    ar.rank = rank;
    ar.world = world;
    return run_linear_wq(&ws->scratch, w_type, W, blk_scales, inv_scale, X, Y, N_out, M_tokens, K, ldw, ldx, ldy_m, ldy_n, alpha, 0.f,
        (cudaStream_t)stream, flags, false, &ar);
}

C_EXPORT unsigned long long cuda_b200_fused_flag_bytes(int world)
{
    return world < 1 ? 0ull : 2ull * kArMaxRowBlocks * (unsigned long long)world * sizeof(unsigned int);
}

C_EXPORT unsigned long long cuda_b200_fused_counter_bytes(void) { return (unsigned long long)kArMaxRowBlocks * sizeof(unsigned int); }

C_EXPORT int cuda_gemm_wq_bf16_plan(int w_type, const void* W, const void* blk_scales, const void* X, const void* Y,
    unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m,
    unsigned int ldy_n)
{
    if (w_type != DT_E4M3 && w_type != DT_E5M2 && w_type != DT_FP4) { return -1; }
    const int plan = plan_for(w_type, W, blk_scales, X, Y, N_out, M_tokens, K, ldw, ldx, ldy_m, ldy_n);
    int sm_count = 148, dev = 0;    // without a device (the query reads no memory and runs on CPU-only hosts too): a B200's
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    {
        cudaGetLastError();
        sm_count = 148;
    }
    if (plan != PLAN_PLAIN && native_by_default(w_type, M_tokens, (unsigned long long)N_out * K, (N_out + NK_BM - 1) / NK_BM, sm_count) && al16(W)
        && (w_type == DT_FP4 ? native_fp4_supported(blk_scales, N_out, M_tokens, K, ldw, ldx) : native_supported(w_type, N_out, M_tokens, K, ldw, ldx)))
    {
        return PLAN_NATIVE;    // (an FP8 scale that is no power of two still goes to the kernels that dequantise)
    }
    return plan;
}

C_EXPORT int cuda_check_error(const char* label) { return sync_and_report(label ? label : "cuda"); }

C_EXPORT void cuda_clear_last_error(void) { cudaGetLastError(); }

C_EXPORT unsigned long long cuda_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

C_EXPORT const char* cuda_b200_version(void) { return "cccc-cuda-b200 0.1 sm_100a"; }
