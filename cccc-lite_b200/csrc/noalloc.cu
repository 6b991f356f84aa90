// cuda_gemm_wq_bf16_static: the decode-side linear for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc when a linear is issued: code under a
// caller-owned memory pool or a fixed memory budget where every byte of device memory is planned
// (or already committed) up front, and latency-critical loops that may not take the allocator's
// locks or the device-wide synchronisation an allocation or a free can imply.  The regular entry point allocates its per-device workspace on first use; this
// one never allocates.  The scratch the split-k schedule needs (FP32 partial tiles, arrival
// counters, a status word) lives in a file-scope device array of fixed size instead, so every GPU
// that loads the library carries those 520 KB until the process exits.
#include "common.cuh"
#include "gemv_launch.cuh"
#include "../../include/cccc_cuda_b200.h"

#include <atomic>
#include <mutex>

namespace
{

using namespace b200;

constexpr unsigned int kStaticMaxTokens = 8;      // the kernels for M <= 8 keep 32 x 8 FP32 per partial tile
constexpr unsigned int kStaticMaxCtas = 256;      // one CTA per SM
constexpr size_t kStaticHeaderBytes = 8192;       // status word at 0, counters at 256
constexpr size_t kStaticTileBytes = 32 * 8 * sizeof(float);
constexpr size_t kStaticPartialBytes = (size_t)kStaticMaxCtas * 2 * kStaticTileBytes;
constexpr size_t kStaticScratchBytes = kStaticHeaderBytes + kStaticPartialBytes;    // 532 480

// In host code this name is only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress below.  Zero-initialised when the module is loaded.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticState
{
    std::atomic<bool> ready{ false };    // set last (release) once base and scratch are complete
    unsigned char* base = nullptr;
    GemvScratch scratch;
};
StaticState g_static[kMaxDevices];
std::mutex g_static_mutex;

// Once per device, with that device current: resolve the array's device address and read the
// device facts the launch logic needs.  Nothing here allocates.
StaticState* static_state()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { return nullptr; }
    StaticState& st = g_static[dev];
    if (st.ready.load(std::memory_order_acquire)) { return &st; }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (st.ready.load(std::memory_order_relaxed)) { return &st; }
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
    {
        fprintf(stderr, "gemm_wq_bf16_static kernel launch failed: cudaGetSymbolAddress: %s\n", cudaGetErrorString(e));
        return nullptr;
    }
    st.base = (unsigned char*)ptr;
    st.scratch.status = reinterpret_cast<unsigned int*>(st.base);
    st.scratch.counters = reinterpret_cast<unsigned int*>(st.base + 256);
    st.scratch.n_counters = kStaticMaxCtas;
    st.scratch.partials = reinterpret_cast<float*>(st.base + kStaticHeaderBytes);
    st.scratch.partial_bytes = kStaticPartialBytes;
    st.scratch.device = dev;
    if (cudaDeviceGetAttribute(&st.scratch.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess
        || cudaDeviceGetAttribute(&st.scratch.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess
        || cudaDeviceGetAttribute(&st.scratch.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess)
    {
        fprintf(stderr, "gemm_wq_bf16_static kernel launch failed: cannot read the device attributes\n");
        return nullptr;
    }
    st.ready.store(true, std::memory_order_release);
    return &st;
}

}    // namespace

C_EXPORT int cuda_gemm_wq_bf16_static(int w_type, const void* W, const void* blk_scales, float inv_scale, const void* X, void* Y,
    unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m,
    unsigned int ldy_n, float alpha, float beta, void* stream, unsigned int flags)
{
    if (w_type != DT_E4M3 && w_type != DT_E5M2 && w_type != DT_FP4) { return -1; }
    if (N_out == 0 || M_tokens == 0) { return 0; }
    if (!W || !X || !Y) { return -1; }
    if (M_tokens > kStaticMaxTokens)
    {
        fprintf(stderr, "gemm_wq_bf16_static: %u tokens exceed the fixed scratch (at most %u tokens); use cuda_gemm_wq_bf16\n",
            M_tokens, kStaticMaxTokens);
        return -1;
    }
    StaticState* st = static_state();
    if (!st) { return 1; }
    if ((unsigned int)st->scratch.sm_count > kStaticMaxCtas)
    {
        fprintf(stderr, "gemm_wq_bf16_static: %d SMs exceed the fixed scratch (at most %u)\n", st->scratch.sm_count, kStaticMaxCtas);
        return -1;
    }
    cudaStream_t s = (cudaStream_t)stream;
    // The array keeps whatever the last call left in it.  Partial tiles are always written before
    // they are read; the arrival counters must start at zero and the status word must describe this
    // call only, so both are cleared on the stream (status word at 0, counters at 256).  A failure of
    // an earlier unchecked call is therefore dropped here, never reported against a later call.
    if (cudaMemsetAsync(st->base, 0, 256 + kStaticMaxCtas * sizeof(unsigned int), s) != cudaSuccess)
    {
        report_launch("gemm_wq_bf16_static");
        return 1;
    }
    const int r = run_linear_wq(&st->scratch, w_type, W, blk_scales, inv_scale, X, Y, N_out, M_tokens, K, ldw, ldx, ldy_m, ldy_n,
        alpha, beta, s, flags & 1u, /*decode_only=*/true);
    if (r == -1)
    {
        fprintf(stderr,
            "gemm_wq_bf16_static: this shape or alignment needs a kernel the fixed scratch does not serve (16-byte aligned "
            "operands, K %% 64 == 0; FP4: block scales, K %% 256 == 0, ldw %% 256 == 0); use cuda_gemm_wq_bf16\n");
        return -1;
    }
    if (r != 0) { return r; }
    if (flags & 2u)
    {
        // Checked mode: wait for the stream and look at the status word (a stack variable, no allocation).
        if (cudaStreamSynchronize(s) != cudaSuccess)
        {
            report_launch("gemm_wq_bf16_static");
            return 1;
        }
        unsigned int status = 0;
        if (cudaMemcpy(&status, st->scratch.status, sizeof(status), cudaMemcpyDeviceToHost) != cudaSuccess) { return 1; }
        if (status != 0)
        {
            fprintf(stderr, "gemm_wq_bf16_static kernel launch failed: a bounded wait ran out (status %u)\n", status);
            return 1;    // the next call clears the header again before it runs
        }
    }
    return 0;
}
