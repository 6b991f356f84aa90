// One-shot all-reduce of the FP32 partial sums of a row-parallel (K-split) linear over NVLink peer
// memory, with the BF16 rounding fused in: out = bf16( sum over ranks of partial ).
//
// Every rank owns a receive area that all its peers have mapped (symmetric memory):
//     recv  [2 sets][world source ranks][n_max floats]
//     flags [2 sets][kArCtas][world source ranks] (32-bit sequence numbers)
// A call on rank r: each CTA c copies its chunk of the local partial into slot [set][r] of EVERY
// rank's receive area with plain peer stores, fences, and publishes the call's sequence number in
// flags[set][c][r] of every rank.  It then waits (bounded) until all `world` flags of its own area
// show that sequence number, adds the world slots in rank order (so every rank computes the same
// bits) and writes BF16.  Sequence numbers are per-CTA device counters, so a CUDA graph can be
// replayed; consecutive calls alternate between the two sets, which is enough because a rank only
// finishes call k+1 after every peer has finished call k.
// Messages here are 8 KB .. 512 KB, so latency, not bandwidth, is what matters: one hop, no
// library call, no separate cast kernel.  No multicast loads, no remote reads.
#include "common.cuh"
#include "gemv_decode.cuh"
#include "../../include/cccc_cuda_b200.h"

namespace b200
{

constexpr int kArCtas = 8;
constexpr int kArThreads = 256;

struct ArParams
{
    float* peer_recv[kArMaxWorld];
    unsigned int* peer_flag[kArMaxWorld];
    const float* partial;
    uint16_t* out;
    unsigned int* seq_counters;    // local, [kArCtas]
    unsigned int* status;
    unsigned int n, n_max;
    int rank, world;
};

__global__ void __launch_bounds__(kArThreads) allreduce_push_kernel(const ArParams p)
{
    __shared__ unsigned int sh_seq, sh_ok;
    pdl_launch_dependents();
    pdl_wait();    // the partial sums come from the previous kernel of the stream
    const unsigned int cta = blockIdx.x;
    if (threadIdx.x == 0)
    {
        sh_seq = p.seq_counters[cta] + 1;
        p.seq_counters[cta] = sh_seq;
        sh_ok = 1;
    }
    __syncthreads();
    const unsigned int seq = sh_seq;
    const unsigned int set = seq & 1u;
    // this CTA's chunk, in float4 units
    const unsigned int n4 = p.n / 4;
    const unsigned int per = (n4 + kArCtas - 1) / kArCtas;
    const unsigned int b4 = min(cta * per, n4), e4 = min(b4 + per, n4);
    const size_t slot = ((size_t)set * p.world + p.rank) * p.n_max;

    // ---- push my chunk into my slot of every rank (own rank included) ----
    const float4* src = reinterpret_cast<const float4*>(p.partial);
    for (unsigned int i = b4 + threadIdx.x; i < e4; i += kArThreads)
    {
        const float4 v = src[i];
        for (int r = 0; r < p.world; r++) { reinterpret_cast<float4*>(p.peer_recv[r] + slot)[i] = v; }
    }
    // The barrier orders every thread's peer stores before the flag stores of threads 0..world-1, whose
    // release at system scope is cumulative over them; a system fence per storing thread cost 4 us.
    __syncthreads();
    if ((int)threadIdx.x < p.world)
    {
        st_release_sys(p.peer_flag[threadIdx.x] + ((size_t)set * kArCtas + cta) * p.world + p.rank, seq);
    }
    // ---- wait for every source rank's chunk to be here ----
    if ((int)threadIdx.x < p.world)
    {
        const unsigned int* f = p.peer_flag[p.rank] + ((size_t)set * kArCtas + cta) * p.world + threadIdx.x;
        const unsigned long long t0 = global_timer_ns();
        unsigned int spins = 0;
        while (ld_acquire_sys(f) != seq)
        {
            if ((++spins & 0xFFu) == 0 && global_timer_ns() - t0 > 1000000000ull)
            {
                atomicMax(p.status, 4u);    // a peer never arrived: report and carry on without hanging
                sh_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (!sh_ok) { return; }
    // ---- add the slots in rank order, round once ----
    const float* mine = p.peer_recv[p.rank] + (size_t)set * p.world * p.n_max;
    for (unsigned int i = b4 + threadIdx.x; i < e4; i += kArThreads)
    {
        float4 acc = __ldcv(reinterpret_cast<const float4*>(mine) + i);    // peers wrote these: never from L1
        for (int r = 1; r < p.world; r++)
        {
            const float4 v = __ldcv(reinterpret_cast<const float4*>(mine + (size_t)r * p.n_max) + i);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        uint2 o;
        o.x = pack_bf16x2(acc.x, acc.y);
        o.y = pack_bf16x2(acc.z, acc.w);
        reinterpret_cast<uint2*>(p.out)[i] = o;
    }
}

}    // namespace b200

using namespace b200;

C_EXPORT int cuda_b200_allreduce_f32_to_bf16(const unsigned long long* peer_recv_ptrs, const unsigned long long* peer_flag_ptrs,
    void* seq_counters, const void* partial, void* out_bf16, unsigned int n, unsigned int n_max, int rank, int world, void* stream,
    unsigned int flags)
{
    if (!peer_recv_ptrs || !peer_flag_ptrs || !seq_counters || !partial || !out_bf16) { return -1; }
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world || n == 0 || n > n_max || (n % 4) != 0 || (n_max % 4) != 0)
    {
        return -1;
    }
    ArParams p;
    for (int r = 0; r < kArMaxWorld; r++)
    {
        p.peer_recv[r] = r < world ? reinterpret_cast<float*>(peer_recv_ptrs[r]) : nullptr;
        p.peer_flag[r] = r < world ? reinterpret_cast<unsigned int*>(peer_flag_ptrs[r]) : nullptr;
    }
    p.partial = (const float*)partial;
    p.out = (uint16_t*)out_bf16;
    p.seq_counters = (unsigned int*)seq_counters;
    p.status = cuda_b200_status_word();
    if (!p.status) { return 1; }
    p.n = n;
    p.n_max = n_max;
    p.rank = rank;
    p.world = world;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kArCtas);
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & 1u) ? 1 : 0;
    count_launch();
    if (cudaLaunchKernelEx(&cfg, allreduce_push_kernel, p) != cudaSuccess)
    {
        report_launch("allreduce_f32_to_bf16");
        return 1;
    }
    return 0;
}

C_EXPORT unsigned long long cuda_b200_allreduce_recv_bytes(int world, unsigned int n_max)
{
    return 2ull * (unsigned long long)world * n_max * sizeof(float);
}
C_EXPORT unsigned long long cuda_b200_allreduce_flag_bytes(int world) { return 2ull * kArCtas * (unsigned long long)world * sizeof(unsigned int); }
C_EXPORT unsigned long long cuda_b200_allreduce_counter_bytes(void) { return kArCtas * sizeof(unsigned int); }
