#include "decode_linears.h"

#include "../../../include/cccc_cuda_b200.h"

#include <cstdio>
#include <cstring>

namespace cccc
{

DecodeLinears::~DecodeLinears()
{
    if (!gpu_) { return; }
    gpu_->setAsCurrent();
    gpu_->synchronize();
    for (auto& g : graphs_) { cudaGraphExecDestroy(g.second); }
    for (auto& l : lin_)
    {
        if (l.w) { gpu_->free(l.w); }
        if (l.s) { gpu_->free(l.s); }
    }
    for (auto& b : buf_) { gpu_->free(b.second); }
    if (partial_) { gpu_->free(partial_); }
    if (d_ids_) { gpu_->free(d_ids_); }
    if (d_vals_) { gpu_->free(d_vals_); }
    if (h_x_) { cudaFreeHost(h_x_); }
    if (h_ids_) { cudaFreeHost(h_ids_); }
    if (h_vals_) { cudaFreeHost(h_vals_); }
}

void DecodeLinears::setAlpha(float attn, float mlp_in, float mlp_out, float head)
{
    alpha_[0] = attn;
    alpha_[1] = mlp_in;
    alpha_[2] = mlp_out;
    alpha_[3] = head;
}

void DecodeLinears::setPeerExchange(const unsigned long long* recv_ptrs, const unsigned long long* flag_ptrs, void* seq_counters,
    unsigned int n_max)
{
    peer_recv_.assign(recv_ptrs, recv_ptrs + world_);
    peer_flag_.assign(flag_ptrs, flag_ptrs + world_);
    peer_seq_ = seq_counters;
    peer_n_max_ = n_max;
}

uint16_t* DecodeLinears::buffer(const std::string& name) const
{
    auto it = buf_.find(name);
    return it == buf_.end() ? nullptr : it->second;
}

bool DecodeLinears::load(GpuControl* gpu, const BinFile& file, const ModelDims& d, int max_tokens, int world, int rank,
    std::string* err)
{
    gpu_ = gpu;
    dims_ = d;
    max_tokens_ = max_tokens;
    world_ = world;
    rank_ = rank;
    gpu_->setAsCurrent();
    struct Spec
    {
        const char* name;
        int N, K;
        char kind;
    };
    const Spec per_layer[7] = { { "W_q", d.q_dim, d.hidden, 'c' }, { "W_k", d.kv_dim, d.hidden, 'c' }, { "W_v", d.kv_dim, d.hidden, 'c' },
        { "W_o", d.hidden, d.q_dim, 'r' }, { "W_gate", d.ffn, d.hidden, 'c' }, { "W_up", d.ffn, d.hidden, 'c' },
        { "W_down", d.hidden, d.ffn, 'r' } };
    auto add = [&](const std::string& name, int N, int K, char kind) {
        Linear l;
        l.kind = kind;
        if (!loadWeightShard(file, name, N, K, kind, world, rank, &l.host, err)) { return false; }
        auto fail = [&](const std::string& what) {
            if (err) { *err = what + " for '" + name + "'"; }
            return false;
        };
        l.w = gpu_->malloc(l.host.weights.size());
        if (!l.w) { return fail("no device memory"); }
        if (cudaMemcpy(l.w, l.host.weights.data(), l.host.weights.size(), cudaMemcpyHostToDevice) != cudaSuccess) { return fail("upload failed"); }
        weight_bytes_ += l.host.weights.size();
        if (!l.host.block_scales.empty())
        {
            l.s = gpu_->malloc(l.host.block_scales.size());
            if (!l.s) { return fail("no device memory for the block scales"); }
            if (cudaMemcpy(l.s, l.host.block_scales.data(), l.host.block_scales.size(), cudaMemcpyHostToDevice) != cudaSuccess)
            {
                return fail("upload of the block scales failed");
            }
            weight_bytes_ += l.host.block_scales.size();
        }
        l.host.weights.clear();
        l.host.weights.shrink_to_fit();
        l.host.block_scales.clear();
        lin_.push_back(std::move(l));
        return true;
    };
    for (int i = 0; i < d.layers; i++)
    {
        for (auto& s : per_layer)
        {
            if (!add(std::string(s.name) + "_" + std::to_string(i), s.N, s.K, s.kind)) { return false; }
        }
    }
    if (!add("W_lm_head", d.vocab, d.hidden, 'c')) { return false; }
    bool buffers_ok = true;
    auto mk = [&](const char* name, int width) {
        void* p = gpu_->malloc((size_t)max_tokens * width * 2);
        if (!p || cudaMemset(p, 0, (size_t)max_tokens * width * 2) != cudaSuccess) { buffers_ok = false; }
        buf_[name] = (uint16_t*)p;
    };
    mk("x", d.hidden);
    mk("q", d.q_dim / world);
    mk("k", d.kv_dim / world);
    mk("v", d.kv_dim / world);
    mk("o", d.hidden);
    mk("gate", d.ffn / world);
    mk("up", d.ffn / world);
    mk("logits", d.vocab / world);
    partial_ = (float*)gpu_->malloc((size_t)max_tokens * d.hidden * 4);
    d_ids_ = (int*)gpu_->malloc((size_t)max_tokens * 4);
    d_vals_ = (float*)gpu_->malloc((size_t)max_tokens * 4);
    const bool pinned_ok = cudaMallocHost((void**)&h_x_, (size_t)max_tokens * d.hidden * 2) == cudaSuccess
        && cudaMallocHost((void**)&h_ids_, (size_t)max_tokens * 4) == cudaSuccess
        && cudaMallocHost((void**)&h_vals_, (size_t)max_tokens * 4) == cudaSuccess;
    if (!(buffers_ok && pinned_ok && partial_ && d_ids_ && d_vals_))
    {
        if (err) { *err = "no memory for the step's buffers"; }
        return false;
    }
    return true;
}

int DecodeLinears::issue(int M, cudaStream_t st)
{
    const unsigned flags = 1;    // programmatic dependent launch along the chain
    int launches = 0;
    auto item = [&](const Linear& l, void* y, float alpha) {
        cuda_wq_linear g;
        g.W = l.w;
        g.blk_scales = l.s;
        g.Y = y;
        g.inv_scale = l.host.quant_scale;
        g.alpha = alpha;
        g.beta = 0.f;
        g.N_out = (unsigned)l.host.n;
        g.ldw = (unsigned)l.host.k;
        g.ldy_m = (unsigned)l.host.n;
        g.ldy_n = 1;
        return g;
    };
    auto row_parallel = [&](const Linear& l, const uint16_t* in, uint16_t* out, float alpha) {
        if (world_ == 1)
        {
            launches++;
            return cuda_gemm_wq_bf16((int)l.host.dtype, l.w, l.s, l.host.quant_scale, in, out, (unsigned)l.host.n, (unsigned)M,
                (unsigned)l.host.k, (unsigned)l.host.k, (unsigned)l.host.k, (unsigned)l.host.n, 1, alpha, 0.f, st, flags);
        }
        if (peer_seq_ != nullptr)
        {
            const int r = cuda_gemm_wq_bf16_allreduce((int)l.host.dtype, l.w, l.s, l.host.quant_scale, in, out, (unsigned)l.host.n,
                (unsigned)M, (unsigned)l.host.k, (unsigned)l.host.k, (unsigned)l.host.k, (unsigned)l.host.n, 1, alpha, peer_recv_.data(),
                peer_flag_.data(), peer_seq_, peer_n_max_, rank_, world_, st, flags);
            if (r != -1)
            {
                launches++;
                return r;
            }
        }
        if (!exchange_) { return -1; }
        launches += 2;
        const int r = cuda_gemm_wq_bf16((int)l.host.dtype, l.w, l.s, l.host.quant_scale, in, partial_, (unsigned)l.host.n, (unsigned)M,
            (unsigned)l.host.k, (unsigned)l.host.k, (unsigned)l.host.k, (unsigned)l.host.n, 1, alpha, 0.f, st, flags | 4u);
        return r != 0 ? r : exchange_(partial_, out, (unsigned)(M * l.host.n), st);
    };
    uint16_t* x = buf_["x"];
    for (int i = 0; i < dims_.layers; i++)
    {
        const Linear* L = &lin_[(size_t)i * 7];
        const int wt = (int)L[0].host.dtype;
        cuda_wq_linear qkv[3] = { item(L[0], buf_["q"], alpha_[0]), item(L[1], buf_["k"], alpha_[0]), item(L[2], buf_["v"], alpha_[0]) };
        if (cuda_gemm_wq_bf16_group(wt, 3, qkv, x, (unsigned)M, (unsigned)dims_.hidden, (unsigned)dims_.hidden, st, flags) != 0) { return -1; }
        launches++;
        if (hook_) { hook_(i, AFTER_QKV, st); }
        if (row_parallel(L[3], buf_["q"], buf_["o"], alpha_[0]) != 0) { return -1; }
        if (hook_) { hook_(i, AFTER_O, st); }
        cuda_wq_linear gu[2] = { item(L[4], buf_["gate"], alpha_[1]), item(L[5], buf_["up"], alpha_[1]) };
        if (cuda_gemm_wq_bf16_group(wt, 2, gu, buf_["o"], (unsigned)M, (unsigned)dims_.hidden, (unsigned)dims_.hidden, st, flags) != 0)
        {
            return -1;
        }
        launches++;
        if (hook_) { hook_(i, AFTER_GATE_UP, st); }
        if (row_parallel(L[6], buf_["gate"], x, alpha_[2]) != 0) { return -1; }
        if (hook_) { hook_(i, AFTER_DOWN, st); }
    }
    const Linear& H = lin_.back();
    if (cuda_gemm_wq_bf16((int)H.host.dtype, H.w, H.s, H.host.quant_scale, x, buf_["logits"], (unsigned)H.host.n, (unsigned)M,
            (unsigned)H.host.k, (unsigned)H.host.k, (unsigned)H.host.k, (unsigned)H.host.n, 1, alpha_[3], 0.f, st, flags)
        != 0)
    {
        return -1;
    }
    if (cuda_argmax_bf16(buf_["logits"], (unsigned)M, (unsigned)H.host.n, (unsigned long long)H.host.n, d_ids_, d_vals_, st) != 0) { return -1; }
    launches += 2;
    launches_per_step_ = launches;
    return 0;
}

int DecodeLinears::step(const uint16_t* x_host, int M, int* token_ids, float* best_logits)
{
    if (!gpu_ || M < 1 || M > max_tokens_) { return -1; }
    gpu_->setAsCurrent();
    cudaStream_t st = gpu_->stream();
    std::memcpy(h_x_, x_host, (size_t)M * dims_.hidden * 2);
    auto it = graphs_.find(M);
    if (it == graphs_.end())
    {
        // One eager pass first: it allocates the library's workspace and sets kernel attributes, which
        // must not happen inside a capture.  Then record.
        cudaMemcpyAsync(buf_["x"], h_x_, (size_t)M * dims_.hidden * 2, cudaMemcpyHostToDevice, st);
        if (issue(M, st) != 0 || cudaStreamSynchronize(st) != cudaSuccess) { return -1; }
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { return -1; }
        cudaMemcpyAsync(buf_["x"], h_x_, (size_t)M * dims_.hidden * 2, cudaMemcpyHostToDevice, st);
        const int r = issue(M, st);
        cudaMemcpyAsync(h_ids_, d_ids_, (size_t)M * 4, cudaMemcpyDeviceToHost, st);
        cudaMemcpyAsync(h_vals_, d_vals_, (size_t)M * 4, cudaMemcpyDeviceToHost, st);
        if (cudaStreamEndCapture(st, &graph) != cudaSuccess || r != 0 || !graph) { return -1; }
        cudaGraphExec_t exec = nullptr;
        if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess)
        {
            cudaGraphDestroy(graph);
            return -1;
        }
        cudaGraphDestroy(graph);
        it = graphs_.emplace(M, exec).first;
    }
    if (cudaGraphLaunch(it->second, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) { return -1; }
    const int off = rank_ * (dims_.vocab / world_);
    for (int m = 0; m < M; m++)
    {
        token_ids[m] = h_ids_[m] < 0 ? -1 : h_ids_[m] + off;
        if (best_logits) { best_logits[m] = h_vals_[m]; }
    }
    return 0;
}

}    // namespace cccc
