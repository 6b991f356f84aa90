// The linears of a decode step, driven the way cccc-llm drives a token (cccc-llm/cccc-llm.cpp:536-548
// -> MainProcess::testExternalData -> Net::inference -> one BATCHED_MUL op per projection), but as a
// device-side program: weights are loaded once from the converter's container (only this rank's shard
// of each tensor), q/k/v and gate/up run as grouped launches, the whole token is one CUDA graph, and
// the token is chosen on the device so that 4 bytes per sequence, not V floats, come back.
//
// The non-linear ops of the real step (RMSNorm, RoPE, attention over the KV cache, SwiGLU, residuals)
// run between these linears; they are hooks here (a callback per layer and position that receives the
// stream), with the default of passing the projection output straight on, which is what the linears-
// only benchmark does.
#pragma once

#include "bin_file.h"
#include "cccc_host.h"

#include <functional>
#include <map>
#include <string>
#include <vector>

namespace cccc
{

struct ModelDims
{
    int hidden = 0, q_dim = 0, kv_dim = 0, ffn = 0, vocab = 0, layers = 0;
};

class DecodeLinears
{
public:
    enum Hook
    {
        AFTER_QKV = 0,       // attention goes here: reads q/k/v buffers, writes the o projection's input
        AFTER_O = 1,         // residual + RMSNorm: writes the gate/up input
        AFTER_GATE_UP = 2,   // SwiGLU: writes the down projection's input
        AFTER_DOWN = 3,      // residual (+ next layer's RMSNorm): writes the next layer's input
    };
    using HookFn = std::function<void(int layer, Hook where, cudaStream_t stream)>;
    // Sums a row-parallel shard's FP32 partial sums over the ranks and writes BF16 (tensor parallel).
    using ExchangeFn = std::function<int(const float* partial, uint16_t* out, unsigned int n, cudaStream_t stream)>;

    DecodeLinears() = default;
    ~DecodeLinears();
    DecodeLinears(const DecodeLinears&) = delete;
    DecodeLinears& operator=(const DecodeLinears&) = delete;

    // Reads this rank's shard of W_q_<i>, W_k_<i>, W_v_<i>, W_o_<i>, W_gate_<i>, W_up_<i>, W_down_<i>
    // (i < layers) and W_lm_head (names of scripts/convert_weights.py:145-166, 200) and uploads them.
    bool load(GpuControl* gpu, const BinFile& file, const ModelDims& dims, int max_tokens, int world, int rank, std::string* err);
    void setHook(HookFn f) { hook_ = std::move(f); }
    void setExchange(ExchangeFn f) { exchange_ = std::move(f); }
    // Peer mappings for cuda_gemm_wq_bf16_allreduce (host arrays of `world` device pointers, the local
    // sequence counters, the receive areas' capacity in floats): row-parallel linears then run with the
    // all-reduce inside their kernel, and the exchange function only serves shapes that kernel refuses.
    void setPeerExchange(const unsigned long long* recv_ptrs, const unsigned long long* flag_ptrs, void* seq_counters, unsigned int n_max);
    void setAlpha(float attn, float mlp_in, float mlp_out, float head);    // per-projection output scale (default 1)

    // One step for M sequences: x_host holds M rows of `hidden` BF16 values (the embedded tokens).
    // Returns 0 and fills token_ids (and best_logits if not null) with the arg-max over this rank's
    // vocabulary shard (ids are global: shard offset added).  The first call for a given M records the
    // CUDA graph; later calls replay it.
    int step(const uint16_t* x_host, int M, int* token_ids, float* best_logits);

    size_t weightBytes() const { return weight_bytes_; }
    int launchesPerStep() const { return launches_per_step_; }
    // Buffers the hooks work on (device, BF16, [max_tokens, width]).
    uint16_t* buffer(const std::string& name) const;

private:
    struct Linear
    {
        WeightShard host;
        void* w = nullptr;
        void* s = nullptr;
        char kind = 'c';
    };
    int issue(int M, cudaStream_t st);
    GpuControl* gpu_ = nullptr;
    ModelDims dims_;
    int max_tokens_ = 0, world_ = 1, rank_ = 0;
    std::vector<Linear> lin_;    // 7 per layer, then lm_head
    std::map<std::string, uint16_t*> buf_;
    float* partial_ = nullptr;
    int* d_ids_ = nullptr;
    float* d_vals_ = nullptr;
    uint16_t* h_x_ = nullptr;    // pinned staging
    int* h_ids_ = nullptr;
    float* h_vals_ = nullptr;
    std::map<int, cudaGraphExec_t> graphs_;
    HookFn hook_;
    ExchangeFn exchange_;
    std::vector<unsigned long long> peer_recv_, peer_flag_;
    void* peer_seq_ = nullptr;
    unsigned int peer_n_max_ = 0;
    float alpha_[4] = { 1.f, 1.f, 1.f, 1.f };
    size_t weight_bytes_ = 0;
    int launches_per_step_ = 0;
};

}    // namespace cccc
