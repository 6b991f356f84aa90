// The whole decode step of a cccc LLM in C++, the way cccc-llm drives one token (cccc-llm/cccc-llm.cpp:536-548
// -> MainProcess::testExternalData -> Net::inference -> the ~40 ops per layer that scripts/convert_weights.py:488-584
// generates), as a device-side program: 8 launches per layer (RMSNorm, q+k+v, attention with q/k norm + RoPE +
// cache append inside, o, RMSNorm, gate+up, SwiGLU, down) in one CUDA graph, or, for one or two sequences on one
// GPU, the recorded decode program (one persistent kernel).  Weights come from the converter's container, each
// rank reading only its shard; tensors stored as BF16 / float are quantised on the GPU while loading with the
// reference's rules (Net::quantizeWeights, cccc/Net.cpp:1142-1233; Matrix::quantizeWeights, cccc/Matrix.cpp:301-355).
//
// Tensor parallel without Python: one process, one host thread and one GpuControl per GPU (as the reference runs
// several devices, cccc/GpuControl.cpp:18), peer access between the devices, the exchange areas of
// cuda_gemm_wq_bf16_allreduce allocated by TensorParallel and handed to every rank.
#pragma once

#include "bin_file.h"
#include "cccc_host.h"

#include <condition_variable>
#include <mutex>
#include <string>
#include <vector>

#include "../../../include/cccc_cuda_b200.h"

namespace cccc
{

struct ModelConfig
{
    int hidden = 0, n_heads = 0, n_kv_heads = 0, head_dim = 0, ffn = 0, vocab = 0, layers = 0;
    float rope_theta = 10000.0f, eps = 1e-6f;
    bool qk_norm = false;
    int max_context = 0;
    DataType weight_data_type = CURRENT;    // FP8_E5M2 / FP8_E4M3 / FP4_E2M1: quantise BF16 / float tensors while loading
};

// What the ranks of one process share: exchange areas, a barrier, the combine of the per-rank arg-max.
class TensorParallel
{
public:
    explicit TensorParallel(int world)
        : world_(world), recv_(world, nullptr), flag_(world, nullptr), device_(world, -1), best_(world), id_(world), absmax_(world), last_best_(world)
    {
        ok_.assign(world, 0);
    }
    ~TensorParallel();
    int world() const { return world_; }
    // Called by every rank's thread with its device current: allocates this rank's areas (n_max floats per
    // source and set), enables peer access to the other ranks' devices, and waits for the others.
    bool join(int rank, GpuControl* gpu, unsigned int n_max, std::string* err);
    void barrier();
    bool allOk(int rank, bool ok);    // a barrier that also tells every rank whether all of them passed `true`
    const unsigned long long* recvPtrs() const { return (const unsigned long long*)recv_.data(); }
    const unsigned long long* flagPtrs() const { return (const unsigned long long*)flag_.data(); }
    unsigned int nMax() const { return n_max_; }
    // Every rank passes its shard's winner; all get the largest logit's global id (lowest rank on a tie).
    int combineArgmax(int rank, int global_id, float value);
    float lastBest(int rank) const { return last_best_[rank]; }    // the winning logit of this rank's last combineArgmax
    // Every rank passes its shard's absmax; all get the tensor's (per-tensor FP8 scales are shared by the shards).
    float combineAbsmax(int rank, float value);
    // Every rank passes its BF16 shard of one row of logits (n values); all get the whole row as floats, rank order.
    void gatherLogits(int rank, const uint16_t* shard, int n, float* full);

private:
    int world_;
    std::vector<void*> recv_, flag_;
    std::vector<int> device_;    // the device of each rank that joined, -1 before
    unsigned int n_max_ = 0;
    std::mutex m_;
    std::condition_variable cv_;
    int waiting_ = 0;
    unsigned long long generation_ = 0;
    std::vector<float> best_;
    std::vector<int> id_, ok_;
    std::vector<float> absmax_, last_best_, row_;
    bool failed_ = false;
};

class DecodeStep
{
public:
    DecodeStep() = default;
    ~DecodeStep();
    DecodeStep(const DecodeStep&) = delete;
    DecodeStep& operator=(const DecodeStep&) = delete;

    // Loads this rank's shard of W_q_<i> .. W_down_<i>, W_lm_head (quantised, or BF16 / float + quantise on load),
    // and W_rms_attn_<i>, W_rms_ffn_<i>, W_qnorm_<i>, W_knorm_<i>, W_rms_final, W_emb as BF16 (names of
    // scripts/convert_weights.py:145-166, 200); builds the RoPE tables (cccc/NetCifa.cpp:431-475) and the caches.
    bool load(GpuControl* gpu, const BinFile& file, const ModelConfig& cfg, int max_batch, TensorParallel* tp, int rank, std::string* err);
    // One step for M sequences: token ids and cache rows in, arg-max token ids out (global ids, the same on every
    // rank); logits_host (nullable) receives this rank's shard of the BF16 logits, [M][vocab / world].
    int step(const int* token_ids, const int* positions, int M, int* next_ids, float* best_logits, uint16_t* logits_host);
    void resetCache();
    // One sequence, one GPU: run steps through the recorded decode program (one persistent kernel) when it takes the model.
    bool useProgram(bool on);
    int launchesPerStep() const { return launches_per_step_; }    // of the launch-per-op step
    int lastLaunches() const { return last_launches_; }         // of the step that ran last
    int quantisedOnLoad() const { return quantised_on_load_; }  // tensors that arrived as BF16 / half / float
    size_t cacheBytes() const { return cache_bytes_; }
    // Writes the quantised tensors as a cache file of named weights (weight_<dtype>_<name>, scale_<name>,
    // blockscale_<name>: the keys cccc/Net.cpp:1324-1527 looks up), so that the next start loads them directly.
    // One rank only, after keepHostCopies(true) and load().
    bool saveNamedWeights(const std::string& path, std::string* err) const;
    int vocabLocal() const { return vocab_loc_; }
    size_t weightBytes() const { return weight_bytes_; }
    DataType weightType() const { return wt_; }
    // the quantised shards as loaded (for writing a cache file): name -> (dtype, bytes, scales, quant_scale)
    struct Stored
    {
        std::string name;
        WeightShard shard;
    };
    const std::vector<Stored>& stored() const { return stored_; }
    void keepHostCopies(bool on) { keep_host_ = on; }

private:
    struct Linear
    {
        void* w = nullptr;
        void* s = nullptr;
        float inv = 1.0f;
        int n = 0, k = 0;
    };
    struct Layer
    {
        Linear q, k, v, o, gate, up, down;
        uint16_t *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
        uint16_t *k_cache = nullptr, *v_cache = nullptr;
    };
    bool loadTensors(const BinFile& file, std::string* err);
    bool loadLinear(const BinFile& f, const std::string& name, int N, int K, char kind, Linear* out, std::string* err);
    bool loadBf16(const BinFile& f, const std::string& name, size_t n, uint16_t** out, bool required, std::string* err);
    int issue(int M, cudaStream_t st);
    cuda_attn_decode attnArgs(const Layer& L, int M) const;
    bool buildProgram();
    void* dmalloc(size_t bytes);
    GpuControl* gpu_ = nullptr;
    TensorParallel* tp_ = nullptr;
    ModelConfig cfg_;
    int world_ = 1, rank_ = 0, max_batch_ = 0;
    int H_ = 0, Hkv_ = 0, q_loc_ = 0, kv_loc_ = 0, ffn_loc_ = 0, vocab_loc_ = 0, qkv_ld_ = 0;
    DataType wt_ = FP8_E5M2;
    std::vector<Layer> layers_;
    Linear lm_head_;
    uint16_t *emb_ = nullptr, *final_norm_ = nullptr, *cos_ = nullptr, *sin_ = nullptr;
    uint16_t *x_ = nullptr, *xn_ = nullptr, *tmp_ = nullptr, *qkv_ = nullptr, *att_ = nullptr, *gu_ = nullptr, *h_ = nullptr, *logits_ = nullptr;
    int *d_ids_ = nullptr, *d_pos_ = nullptr, *h_ids_ = nullptr, *h_pos_ = nullptr, *h_out_ = nullptr;
    float *d_best_ = nullptr, *h_best_ = nullptr;
    uint16_t* h_logits_ = nullptr;
    std::vector<Matrix> quantised_;    // tensors quantised while loading own their device memory
    int quantised_on_load_ = 0, layers_loaded_ = 0, last_launches_ = 0;
    size_t cache_bytes_ = 0;
    void* seq_counters_ = nullptr;
    std::vector<void*> owned_;
    std::vector<Stored> stored_;
    std::vector<std::pair<std::string, std::vector<uint16_t>>> plain_;    // norm weights and the embedding, as BF16
    bool keep_host_ = false;
    std::vector<cudaGraphExec_t> graphs_;    // index M
    ::cuda_decode_program* program_ = nullptr;
    bool use_program_ = false;
    size_t weight_bytes_ = 0;
    int launches_per_step_ = 0;
};

}    // namespace cccc
