// A small C harness over the C++ host layer so that the tests (ctypes) can drive Matrix::mul /
// mulBatched / quantizeWeights and Cublas::gemm exactly as cccc code would.
#include "cccc_host.h"

#include <vector>

using namespace cccc;

#define HOST_EXPORT extern "C" __attribute__((visibility("default")))

HOST_EXPORT void* cccc_host_gpu_create(int device)
{
    auto* g = new GpuControl();
    if (g->init(device) != 0)
    {
        delete g;
        return nullptr;
    }
    return g;
}
HOST_EXPORT void cccc_host_gpu_destroy(void* g) { delete (GpuControl*)g; }
HOST_EXPORT void cccc_host_gpu_sync(void* g) { ((GpuControl*)g)->synchronize(); }
HOST_EXPORT int cccc_host_fused_calls(void* g) { return ((GpuControl*)g)->cublas_->fusedCalls(); }
HOST_EXPORT int cccc_host_fallback_calls(void* g) { return ((GpuControl*)g)->cublas_->fallbackCalls(); }
// W8A16 (BFLOAT16) or W8A8 (FP8_E4M3) for the quantised linears that follow: Cublas::setActDataType
HOST_EXPORT void cccc_host_set_act_type(void* g, int dt) { ((GpuControl*)g)->cublas_->setActDataType((DataType)dt); }

// Views over caller-owned device memory; dims are cccc's (width, height, channel, number).
HOST_EXPORT void* cccc_host_matrix_view(void* g, void* data, int w, int h, int c, int n, int dt, float quant_scale, void* blk)
{
    auto* m = new Matrix(Matrix::view(data, w, h, c, n, (DataType)dt, (GpuControl*)g));
    m->setQuantScale(quant_scale);
    m->setBlockScaleData(blk);
    return m;
}
HOST_EXPORT void* cccc_host_matrix_new(void* g, int w, int h, int c, int n, int dt) { return new Matrix(w, h, c, n, (DataType)dt, (GpuControl*)g); }
HOST_EXPORT void cccc_host_matrix_free(void* m) { delete (Matrix*)m; }
HOST_EXPORT void* cccc_host_matrix_data(void* m) { return ((Matrix*)m)->data(); }
HOST_EXPORT void* cccc_host_matrix_block_scale(void* m) { return ((Matrix*)m)->getBlockScaleData(); }
HOST_EXPORT float cccc_host_matrix_quant_scale(void* m) { return ((Matrix*)m)->getQuantScale(); }
HOST_EXPORT int cccc_host_matrix_dtype(void* m) { return (int)((Matrix*)m)->getDataType(); }
HOST_EXPORT void cccc_host_matrix_quantize(void* m, int target) { ((Matrix*)m)->quantizeWeights((DataType)target); }

HOST_EXPORT void cccc_host_mul(void* A, void* B, void* R, float a, float r, int ta, int tb)
{
    Matrix::mul(*(Matrix*)A, *(Matrix*)B, *(Matrix*)R, a, r, (MatrixTransType)ta, (MatrixTransType)tb);
}
HOST_EXPORT void cccc_host_mul_batched(void* A, void* B, void* R, int ta, int tb, float a, float r)
{
    Matrix::mulBatched(*(Matrix*)A, *(Matrix*)B, *(Matrix*)R, (MatrixTransType)ta, (MatrixTransType)tb, a, r);
}
HOST_EXPORT void cccc_host_gemm(void* g, int ta, int tb, int M, int N, int K, float alpha, const void* A, int typeA, int lda,
    float invA, const void* B, int typeB, int ldb, float invB, float beta, void* C, int typeC, int ldc, const void* blkA,
    const void* blkB)
{
    ((GpuControl*)g)->setAsCurrent();
    ((GpuControl*)g)->cublas_->gemm((MatrixTransType)ta, (MatrixTransType)tb, M, N, K, alpha, A, (DataType)typeA, lda, invA, B,
        (DataType)typeB, ldb, invB, beta, C, (DataType)typeC, ldc, 0.0f, (const uint8_t*)blkA, (const uint8_t*)blkB);
}

// ---- weight container ---------------------------------------------------------------------------------
#include "bin_file.h"

#include <cstring>
#include <string>

HOST_EXPORT void* cccc_host_bin_open(const char* path)
{
    auto* f = new BinFile();
    if (!f->open(path))
    {
        delete f;
        return nullptr;
    }
    return f;
}
HOST_EXPORT void cccc_host_bin_close(void* f) { delete (BinFile*)f; }
HOST_EXPORT int cccc_host_bin_has(void* f, const char* key) { return ((BinFile*)f)->has(key) ? 1 : 0; }
HOST_EXPORT unsigned long long cccc_host_bin_bytes_read(void* f) { return ((BinFile*)f)->bytesRead(); }
// Loads one rank's shard into caller buffers (sizes from the shard shape); returns 0, or -1 with a
// message in err (at most err_len bytes).  dims[0..2] = dtype, n, k.
HOST_EXPORT int cccc_host_bin_load_shard(void* f, const char* name, int N, int K, char kind, int world, int rank, void* weights,
    unsigned long long weights_cap, void* scales, unsigned long long scales_cap, float* quant_scale, int* dims, char* err,
    int err_len)
{
    WeightShard s;
    std::string e;
    if (!loadWeightShard(*(BinFile*)f, name, N, K, kind, world, rank, &s, &e) || s.weights.size() > weights_cap
        || s.block_scales.size() > scales_cap)
    {
        if (e.empty()) { e = "destination too small"; }
        if (err && err_len > 0)
        {
            std::strncpy(err, e.c_str(), (size_t)err_len - 1);
            err[err_len - 1] = '\0';
        }
        return -1;
    }
    std::memcpy(weights, s.weights.data(), s.weights.size());
    if (!s.block_scales.empty()) { std::memcpy(scales, s.block_scales.data(), s.block_scales.size()); }
    *quant_scale = s.quant_scale;
    dims[0] = (int)s.dtype;
    dims[1] = s.n;
    dims[2] = s.k;
    return 0;
}
// Writes a container from parallel arrays of keys / blobs (tests, and saving a quantised cache).
HOST_EXPORT int cccc_host_bin_write(const char* path, int count, const char** keys, const void** blobs, const unsigned long long* lens)
{
    BinWriter w;
    for (int i = 0; i < count; i++) { w.add(keys[i], blobs[i], (size_t)lens[i]); }
    return w.save(path) ? 0 : -1;
}

// ---- decode-step linears ------------------------------------------------------------------------------
#include "decode_linears.h"

HOST_EXPORT void* cccc_host_decode_create(void* g, void* binfile, int hidden, int q_dim, int kv_dim, int ffn, int vocab, int layers,
    int max_tokens, float a_attn, float a_mlp_in, float a_mlp_out, float a_head, char* err, int err_len)
{
    auto* d = new DecodeLinears();
    ModelDims dims;
    dims.hidden = hidden;
    dims.q_dim = q_dim;
    dims.kv_dim = kv_dim;
    dims.ffn = ffn;
    dims.vocab = vocab;
    dims.layers = layers;
    std::string e;
    if (!d->load((GpuControl*)g, *(BinFile*)binfile, dims, max_tokens, 1, 0, &e))
    {
        if (err && err_len > 0)
        {
            std::strncpy(err, e.c_str(), (size_t)err_len - 1);
            err[err_len - 1] = '\0';
        }
        delete d;
        return nullptr;
    }
    d->setAlpha(a_attn, a_mlp_in, a_mlp_out, a_head);
    return d;
}
HOST_EXPORT void cccc_host_decode_destroy(void* d) { delete (DecodeLinears*)d; }
HOST_EXPORT int cccc_host_decode_step(void* d, const void* x_host, int M, int* ids, float* vals)
{
    return ((DecodeLinears*)d)->step((const uint16_t*)x_host, M, ids, vals);
}
HOST_EXPORT int cccc_host_decode_launches(void* d) { return ((DecodeLinears*)d)->launchesPerStep(); }
HOST_EXPORT unsigned long long cccc_host_decode_weight_bytes(void* d) { return ((DecodeLinears*)d)->weightBytes(); }
HOST_EXPORT void* cccc_host_decode_buffer(void* d, const char* name) { return ((DecodeLinears*)d)->buffer(name); }

// ---- typed gemm overloads (cublas_real.h:599-685, 688-752) ----------------------------------------------
HOST_EXPORT void cccc_host_gemm_typed(void* g, int weight_is_a, int ta, int tb, int M, int N, int K, float alpha, const void* A, int lda,
    const void* B, int ldb, float beta, void* Cm, int ldc, float inv_scale, int weight_type)
{
    auto* gpu = (GpuControl*)g;
    gpu->setAsCurrent();
    if (weight_is_a)
    {
        gpu->cublas_->gemm((MatrixTransType)ta, (MatrixTransType)tb, M, N, K, alpha, (const uint8_t*)A, lda, (const bfloat16*)B, ldb, beta,
            (bfloat16*)Cm, ldc, inv_scale, (DataType)weight_type);
    }
    else
    {
        gpu->cublas_->gemm((MatrixTransType)ta, (MatrixTransType)tb, M, N, K, alpha, (const bfloat16*)A, lda, (const uint8_t*)B, ldb, beta,
            (bfloat16*)Cm, ldc, inv_scale, (DataType)weight_type);
    }
}

// ---- sampler, generation loop, whole decode step ----------------------------------------------------
#include "decode_step.h"
#include "generate.h"

#include <functional>
#include <thread>

namespace
{
void setErr(char* err, int err_len, const std::string& e)
{
    if (err && err_len > 0)
    {
        std::strncpy(err, e.c_str(), (size_t)err_len - 1);
        err[err_len - 1] = '\0';
    }
}

SamplerConfig samplerOf(float temperature, int top_k, float top_p, float rep, const int* banned, int n_banned)
{
    SamplerConfig s;
    s.temperature = temperature;
    s.top_k = top_k;
    s.top_p = top_p;
    s.repetition_penalty = rep;
    s.banned_ids.assign(banned, banned + n_banned);
    return s;
}

float bf16ToFloat(uint16_t b)
{
    const uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// ints: hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, layers, qk_norm, max_context, weight_data_type
ModelConfig configOf(const int* ints, float rope_theta, float eps)
{
    ModelConfig c;
    c.hidden = ints[0];
    c.n_heads = ints[1];
    c.n_kv_heads = ints[2];
    c.head_dim = ints[3];
    c.ffn = ints[4];
    c.vocab = ints[5];
    c.layers = ints[6];
    c.qk_norm = ints[7] != 0;
    c.max_context = ints[8];
    c.weight_data_type = (DataType)ints[9];
    c.rope_theta = rope_theta;
    c.eps = eps;
    return c;
}

// gen: eos_n, eos ids..., then think_open, think_close, sys_n, turn_n, T, T_kv
GenerateConfig generateOf(const int* gen, const SamplerConfig& s)
{
    GenerateConfig g;
    const int n = gen[0];
    g.eos_ids.assign(gen + 1, gen + 1 + n);
    const int* r = gen + 1 + n;
    g.think_open_id = r[0];
    g.think_close_id = r[1];
    g.sys_n = r[2];
    g.turn_n = r[3];
    g.T = r[4];
    g.T_kv = r[5];
    g.sampler = s;
    return g;
}
}    // namespace

HOST_EXPORT int cccc_host_sample(float* logits, int V, float temperature, int top_k, float top_p, float rep, const int* banned, int n_banned,
    const int* ctx, int n_ctx, unsigned int seed)
{
    std::vector<float> l(logits, logits + V);
    std::vector<int> c(ctx, ctx + n_ctx);
    std::mt19937 rng(seed);
    return sampleLogits(l, samplerOf(temperature, top_k, top_p, rep, banned, n_banned), c, rng);
}

// The generation loop over a table of canned logits (step s returns row s % n_rows): the loop's bookkeeping
// (prefill, stop conditions, the rebuild of a full cache) without a model.  trace receives (token, pos) of
// every model step, up to trace_cap pairs; stats = rebuilds, decode steps, prefill tokens, model steps, resets,
// final context length.  ctx is updated in place (ctx_cap entries), its new length is stats[5].
HOST_EXPORT int cccc_host_generate_canned(const float* table, int n_rows, int V, int* ctx, int n_ctx, int ctx_cap, const int* gen, float temperature,
    int top_k, float top_p, float rep, const int* banned, int n_banned, unsigned int seed, int max_new, int* out, int out_cap, int* trace,
    int trace_cap, int* stats)
{
    int calls = 0, resets = 0;
    Generator g(
        V,
        [&](int token, int pos, std::vector<float>* logits_out) {
            const float* row = table + (size_t)(calls % n_rows) * V;
            if (calls < trace_cap)
            {
                trace[2 * calls] = token;
                trace[2 * calls + 1] = pos;
            }
            calls++;
            if (logits_out) { logits_out->assign(row, row + V); }
            int best = 0;
            for (int i = 1; i < V; i++)
            {
                if (row[i] > row[best]) { best = i; }
            }
            return best;
        },
        [&]() { resets++; }, seed);
    std::vector<int> c(ctx, ctx + n_ctx);
    const GenerateConfig cfg = generateOf(gen, samplerOf(temperature, top_k, top_p, rep, banned, n_banned));
    const std::vector<int> got = g.generate(c, cfg, max_new);
    const int n = (int)std::min<size_t>(got.size(), (size_t)out_cap);
    for (int i = 0; i < n; i++) { out[i] = got[i]; }
    for (int i = 0; i < (int)c.size() && i < ctx_cap; i++) { ctx[i] = c[i]; }
    stats[0] = g.rebuilds();
    stats[1] = g.decodeSteps();
    stats[2] = g.prefillTokens();
    stats[3] = calls;
    stats[4] = resets;
    stats[5] = (int)c.size();
    return (int)got.size();
}

HOST_EXPORT void* cccc_host_step_create(void* g, void* binfile, const int* ints, float rope_theta, float eps, int max_batch, int keep_host,
    char* err, int err_len)
{
    auto* d = new DecodeStep();
    d->keepHostCopies(keep_host != 0);
    std::string e;
    if (!d->load((GpuControl*)g, *(BinFile*)binfile, configOf(ints, rope_theta, eps), max_batch, nullptr, 0, &e))
    {
        setErr(err, err_len, e);
        delete d;
        return nullptr;
    }
    return d;
}
HOST_EXPORT void cccc_host_step_destroy(void* d) { delete (DecodeStep*)d; }
HOST_EXPORT int cccc_host_step_run(void* d, const int* ids, const int* pos, int M, int* next_ids, float* best, void* logits_bf16)
{
    return ((DecodeStep*)d)->step(ids, pos, M, next_ids, best, (uint16_t*)logits_bf16);
}
HOST_EXPORT void cccc_host_step_reset(void* d) { ((DecodeStep*)d)->resetCache(); }
HOST_EXPORT int cccc_host_step_use_program(void* d, int on) { return ((DecodeStep*)d)->useProgram(on != 0) ? 1 : 0; }
// what: 0 launches of the launch-per-op step, 1 launches of the last step, 2 tensors quantised while loading,
// 3 weight type, 4 weight bytes, 5 cache bytes
HOST_EXPORT unsigned long long cccc_host_step_info(void* d, int what)
{
    auto* s = (DecodeStep*)d;
    switch (what)
    {
    case 0: return (unsigned long long)s->launchesPerStep();
    case 1: return (unsigned long long)s->lastLaunches();
    case 2: return (unsigned long long)s->quantisedOnLoad();
    case 3: return (unsigned long long)s->weightType();
    case 4: return s->weightBytes();
    case 5: return s->cacheBytes();
    default: return 0;
    }
}
HOST_EXPORT int cccc_host_step_save(void* d, const char* path, char* err, int err_len)
{
    std::string e;
    if (((DecodeStep*)d)->saveNamedWeights(path, &e)) { return 0; }
    setErr(err, err_len, e);
    return -1;
}

namespace
{
// The generation loop of one rank over its DecodeStep; with several ranks every rank runs the same loop and gets the
// same tokens (the arg-max and the logits are combined across the ranks inside the step).
std::vector<int> generateOn(DecodeStep* step, TensorParallel* tp, int rank, int vocab, std::vector<int>& ctx, const GenerateConfig& cfg,
    unsigned int seed, int max_new, int* stats, int* failed)
{
    const int vloc = step->vocabLocal();
    std::vector<uint16_t> shard((size_t)vloc);
    Generator g(
        vocab,
        [&](int token, int pos, std::vector<float>* logits_out) {
            int next = -1;
            if (step->step(&token, &pos, 1, &next, nullptr, logits_out ? shard.data() : nullptr) != 0) { *failed = 1; }
            if (logits_out)
            {
                logits_out->resize((size_t)vocab);
                if (tp && tp->world() > 1) { tp->gatherLogits(rank, shard.data(), vloc, logits_out->data()); }
                else
                {
                    for (int i = 0; i < vloc; i++) { (*logits_out)[i] = bf16ToFloat(shard[i]); }
                }
            }
            return next;
        },
        [&]() { step->resetCache(); }, seed);
    std::vector<int> got = g.generate(ctx, cfg, max_new);
    if (stats)
    {
        stats[0] = g.rebuilds();
        stats[1] = g.decodeSteps();
        stats[2] = g.prefillTokens();
    }
    return got;
}
}    // namespace

// run_generate (cccc-llm/cccc-llm.cpp:347-577) over a loaded DecodeStep: prefill token by token, then decode until an
// EOS id, max_new tokens, or a full cache (rebuild).  Returns the number of generated ids (out gets up to out_cap), -1
// if a step failed.  stats = rebuilds, decode steps, prefill tokens.
HOST_EXPORT int cccc_host_step_generate(void* d, int vocab, int* ctx, int n_ctx, const int* gen, float temperature, int top_k, float top_p, float rep,
    const int* banned, int n_banned, unsigned int seed, int max_new, int* out, int out_cap, int* stats)
{
    std::vector<int> c(ctx, ctx + n_ctx);
    int failed = 0;
    const std::vector<int> got = generateOn((DecodeStep*)d, nullptr, 0, vocab, c, generateOf(gen, samplerOf(temperature, top_k, top_p, rep, banned, n_banned)),
        seed, max_new, stats, &failed);
    if (failed) { return -1; }
    for (int i = 0; i < (int)got.size() && i < out_cap; i++) { out[i] = got[i]; }
    return (int)got.size();
}

namespace
{
// Tensor parallel in one process: one thread, GpuControl and DecodeStep per device of `devices`; every rank loads its
// shard from `path`, then runs body(rank, step, tp).  Returns false with a message when a rank could not be set up (all
// ranks then stop together: a rank takes part in every barrier of join() and load() or in none).
bool runRanks(const char* path, const int* devices, int world, const ModelConfig& cfg, int max_batch,
    const std::function<void(int, DecodeStep&, TensorParallel&)>& body, std::string* err)
{
    TensorParallel tp(world);
    std::vector<std::string> errs(world);
    std::vector<int> ok_flag(world, 0), failed(world, 0);
    auto agree = [&](int r, bool ok) {
        ok_flag[r] = ok ? 1 : 0;
        tp.barrier();
        bool all = true;
        for (int i = 0; i < world; i++) { all = all && ok_flag[i] != 0; }
        tp.barrier();
        return all;
    };
    auto work = [&](int r) {
        GpuControl gpu;
        BinFile file;
        DecodeStep step;
        bool ok = gpu.init(devices[r]) == 0 && file.open(path);
        if (!ok) { errs[r] = "cannot open the device or the weight file"; }
        if (agree(r, ok)) { ok = agree(r, tp.join(r, &gpu, (unsigned int)(cfg.hidden * max_batch), &errs[r])); }
        else { ok = false; }
        if (ok) { ok = agree(r, step.load(&gpu, file, cfg, max_batch, &tp, r, &errs[r])); }
        if (!ok)
        {
            failed[r] = 1;
            return;
        }
        body(r, step, tp);
        tp.barrier();
    };
    std::vector<std::thread> threads;
    for (int r = 0; r < world; r++) { threads.emplace_back(work, r); }
    for (auto& t : threads) { t.join(); }
    bool good = true;
    std::string e;
    for (int r = 0; r < world; r++)
    {
        good = good && !failed[r];
        if (!errs[r].empty()) { e += "rank " + std::to_string(r) + ": " + errs[r] + "; "; }
    }
    if (!good && err) { *err = e.empty() ? "a rank failed to load" : e; }
    return good;
}
}    // namespace

// The generation loop on `world` GPUs of this process.  out receives rank 0's ids; returns their count, -1 on a load or
// step failure (message in err), -2 if the ranks disagree on a token.
HOST_EXPORT int cccc_host_tp_generate(const char* path, const int* devices, int world, const int* ints, float rope_theta, float eps, int* ctx,
    int n_ctx, const int* gen, float temperature, int top_k, float top_p, float rep, const int* banned, int n_banned, unsigned int seed, int max_new,
    int* out, int out_cap, int* stats, char* err, int err_len)
{
    const ModelConfig cfg = configOf(ints, rope_theta, eps);
    const GenerateConfig gcfg = generateOf(gen, samplerOf(temperature, top_k, top_p, rep, banned, n_banned));
    std::vector<std::vector<int>> got(world);
    std::vector<int> failed(world, 0), stats0(3, 0);
    std::string e;
    const bool ok = runRanks(
        path, devices, world, cfg, 1,
        [&](int r, DecodeStep& step, TensorParallel& tp) {
            std::vector<int> c(ctx, ctx + n_ctx);
            int f = 0;
            got[r] = generateOn(&step, &tp, r, cfg.vocab, c, gcfg, seed, max_new, r == 0 ? stats0.data() : nullptr, &f);
            failed[r] = f;
        },
        &e);
    if (!ok)
    {
        setErr(err, err_len, e);
        return -1;
    }
    for (int r = 0; r < world; r++)
    {
        if (failed[r])
        {
            setErr(err, err_len, "a decode step failed on rank " + std::to_string(r));
            return -1;
        }
    }
    for (int r = 1; r < world; r++)
    {
        if (got[r] != got[0]) { return -2; }
    }
    if (stats) { std::memcpy(stats, stats0.data(), 3 * sizeof(int)); }
    for (int i = 0; i < (int)got[0].size() && i < out_cap; i++) { out[i] = got[0][i]; }
    return (int)got[0].size();
}

// Feeds `tokens` (n of them, one sequence) at cache rows 0..n-1 on `world` GPUs and returns what every step gave: next_ids
// [world][n] (the combined arg-max as each rank saw it), best [n] and logits [n][vocab] floats (rank 0's gathered rows).
// Returns 0, -1 (load failure, message in err) or the number of failed steps.
HOST_EXPORT int cccc_host_tp_steps(const char* path, const int* devices, int world, const int* ints, float rope_theta, float eps, const int* tokens,
    int n, int* next_ids, float* best, float* logits, char* err, int err_len)
{
    const ModelConfig cfg = configOf(ints, rope_theta, eps);
    std::vector<int> bad(world, 0);
    std::string e;
    const bool ok = runRanks(
        path, devices, world, cfg, 1,
        [&](int r, DecodeStep& step, TensorParallel& tp) {
            std::vector<uint16_t> shard((size_t)step.vocabLocal());
            std::vector<float> row((size_t)cfg.vocab);
            for (int i = 0; i < n; i++)
            {
                int tok = tokens[i], pos = i, next = -1;
                float b = 0.f;
                if (step.step(&tok, &pos, 1, &next, &b, shard.data()) != 0) { bad[r]++; }
                tp.gatherLogits(r, shard.data(), step.vocabLocal(), row.data());
                next_ids[(size_t)r * n + i] = next;
                if (r == 0)
                {
                    best[i] = b;
                    std::memcpy(logits + (size_t)i * cfg.vocab, row.data(), row.size() * sizeof(float));
                }
            }
        },
        &e);
    if (!ok)
    {
        setErr(err, err_len, e);
        return -1;
    }
    int total = 0;
    for (int r = 0; r < world; r++) { total += bad[r]; }
    return total;
}

// ---- CPU-only checks of the host-side pieces ------------------------------------------------------------
// Writes one quantised tensor under the loaders' keys (BinWriter::addQuantised).
HOST_EXPORT int cccc_host_bin_write_quantised(const char* path, const char* name, int dtype, int n, int k, const void* weights,
    unsigned long long weight_bytes, const void* scales, unsigned long long scale_bytes, float quant_scale)
{
    WeightShard s;
    s.dtype = (DataType)dtype;
    s.n = n;
    s.k = k;
    s.quant_scale = quant_scale;
    s.weights.assign((const uint8_t*)weights, (const uint8_t*)weights + weight_bytes);
    if (scales && scale_bytes) { s.block_scales.assign((const uint8_t*)scales, (const uint8_t*)scales + scale_bytes); }
    BinWriter w;
    w.addQuantised(name, s);
    return w.save(path) ? 0 : -1;
}

// The combines of TensorParallel with `world` host threads and no device: rank r passes ids[r], values[r] (arg-max),
// absmax[r], and its shard of `per` BF16 logits; out_ids / out_best / out_absmax get what each rank received, full
// (world * world * per floats) the gathered rows as each rank saw them.  `rounds` repetitions exercise the barrier's reuse.
HOST_EXPORT int cccc_host_tp_combine_selftest(int world, int rounds, const int* ids, const float* values, const float* absmax, const void* shards,
    int per, int* out_ids, float* out_best, float* out_absmax, float* full)
{
    TensorParallel tp(world);
    std::vector<std::thread> threads;
    std::vector<int> bad(world, 0);
    for (int r = 0; r < world; r++)
    {
        threads.emplace_back([&, r]() {
            for (int it = 0; it < rounds; it++)
            {
                const int id = tp.combineArgmax(r, ids[r], values[r]);
                const float best = tp.lastBest(r);
                const float am = tp.combineAbsmax(r, absmax[r]);
                std::vector<float> row((size_t)world * per);
                tp.gatherLogits(r, (const uint16_t*)shards + (size_t)r * per, per, row.data());
                if (it == 0)
                {
                    out_ids[r] = id;
                    out_best[r] = best;
                    out_absmax[r] = am;
                    std::memcpy(full + (size_t)r * world * per, row.data(), row.size() * sizeof(float));
                }
                else if (out_ids[r] != id || out_best[r] != best || out_absmax[r] != am) { bad[r]++; }
                if (!tp.allOk(r, true) || tp.allOk(r, r != 0)) { bad[r]++; }    // all true -> true; rank 0 false -> false for all
            }
        });
    }
    for (auto& t : threads) { t.join(); }
    int total = 0;
    for (int b : bad) { total += b; }
    return total;
}
