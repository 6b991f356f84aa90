#include "decode_step.h"

#include "../../../include/cccc_cuda_b200.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

namespace cccc
{

namespace
{
bool fail(std::string* err, const std::string& what)
{
    if (err) { *err = what; }
    return false;
}

// the host bfloat16 constructor of the reference truncates (cccc/types.h:36-60)
uint16_t bf16Trunc(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return (uint16_t)(u >> 16);
}

uint16_t bf16Round(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) { return (uint16_t)((u >> 16) | 0x40); }
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float halfToFloat(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
    if (exp == 0)
    {
        if (man == 0) { u = sign; }
        else
        {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    }
    else if (exp == 31) { u = sign | 0x7f800000u | (man << 13); }
    else { u = sign | ((exp + 112) << 23) | (man << 13); }
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
}    // namespace

// ---- TensorParallel ----

TensorParallel::~TensorParallel()
{
    // The areas belong to this object, not to the ranks' GpuControl objects: those live on the ranks' threads and are
    // gone by the time the last owner of the TensorParallel lets go of it.
    for (int r = 0; r < world_; r++)
    {
        if (device_[r] < 0) { continue; }
        cudaSetDevice(device_[r]);
        if (recv_[r]) { cudaFree(recv_[r]); }
        if (flag_[r]) { cudaFree(flag_[r]); }
    }
}

void TensorParallel::barrier()
{
    std::unique_lock<std::mutex> lk(m_);
    const unsigned long long gen = generation_;
    if (++waiting_ == world_)
    {
        waiting_ = 0;
        generation_++;
        cv_.notify_all();
        return;
    }
    cv_.wait(lk, [&] { return generation_ != gen; });
}

bool TensorParallel::allOk(int rank, bool ok)
{
    {
        std::lock_guard<std::mutex> lk(m_);
        ok_[rank] = ok ? 1 : 0;
    }
    barrier();
    bool all = true;
    for (int r = 0; r < world_; r++) { all = all && ok_[r] != 0; }
    barrier();
    return all;
}

bool TensorParallel::join(int rank, GpuControl* gpu, unsigned int n_max, std::string* err)
{
    if (rank < 0 || rank >= world_ || !gpu) { return fail(err, "bad rank"); }
    gpu->setAsCurrent();
    n_max = (n_max + 3u) & ~3u;
    const size_t rb = cuda_b200_allreduce_recv_bytes(world_, n_max), fb = cuda_b200_fused_flag_bytes(world_);
    void *recv = nullptr, *flag = nullptr;
    bool ok = cudaMalloc(&recv, rb) == cudaSuccess && cudaMalloc(&flag, fb) == cudaSuccess;
    if (ok) { ok = cudaMemset(recv, 0, rb) == cudaSuccess && cudaMemset(flag, 0, fb) == cudaSuccess; }
    if (!ok) { cudaGetLastError(); }
    {
        std::lock_guard<std::mutex> lk(m_);
        device_[rank] = gpu->getDeviceID();
        recv_[rank] = recv;
        flag_[rank] = flag;
        n_max_ = n_max;
        if (!ok) { failed_ = true; }
    }
    barrier();    // every rank's areas exist
    // peer access to every other rank's device (the reference's multi-device mode uses cudaMemcpyPeer,
    // cccc/Matrix.cpp:498-517; the fused exchange stores straight into the peers' areas)
    for (int r = 0; r < world_ && !failed_; r++)
    {
        if (r == rank) { continue; }
        const int peer = device_[r];
        if (peer == gpu->getDeviceID()) { continue; }
        int can = 0;
        cudaDeviceCanAccessPeer(&can, gpu->getDeviceID(), peer);
        if (!can)
        {
            std::lock_guard<std::mutex> lk(m_);
            failed_ = true;
            break;
        }
        const cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); }
        else if (e != cudaSuccess)
        {
            std::lock_guard<std::mutex> lk(m_);
            failed_ = true;
        }
    }
    cudaDeviceSynchronize();
    barrier();
    if (failed_) { return fail(err, "tensor parallel setup failed (allocation or peer access)"); }
    return true;
}

int TensorParallel::combineArgmax(int rank, int global_id, float value)
{
    {
        std::lock_guard<std::mutex> lk(m_);
        best_[rank] = value;
        id_[rank] = global_id;
    }
    barrier();
    int win = -1;
    float top = 0.f;
    for (int r = 0; r < world_; r++)
    {
        if (id_[r] < 0) { continue; }    // a shard of only NaN
        if (win < 0 || best_[r] > top)
        {
            win = id_[r];
            top = best_[r];
        }
    }
    last_best_[rank] = top;
    barrier();    // nobody overwrites the slots before all have read them
    return win;
}

float TensorParallel::combineAbsmax(int rank, float value)
{
    {
        std::lock_guard<std::mutex> lk(m_);
        absmax_[rank] = value;
    }
    barrier();
    float top = 0.f;
    for (int r = 0; r < world_; r++) { top = std::fmax(top, absmax_[r]); }
    barrier();
    return top;
}

void TensorParallel::gatherLogits(int rank, const uint16_t* shard, int n, float* full)
{
    {
        std::lock_guard<std::mutex> lk(m_);
        if (row_.size() != (size_t)world_ * n) { row_.assign((size_t)world_ * n, 0.f); }
    }
    barrier();    // the row has its size before anyone writes a slice
    for (int i = 0; i < n; i++)
    {
        const uint32_t u = (uint32_t)shard[i] << 16;
        std::memcpy(&row_[(size_t)rank * n + i], &u, 4);
    }
    barrier();
    std::memcpy(full, row_.data(), row_.size() * sizeof(float));
    barrier();
}

// ---- DecodeStep ----

DecodeStep::~DecodeStep()
{
    if (!gpu_) { return; }
    gpu_->setAsCurrent();
    gpu_->synchronize();
    if (program_) { cuda_decode_program_destroy(program_); }
    for (auto g : graphs_)
    {
        if (g) { cudaGraphExecDestroy(g); }
    }
    quantised_.clear();
    for (void* p : owned_) { gpu_->free(p); }
    if (h_ids_) { cudaFreeHost(h_ids_); }
    if (h_logits_) { cudaFreeHost(h_logits_); }
}

void* DecodeStep::dmalloc(size_t bytes)
{
    void* p = gpu_->malloc(bytes);
    if (p) { owned_.push_back(p); }
    return p;
}

bool DecodeStep::loadLinear(const BinFile& f, const std::string& name, int N, int K, char kind, Linear* out, std::string* err)
{
    WeightShard sh;
    if (!loadWeightShard(f, name, N, K, kind, world_, rank_, &sh, err)) { return false; }
    out->n = sh.n;
    out->k = sh.k;
    if (Cublas::isQuantized(sh.dtype))
    {
        if (wt_ == CURRENT) { wt_ = sh.dtype; }
        if (sh.dtype != wt_) { return fail(err, "weight '" + name + "' has another quantised type than the first one"); }
        if (sh.dtype == FP4_E2M1 && sh.block_scales.empty()) { return fail(err, "weight '" + name + "' is FP4 without block scales"); }
        out->w = dmalloc(sh.weights.size());
        if (!out->w || cudaMemcpy(out->w, sh.weights.data(), sh.weights.size(), cudaMemcpyHostToDevice) != cudaSuccess)
        {
            return fail(err, "no device memory for '" + name + "'");
        }
        if (!sh.block_scales.empty())
        {
            out->s = dmalloc(sh.block_scales.size());
            if (!out->s || cudaMemcpy(out->s, sh.block_scales.data(), sh.block_scales.size(), cudaMemcpyHostToDevice) != cudaSuccess)
            {
                return fail(err, "no device memory for the block scales of '" + name + "'");
            }
        }
        out->inv = sh.quant_scale;
    }
    else
    {
        // BF16 / half / float tensor: quantise on the GPU while loading (cccc/Net.cpp:1142-1233 -> cccc/Matrix.cpp:301-355)
        if (!Cublas::isQuantized(cfg_.weight_data_type)) { return fail(err, "weight '" + name + "' is not quantised and no weight_data_type is set"); }
        if (wt_ == CURRENT) { wt_ = cfg_.weight_data_type; }
        if (wt_ != cfg_.weight_data_type) { return fail(err, "weight '" + name + "' would get another quantised type than the first one"); }
        const size_t n = (size_t)sh.n * sh.k;
        if (sh.dtype == HALF)
        {
            // the device converter takes float and BF16: widen half on the host
            std::vector<uint8_t> wide(n * 4);
            const uint16_t* src = (const uint16_t*)sh.weights.data();
            float* dst = (float*)wide.data();
            for (size_t i = 0; i < n; i++) { dst[i] = halfToFloat(src[i]); }
            sh.weights.swap(wide);
            sh.dtype = FLOAT;
        }
        Matrix m(sh.k, sh.n, 1, 1, sh.dtype, gpu_);
        if (!m.data() || cudaMemcpy(m.data(), sh.weights.data(), sh.weights.size(), cudaMemcpyHostToDevice) != cudaSuccess)
        {
            return fail(err, "no device memory for '" + name + "'");
        }
        if (tp_ && world_ > 1)
        {
            m.quantizeWeights(wt_, [&](float a) { return tp_->combineAbsmax(rank_, a); });
        }
        else { m.quantizeWeights(wt_); }
        if (m.getDataType() != wt_) { return fail(err, "quantising '" + name + "' failed"); }
        out->w = m.data();
        out->s = (void*)m.getBlockScaleData();
        out->inv = m.getQuantScale();
        if (keep_host_)
        {
            const size_t wb = wt_ == FP4_E2M1 ? n / 2 : n;
            sh.weights.resize(wb);
            cudaMemcpy(sh.weights.data(), out->w, wb, cudaMemcpyDeviceToHost);
            sh.block_scales.clear();
            if (out->s)
            {
                sh.block_scales.resize(n / 16);
                cudaMemcpy(sh.block_scales.data(), out->s, n / 16, cudaMemcpyDeviceToHost);
            }
            sh.dtype = wt_;
            sh.quant_scale = out->inv;
        }
        quantised_.push_back(std::move(m));
        quantised_on_load_++;
    }
    weight_bytes_ += (wt_ == FP4_E2M1 ? (size_t)sh.n * sh.k / 2 + (size_t)sh.n * sh.k / 16 : (size_t)sh.n * sh.k);
    if (keep_host_) { stored_.push_back(Stored{ name, std::move(sh) }); }
    return true;
}

bool DecodeStep::loadBf16(const BinFile& f, const std::string& name, size_t n, uint16_t** out, bool required, std::string* err)
{
    *out = nullptr;
    std::string key;
    DataType dt;
    if (!f.findTypedWeight(name, &key, &dt))
    {
        return required ? fail(err, "tensor '" + name + "' is missing") : true;
    }
    std::vector<uint16_t> host(n);
    if (dt == BFLOAT16)
    {
        if (f.entry(key).length != n * 2 || !f.read(key, 0, n * 2, host.data())) { return fail(err, "tensor '" + name + "' has the wrong size"); }
    }
    else if (dt == FLOAT)
    {
        // float checkpoints: to BF16 as the device conversion of the reference rounds (cccc/Net.cpp:1404-1440)
        std::vector<float> tmp(n);
        if (f.entry(key).length != n * 4 || !f.read(key, 0, n * 4, tmp.data())) { return fail(err, "tensor '" + name + "' has the wrong size"); }
        for (size_t i = 0; i < n; i++) { host[i] = bf16Round(tmp[i]); }
    }
    else if (dt == HALF)
    {
        if (f.entry(key).length != n * 2 || !f.read(key, 0, n * 2, host.data())) { return fail(err, "tensor '" + name + "' has the wrong size"); }
        for (size_t i = 0; i < n; i++) { host[i] = bf16Round(halfToFloat(host[i])); }
    }
    else { return fail(err, "tensor '" + name + "' must be BF16, half or float"); }
    *out = (uint16_t*)dmalloc(n * 2);
    if (!*out || cudaMemcpy(*out, host.data(), n * 2, cudaMemcpyHostToDevice) != cudaSuccess) { return fail(err, "no device memory for '" + name + "'"); }
    if (keep_host_) { plain_.emplace_back(name, std::move(host)); }
    return true;
}

bool DecodeStep::load(GpuControl* gpu, const BinFile& file, const ModelConfig& cfg, int max_batch, TensorParallel* tp, int rank, std::string* err)
{
    gpu_ = gpu;
    tp_ = tp;
    cfg_ = cfg;
    world_ = tp ? tp->world() : 1;
    rank_ = tp ? rank : 0;
    max_batch_ = max_batch;
    wt_ = CURRENT;
    gpu_->setAsCurrent();
    if (cfg.hidden <= 0 || cfg.layers <= 0 || cfg.head_dim <= 0 || cfg.max_context <= 0 || max_batch <= 0 || max_batch > 32)
    {
        return fail(err, "bad model configuration");
    }
    if (cfg.n_heads % world_ || cfg.n_kv_heads % world_ || cfg.ffn % world_ || cfg.vocab % world_)
    {
        return fail(err, "heads, ffn or vocabulary do not divide over the ranks");
    }
    H_ = cfg.n_heads / world_;
    Hkv_ = cfg.n_kv_heads / world_;
    q_loc_ = H_ * cfg.head_dim;
    kv_loc_ = Hkv_ * cfg.head_dim;
    ffn_loc_ = cfg.ffn / world_;
    vocab_loc_ = cfg.vocab / world_;
    qkv_ld_ = q_loc_ + 2 * kv_loc_;

    // With several ranks, the tensors are loaded first and the ranks agree that all of them succeeded before the
    // first step (whose exchange waits for every peer) is issued.
    bool ok = loadTensors(file, err);
    if (tp_ && world_ > 1 && !tp_->allOk(rank_, ok))
    {
        if (ok) { fail(err, "another rank failed to load"); }
        return false;
    }
    if (!ok) { return false; }
    // first use of the kernels allocates the library's per-device workspace: do it before any capture
    std::vector<int> z(max_batch, 0);
    cudaMemcpy(d_ids_, z.data(), (size_t)max_batch * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_pos_, z.data(), (size_t)max_batch * 4, cudaMemcpyHostToDevice);
    if (tp_) { tp_->barrier(); }
    const int rc = issue(1, gpu_->stream());
    gpu_->synchronize();
    const bool stepped = rc >= 0 && cuda_check_error("decode step warm-up") == 0;
    launches_per_step_ = rc;
    resetCache();
    if (tp_ && world_ > 1)
    {
        if (!tp_->allOk(rank_, stepped)) { return fail(err, "the first decode step failed"); }
    }
    else if (!stepped) { return fail(err, "the first decode step failed"); }
    return true;
}

bool DecodeStep::loadTensors(const BinFile& file, std::string* err)
{
    const ModelConfig& cfg = cfg_;
    const int max_batch = max_batch_;
    const int q_dim = cfg.n_heads * cfg.head_dim, kv_dim = cfg.n_kv_heads * cfg.head_dim;
    layers_.resize(cfg.layers);
    layers_loaded_ = 0;
    for (int i = 0; i < cfg.layers; i++)
    {
        Layer& L = layers_[i];
        const std::string s = "_" + std::to_string(i);
        if (!loadLinear(file, "W_q" + s, q_dim, cfg.hidden, 'c', &L.q, err) || !loadLinear(file, "W_k" + s, kv_dim, cfg.hidden, 'c', &L.k, err)
            || !loadLinear(file, "W_v" + s, kv_dim, cfg.hidden, 'c', &L.v, err) || !loadLinear(file, "W_o" + s, cfg.hidden, q_dim, 'r', &L.o, err)
            || !loadLinear(file, "W_gate" + s, cfg.ffn, cfg.hidden, 'c', &L.gate, err) || !loadLinear(file, "W_up" + s, cfg.ffn, cfg.hidden, 'c', &L.up, err)
            || !loadLinear(file, "W_down" + s, cfg.hidden, cfg.ffn, 'r', &L.down, err))
        {
            return false;
        }
        layers_loaded_++;
        if (!loadBf16(file, "W_rms_attn" + s, cfg.hidden, &L.attn_norm, true, err) || !loadBf16(file, "W_rms_ffn" + s, cfg.hidden, &L.ffn_norm, true, err)
            || !loadBf16(file, "W_qnorm" + s, cfg.head_dim, &L.q_norm, cfg.qk_norm, err) || !loadBf16(file, "W_knorm" + s, cfg.head_dim, &L.k_norm, cfg.qk_norm, err))
        {
            return false;
        }
        if (!cfg.qk_norm) { L.q_norm = L.k_norm = nullptr; }
        const size_t cache = (size_t)max_batch * Hkv_ * cfg.max_context * cfg.head_dim * 2;
        L.k_cache = (uint16_t*)dmalloc(cache);
        L.v_cache = (uint16_t*)dmalloc(cache);
        if (!L.k_cache || !L.v_cache) { return fail(err, "no device memory for the KV cache"); }
        cudaMemset(L.k_cache, 0, cache);
        cudaMemset(L.v_cache, 0, cache);
        cache_bytes_ += 2 * cache;
    }
    if (!loadLinear(file, "W_lm_head", cfg.vocab, cfg.hidden, 'c', &lm_head_, err)) { return false; }
    if (!loadBf16(file, "W_emb", (size_t)cfg.vocab * cfg.hidden, &emb_, true, err) || !loadBf16(file, "W_rms_final", cfg.hidden, &final_norm_, true, err))
    {
        return false;
    }

    // RoPE tables, computed on the host in float and stored through the truncating host constructor
    // (cccc/NetCifa.cpp:431-475)
    {
        const int half = cfg.head_dim / 2;
        std::vector<uint16_t> c((size_t)cfg.max_context * half), s((size_t)cfg.max_context * half);
        for (int t = 0; t < cfg.max_context; t++)
        {
            for (int d = 0; d < half; d++)
            {
                const float ang = (float)t * std::pow(cfg.rope_theta, -2.0f * (float)d / (float)cfg.head_dim);
                c[(size_t)t * half + d] = bf16Trunc(std::cos(ang));
                s[(size_t)t * half + d] = bf16Trunc(std::sin(ang));
            }
        }
        cos_ = (uint16_t*)dmalloc(c.size() * 2);
        sin_ = (uint16_t*)dmalloc(s.size() * 2);
        if (!cos_ || !sin_) { return fail(err, "no device memory for the RoPE tables"); }
        cudaMemcpy(cos_, c.data(), c.size() * 2, cudaMemcpyHostToDevice);
        cudaMemcpy(sin_, s.data(), s.size() * 2, cudaMemcpyHostToDevice);
    }

    const size_t B = (size_t)max_batch;
    x_ = (uint16_t*)dmalloc(B * cfg.hidden * 2);
    xn_ = (uint16_t*)dmalloc(B * cfg.hidden * 2);
    tmp_ = (uint16_t*)dmalloc(B * cfg.hidden * 2);
    qkv_ = (uint16_t*)dmalloc(B * qkv_ld_ * 2);
    att_ = (uint16_t*)dmalloc(B * q_loc_ * 2);
    gu_ = (uint16_t*)dmalloc(B * 2 * ffn_loc_ * 2);
    h_ = (uint16_t*)dmalloc(B * ffn_loc_ * 2);
    logits_ = (uint16_t*)dmalloc(B * vocab_loc_ * 2);
    d_ids_ = (int*)dmalloc(B * 4);
    d_pos_ = (int*)dmalloc(B * 4);
    d_best_ = (float*)dmalloc(B * 4);
    if (!x_ || !xn_ || !tmp_ || !qkv_ || !att_ || !gu_ || !h_ || !logits_ || !d_ids_ || !d_pos_ || !d_best_) { return fail(err, "no device memory for the step's buffers"); }
    // one pinned block: ids in, positions in, ids out, best out
    if (cudaMallocHost((void**)&h_ids_, B * 16) != cudaSuccess) { return fail(err, "no pinned memory"); }
    h_pos_ = h_ids_ + B;
    h_out_ = h_pos_ + B;
    h_best_ = (float*)(h_out_ + B);
    if (cudaMallocHost((void**)&h_logits_, B * vocab_loc_ * 2) != cudaSuccess) { return fail(err, "no pinned memory for the logits"); }
    if (world_ > 1)
    {
        const size_t cb = cuda_b200_fused_counter_bytes();
        seq_counters_ = dmalloc(cb);
        if (!seq_counters_) { return fail(err, "no device memory"); }
        cudaMemset(seq_counters_, 0, cb);
        if (tp_->nMax() < (unsigned int)(B * cfg.hidden)) { return fail(err, "the exchange areas are smaller than max_batch * hidden"); }
    }
    graphs_.assign(max_batch + 1, nullptr);
    gpu_->synchronize();
    return true;
}

void DecodeStep::resetCache()
{
    gpu_->setAsCurrent();
    const size_t cache = (size_t)max_batch_ * Hkv_ * cfg_.max_context * cfg_.head_dim * 2;
    for (auto& L : layers_)
    {
        cudaMemsetAsync(L.k_cache, 0, cache, gpu_->stream());
        cudaMemsetAsync(L.v_cache, 0, cache, gpu_->stream());
    }
    gpu_->synchronize();
}

int DecodeStep::issue(int M, cudaStream_t st)
{
    const unsigned int PDL = 1u, RES = 8u;
    const int wt = (int)wt_;
    const bool tp = world_ > 1;
    const unsigned int hid = cfg_.hidden;
    int n = 0, bad = 0;
    auto ok = [&](int rc) {
        if (rc != 0) { bad++; }
        n++;
    };
    auto norm = [&](const uint16_t* scale, bool pending) {
        ok(cuda_rms_norm_bf16(x_, pending ? tmp_ : nullptr, pending ? x_ : nullptr, xn_, scale, M, hid, cfg_.eps, st, PDL));
    };
    auto row_linear = [&](const Linear& L, const uint16_t* src) {
        if (tp)
        {
            ok(cuda_gemm_wq_bf16_allreduce(wt, L.w, L.s, L.inv, src, tmp_, hid, M, L.k, L.k, L.k, hid, 1, 1.0f, tp_->recvPtrs(), tp_->flagPtrs(),
                seq_counters_, tp_->nMax(), rank_, world_, st, PDL));
        }
        else { ok(cuda_gemm_wq_bf16(wt, L.w, L.s, L.inv, src, x_, hid, M, L.k, L.k, L.k, hid, 1, 1.0f, 1.0f, st, PDL | RES)); }
    };
    ok(cuda_embed_bf16(d_ids_, emb_, x_, hid, M, cfg_.vocab, st, PDL));
    bool pending = false;
    for (auto& L : layers_)
    {
        norm(L.attn_norm, pending);
        cuda_wq_linear g[3] = {};
        const Linear* qkv[3] = { &L.q, &L.k, &L.v };
        unsigned int off = 0;
        for (int j = 0; j < 3; j++)
        {
            g[j].W = qkv[j]->w;
            g[j].blk_scales = qkv[j]->s;
            g[j].Y = qkv_ + off;
            g[j].inv_scale = qkv[j]->inv;
            g[j].alpha = 1.0f;
            g[j].beta = 0.0f;
            g[j].N_out = qkv[j]->n;
            g[j].ldw = hid;
            g[j].ldy_m = qkv_ld_;
            g[j].ldy_n = 1;
            off += qkv[j]->n;
        }
        ok(cuda_gemm_wq_bf16_group(wt, 3, g, xn_, M, hid, hid, st, PDL));
        cuda_attn_decode a = attnArgs(L, M);
        ok(cuda_attn_decode_bf16(&a, st, PDL));
        row_linear(L.o, att_);
        norm(L.ffn_norm, tp);
        cuda_wq_linear u[2] = {};
        const Linear* gu[2] = { &L.gate, &L.up };
        for (int j = 0; j < 2; j++)
        {
            u[j].W = gu[j]->w;
            u[j].blk_scales = gu[j]->s;
            u[j].Y = gu_ + (size_t)j * ffn_loc_;
            u[j].inv_scale = gu[j]->inv;
            u[j].alpha = 1.0f;
            u[j].beta = 0.0f;
            u[j].N_out = ffn_loc_;
            u[j].ldw = hid;
            u[j].ldy_m = 2 * ffn_loc_;
            u[j].ldy_n = 1;
        }
        ok(cuda_gemm_wq_bf16_group(wt, 2, u, xn_, M, hid, hid, st, PDL));
        ok(cuda_swiglu_bf16(gu_, gu_ + ffn_loc_, h_, M, ffn_loc_, 2 * ffn_loc_, 2 * ffn_loc_, ffn_loc_, st, PDL));
        row_linear(L.down, h_);
        pending = tp;
    }
    norm(final_norm_, pending);
    ok(cuda_gemm_wq_bf16(wt, lm_head_.w, lm_head_.s, lm_head_.inv, xn_, logits_, vocab_loc_, M, hid, hid, hid, vocab_loc_, 1, 1.0f, 0.0f, st, PDL));
    ok(cuda_argmax_bf16(logits_, M, vocab_loc_, vocab_loc_, d_ids_, d_best_, st));
    return bad ? -1 : n;
}

cuda_attn_decode DecodeStep::attnArgs(const Layer& L, int M) const
{
    cuda_attn_decode a = {};
    a.q = qkv_;
    a.k = qkv_ + q_loc_;
    a.v = qkv_ + q_loc_ + kv_loc_;
    a.q_norm = L.q_norm;
    a.k_norm = L.k_norm;
    a.cos_tab = cos_;
    a.sin_tab = sin_;
    a.k_cache = L.k_cache;
    a.v_cache = L.v_cache;
    a.pos = d_pos_;
    a.out = att_;
    a.ldq = a.ldk = a.ldv = qkv_ld_;
    a.ldo = q_loc_;
    a.B = M;
    a.H = H_;
    a.Hkv = Hkv_;
    a.head_dim = cfg_.head_dim;
    a.T_max = cfg_.max_context;
    a.epsilon = cfg_.eps;
    a.dk = 0.f;
    return a;
}

bool DecodeStep::buildProgram()
{
    if (program_) { return true; }
    if (world_ > 1) { return false; }
    const unsigned int RES = 8u, PAIRED = 16u;
    const unsigned int hid = cfg_.hidden;
    ::cuda_decode_program* p = nullptr;
    if (cuda_decode_program_create(&p, (int)wt_, 1) != 0) { return false; }
    bool good = true;
    auto lin = [](const Linear& L, void* Y, unsigned int ldw, unsigned int ldy, float beta) {
        cuda_wq_linear g = {};
        g.W = L.w;
        g.blk_scales = L.s;
        g.Y = Y;
        g.inv_scale = L.inv;
        g.alpha = 1.0f;
        g.beta = beta;
        g.N_out = L.n;
        g.ldw = ldw;
        g.ldy_m = ldy;
        g.ldy_n = 1;
        return g;
    };
    auto input = [&](int mode, const void* x, unsigned int ld, const void* w) {
        cuda_decode_input in = {};
        in.mode = mode;
        in.x = x;
        in.ldx = ld;
        in.norm_weight = w;
        in.epsilon = cfg_.eps;
        return in;
    };
    for (auto& L : layers_)
    {
        if (!good) { break; }
        cuda_wq_linear g[3] = { lin(L.q, qkv_, hid, qkv_ld_, 0.f), lin(L.k, qkv_ + q_loc_, hid, qkv_ld_, 0.f), lin(L.v, qkv_ + q_loc_ + kv_loc_, hid, qkv_ld_, 0.f) };
        cuda_decode_input in = input(1, x_, hid, L.attn_norm);
        good = good && cuda_decode_program_add_linears(p, 3, g, &in, hid, 0) == 0;
        cuda_attn_decode a = attnArgs(L, 1);
        good = good && cuda_decode_program_add_attention(p, &a) == 0;
        cuda_wq_linear o = lin(L.o, x_, q_loc_, hid, 1.0f);
        in = input(0, att_, q_loc_, nullptr);
        good = good && cuda_decode_program_add_linears(p, 1, &o, &in, q_loc_, RES) == 0;
        cuda_wq_linear gu[2] = { lin(L.gate, h_, hid, ffn_loc_, 0.f), lin(L.up, h_, hid, ffn_loc_, 0.f) };
        in = input(1, x_, hid, L.ffn_norm);
        good = good && cuda_decode_program_add_linears(p, 2, gu, &in, hid, PAIRED) == 0;
        cuda_wq_linear d = lin(L.down, x_, ffn_loc_, hid, 1.0f);
        in = input(0, h_, ffn_loc_, nullptr);
        good = good && cuda_decode_program_add_linears(p, 1, &d, &in, ffn_loc_, RES) == 0;
    }
    if (good)
    {
        cuda_wq_linear h = lin(lm_head_, logits_, hid, vocab_loc_, 0.f);
        cuda_decode_input in = input(1, x_, hid, final_norm_);
        good = cuda_decode_program_add_linears(p, 1, &h, &in, hid, 0) == 0 && cuda_decode_program_finalize(p) == 0;
    }
    if (!good)
    {
        cuda_decode_program_destroy(p);
        return false;
    }
    program_ = p;
    return true;
}

bool DecodeStep::useProgram(bool on)
{
    if (!on)
    {
        use_program_ = false;
        return true;
    }
    gpu_->setAsCurrent();
    use_program_ = buildProgram();
    return use_program_;
}

int DecodeStep::step(const int* token_ids, const int* positions, int M, int* next_ids, float* best_logits, uint16_t* logits_host)
{
    if (M < 1 || M > max_batch_) { return -1; }
    gpu_->setAsCurrent();
    cudaStream_t st = gpu_->stream();
    for (int i = 0; i < M; i++)
    {
        h_ids_[i] = token_ids[i];
        h_pos_[i] = positions[i];
    }
    cudaMemcpyAsync(d_ids_, h_ids_, (size_t)M * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_pos_, h_pos_, (size_t)M * 4, cudaMemcpyHostToDevice, st);
    int rc = 0;
    if (use_program_ && M == 1 && program_)
    {
        rc = cuda_embed_bf16(d_ids_, emb_, x_, cfg_.hidden, 1, cfg_.vocab, st, 0);
        rc |= cuda_decode_program_launch(program_, st);
        rc |= cuda_argmax_bf16(logits_, 1, vocab_loc_, vocab_loc_, d_ids_, d_best_, st);
        last_launches_ = 3;
    }
    else
    {
        if (!graphs_[M])
        {
            // the first step for this M records the launches; later ones replay the graph
            cudaGraph_t graph = nullptr;
            if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { return 1; }
            const int n = issue(M, st);
            const cudaError_t e = cudaStreamEndCapture(st, &graph);
            if (n < 0 || e != cudaSuccess || !graph)
            {
                if (graph) { cudaGraphDestroy(graph); }
                cudaGetLastError();
                return n < 0 ? -1 : 1;
            }
            cudaGraphExec_t exec = nullptr;
            const cudaError_t ei = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (ei != cudaSuccess) { return 1; }
            graphs_[M] = exec;
        }
        // every rank is about to launch: the exchange inside the row-parallel linears waits for the peers
        if (tp_ && world_ > 1) { tp_->barrier(); }
        rc = cudaGraphLaunch(graphs_[M], st) == cudaSuccess ? 0 : 1;
        last_launches_ = launches_per_step_;
    }
    cudaMemcpyAsync(h_out_, d_ids_, (size_t)M * 4, cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(h_best_, d_best_, (size_t)M * 4, cudaMemcpyDeviceToHost, st);
    if (logits_host) { cudaMemcpyAsync(h_logits_, logits_, (size_t)M * vocab_loc_ * 2, cudaMemcpyDeviceToHost, st); }
    if (cudaStreamSynchronize(st) != cudaSuccess) { rc = 1; }
    if (cuda_check_error("decode step") != 0) { rc = 1; }
    if (logits_host) { std::memcpy(logits_host, h_logits_, (size_t)M * vocab_loc_ * 2); }
    for (int i = 0; i < M; i++)
    {
        int id = h_out_[i] < 0 ? -1 : h_out_[i] + rank_ * vocab_loc_;
        float best = h_best_[i];
        if (tp_ && world_ > 1)
        {
            id = tp_->combineArgmax(rank_, id, best);
            best = tp_->lastBest(rank_);
        }
        next_ids[i] = id;
        if (best_logits) { best_logits[i] = best; }
    }
    return rc;
}

bool DecodeStep::saveNamedWeights(const std::string& path, std::string* err) const
{
    if (world_ != 1) { return fail(err, "a cache file holds whole tensors: load on one rank to write it"); }
    if (stored_.empty()) { return fail(err, "keepHostCopies(true) before load() keeps what this writes"); }
    BinWriter w;
    for (const auto& s : stored_) { w.addQuantised(s.name, s.shard); }
    for (const auto& t : plain_) { w.add("weight_bf16_" + t.first, t.second.data(), t.second.size() * 2); }
    return w.save(path) ? true : fail(err, "cannot write '" + path + "'");
}

}    // namespace cccc
