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
