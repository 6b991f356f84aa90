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
