// Thin C-ABI around the REFERENCE's own quantised GEMM dispatcher, cccc::Cublas::gemm
// (cccc/cublas_real.h:875-1166), compiled unmodified from the reference tree through the
// include path given by the Makefile.  Test infrastructure only: it lets the GPU tests and
// the benchmark's comparison leg run the reference's dequantise-then-cuBLAS path on the
// same device buffers as the new kernels.  Nothing of the reference is copied here.
#define ENABLE_CUDA 1
#include <cuda_runtime.h>
#include <cstdint>
#include <cstring>
#include "types.h"
#include "cublas_real.h"

namespace
{
cccc::Cublas* g_blas = nullptr;
}

extern "C" __attribute__((visibility("default"))) int ref_cublas_init(void)
{
    if (!g_blas)
    {
        g_blas = new cccc::Cublas();
        if (g_blas->init() != CUBLAS_STATUS_SUCCESS) { return 1; }
    }
    return 0;
}

// Argument meaning is exactly that of cccc::Cublas::gemm (column-major, C = alpha*op(A)*op(B) + beta*C).
extern "C" __attribute__((visibility("default"))) int ref_cublas_gemm(int transA, int transB, int M, int N, int K,
    float alpha, const void* A, int typeA, int lda, float invScaleA, const void* B, int typeB, int ldb,
    float invScaleB, float beta, void* C, int typeC, int ldc, float act_scale, const void* blk_scA,
    const void* blk_scB)
{
    if (ref_cublas_init()) { return 1; }
    g_blas->gemm((cccc::MatrixTransType)transA, (cccc::MatrixTransType)transB, M, N, K, alpha, A,
        (cccc::DataType)typeA, lda, invScaleA, B, (cccc::DataType)typeB, ldb, invScaleB, beta, C,
        (cccc::DataType)typeC, ldc, act_scale, (const uint8_t*)blk_scA, (const uint8_t*)blk_scB);
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : 1;
}

extern "C" __attribute__((visibility("default"))) void ref_cublas_destroy(void)
{
    delete g_blas;
    g_blas = nullptr;
}
