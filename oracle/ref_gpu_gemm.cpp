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

// The reference's switch between W8A16 (BFLOAT16 activations, the default) and W8A8 (FP8_E4M3 activations):
// cccc::Cublas::setActDataType (cccc/cublas_real.h:1233).
extern "C" __attribute__((visibility("default"))) int ref_cublas_set_act_type(int type)
{
    if (ref_cublas_init()) { return 1; }
    g_blas->setActDataType((cccc::DataType)type);
    return 0;
}

// The typed overload the reference's W8A8 lives in (cccc/cublas_real.h:599-684: E4M3 weight as A, BF16 activations as B,
// quantised to E4M3 inside when the activation type is FP8_E4M3).  The type-erased dispatcher above never reaches it
// for BF16 activations (cublas_real.h:940-964 always dequantises), so it is called directly.
extern "C" __attribute__((visibility("default"))) int ref_cublas_gemm_w8_typed(int transA, int transB, int M, int N, int K, float alpha,
    const void* A, int lda, const void* B, int ldb, float beta, void* C, int ldc, float inv_scale, int weight_type, float act_scale)
{
    if (ref_cublas_init()) { return 1; }
    g_blas->gemm((cccc::MatrixTransType)transA, (cccc::MatrixTransType)transB, M, N, K, alpha, (const uint8_t*)A, lda,
        (const cccc::bfloat16*)B, ldb, beta, (cccc::bfloat16*)C, ldc, inv_scale, (cccc::DataType)weight_type, act_scale);
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : 1;
}

extern "C" __attribute__((visibility("default"))) void ref_cublas_destroy(void)
{
    delete g_blas;
    g_blas = nullptr;
}
