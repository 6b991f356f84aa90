// The REFERENCE's CPU form of the quantized-weight linear, assembled from its own two CPU primitives
// and timed as the benchmark's CPU arm.  Test/benchmark infrastructure only; nothing of the reference
// is copied here: its cccc/types.h is found through the include path given by the Makefile.
//
//   1. per-element decode with the reference's host codecs (cccc/types.h:69-90 fp8_e4m3 -> float,
//      :136-166 fp8_e5m2 -> float, :257-261 fp4_e2m1::get), times the dequant multiplier, into a
//      float buffer - what MatrixData::getData does element by element (cccc/MatrixData.h:61-77);
//   2. the column-major sgemm the reference's CPU branch calls (cccc/cblas_real.h:332-335 from
//      cccc/Matrix.cpp:1155): C[N_out x M] = A^T[N_out x K] * B[K x M], lda = K, ldb = K, ldc = N_out,
//      through OpenBLAS's cblas_sgemm loaded at run time (the reference links OpenBLAS; its library is
//      not vendored, so the one shipped inside the Python environment is used when present).
#include "types.h"

#include <cstddef>
#include <cstdint>
#include <dlfcn.h>
#include <cstdio>
#include <omp.h>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace
{
typedef void (*sgemm_fn)(int order, int transA, int transB, int M, int N, int K, float alpha, const float* A, int lda, const float* B,
    int ldb, float beta, float* C, int ldc);
typedef void (*set_threads_fn)(int);
sgemm_fn g_sgemm = nullptr;
}

// blas_path: an OpenBLAS shared library; prefix: its symbol prefix ("" or "scipy_").  0 = ready.
REF_API int ref_cpu_blas_init(const char* blas_path, const char* prefix, int threads)
{
    void* h = dlopen(blas_path, RTLD_NOW | RTLD_LOCAL);
    if (!h) { return 1; }
    char name[128];
    snprintf(name, sizeof(name), "%scblas_sgemm", prefix);
    g_sgemm = (sgemm_fn)dlsym(h, name);
    snprintf(name, sizeof(name), "%sopenblas_set_num_threads", prefix);
    set_threads_fn st = (set_threads_fn)dlsym(h, name);
    if (st && threads > 0) { st(threads); }
    return g_sgemm ? 0 : 1;
}

REF_API int ref_cpu_threads(void) { return omp_get_max_threads(); }
REF_API void ref_cpu_set_threads(int n) { omp_set_num_threads(n); }

// Step 1.  w_type: cccc::DataType (4 e4m3, 5 e5m2, 6 fp4).  blk: FP4 block scales (E4M3 bytes, one per
// 16 elements) or NULL.  n elements.
REF_API void ref_cpu_dequant(int w_type, const uint8_t* W, const uint8_t* blk, float inv_scale, float* wf, size_t n)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++)
    {
        float v;
        if (w_type == 6)
        {
            float sc = inv_scale;
            if (blk)
            {
                cccc::fp8_e4m3 s;
                s.bits = blk[i / 16];
                sc = (float)s;
            }
            v = cccc::fp4_e2m1::get(W, (int)i) * sc;
        }
        else if (w_type == 5)
        {
            cccc::fp8_e5m2 b;
            b.bits = W[i];
            v = (float)b * inv_scale;
        }
        else
        {
            cccc::fp8_e4m3 b;
            b.bits = W[i];
            v = (float)b * inv_scale;
        }
        wf[i] = v;
    }
}

// Step 2.  wf [N_out][K] floats (= the reference's (K, N_out) column-major A), X [M][K], Y [M][N_out].
// Returns 1 when no BLAS was loaded.
REF_API int ref_cpu_sgemm(const float* wf, const float* X, float* Y, int N_out, int M, int K)
{
    if (!g_sgemm) { return 1; }
    // CblasColMajor = 102, CblasTrans = 112, CblasNoTrans = 111
    g_sgemm(102, 112, 111, N_out, M, K, 1.0f, wf, K, X, K, 0.0f, Y, N_out);
    return 0;
}
