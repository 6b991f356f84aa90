// C++ host layer above the C-ABI: the reference's own interface for the quantized-weight linear
// path, so that cccc code written against Matrix / Cublas / GpuControl runs unchanged.
//
//   GpuControl   device ownership (cccc/GpuControl.h:50-165) plus the stream the reference lacks
//   Cublas       gemm(...) with the signature and routing of cccc/cublas_real.h:875-1166
//   Matrix       the tensor facts the path needs (cccc/Matrix.h) and the static entry points
//                mul (cccc/Matrix.cpp:1107-1157), mulBatched (:1162-1268), quantizeWeights (:301-355),
//                loadQuantizedDirect (:357-375)
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>

#include <cublas_v2.h>
#include <cuda_runtime.h>

namespace cccc
{

// cccc/types.h:24-34
enum DataType
{
    FLOAT = 0,
    DOUBLE = 1,
    HALF = 2,
    BFLOAT16 = 3,
    FP8_E4M3 = 4,
    FP8_E5M2 = 5,
    FP4_E2M1 = 6,
    CURRENT = 65535,
};

// cccc/blas_types.h:10-14
enum MatrixTransType
{
    MATRIX_NO_TRANS = 0,
    MATRIX_TRANS = 1,
};

// cccc/types.h:36-60: the 16-bit storage type (bit pattern only here)
struct bfloat16
{
    uint16_t bits;
};

class GpuControl;

// The quantised GEMM dispatcher.  One per GpuControl, as in the reference.
class Cublas
{
public:
    Cublas() = default;
    ~Cublas() { destroy(); }
    Cublas(const Cublas&) = delete;
    Cublas& operator=(const Cublas&) = delete;

    cublasStatus_t init(cudaStream_t stream);
    void destroy();

    static bool isQuantized(DataType dt) { return dt == FP8_E4M3 || dt == FP8_E5M2 || dt == FP4_E2M1; }    // cublas_real.h:855
    static size_t elemBytes(DataType dt);                                                                  // cublas_real.h:860

    // C = alpha * op(A) * op(B) + beta * C, column-major; either operand may be the quantised weight.
    // Same arguments as cccc/cublas_real.h:875-880.  Quantised x BF16 -> BF16 with the weight's K
    // contiguous goes to the fused kernel; every other supported combination keeps the reference's
    // behaviour (dequantise into the grow-only workspace, then cublasGemmEx).
    void gemm(MatrixTransType TransA, MatrixTransType TransB, int M, int N, int K, float alpha, const void* A, DataType typeA,
        int lda, float invScaleA, const void* B, DataType typeB, int ldb, float invScaleB, float beta, void* C, DataType typeC,
        int ldc, float act_scale = 0.0f, const uint8_t* blk_scA = nullptr, const uint8_t* blk_scB = nullptr);

    // The typed overloads of cccc/cublas_real.h:599-685 (quantised weight as A) and :688-752 (as B): BF16 activations
    // and output, weight_type says how the bytes of the uint8_t operand decode.  They forward to the dispatcher above,
    // so the fused kernel serves them where the reference dequantises and calls cublasGemmEx (:673-684, :740-751).
    void gemm(MatrixTransType TransA, MatrixTransType TransB, int M, int N, int K, float alpha, const uint8_t* A, int lda,
        const bfloat16* B, int ldb, float beta, bfloat16* C, int ldc, float inv_scale = 1.0f, DataType weight_type = FP8_E4M3,
        float act_scale = 0.0f)
    {
        gemm(TransA, TransB, M, N, K, alpha, A, weight_type, lda, inv_scale, B, BFLOAT16, ldb, 1.0f, beta, C, BFLOAT16, ldc, act_scale);
    }
    void gemm(MatrixTransType TransA, MatrixTransType TransB, int M, int N, int K, float alpha, const bfloat16* A, int lda,
        const uint8_t* B, int ldb, float beta, bfloat16* C, int ldc, float inv_scale = 1.0f, DataType weight_type = FP8_E4M3,
        float act_scale = 0.0f)
    {
        gemm(TransA, TransB, M, N, K, alpha, A, BFLOAT16, lda, 1.0f, B, weight_type, ldb, inv_scale, beta, C, BFLOAT16, ldc, act_scale);
    }
    // Largest |x| of n floats on the device, as Matrix::quantizeWeights finds it (cublasIsamax, cccc/Matrix.cpp:340-343).
    float absmax(const float* x, size_t n);

    // W8A16 (BFLOAT16, the default) or W8A8 (FP8_E4M3): cccc/cublas_real.h:1228-1233
    void setActDataType(DataType dt) { act_data_type_ = dt; }
    DataType getActDataType() const { return act_data_type_; }
    int fusedCalls() const { return fused_calls_; }
    int fallbackCalls() const { return fallback_calls_; }
    float getLastFp8OutScale() const { return 1.0f; }

private:
    void* ensureWS(size_t bytes);    // cublas_real.h:1188-1225: grow-only
    cublasHandle_t handle_ = nullptr;
    cudaStream_t stream_ = nullptr;
    void* ws_ = nullptr;
    size_t ws_cap_ = 0;
    int fused_calls_ = 0, fallback_calls_ = 0;
    DataType act_data_type_ = BFLOAT16;
};

// One per device.  The reference creates no stream (everything runs on the legacy default stream
// and every wrapper synchronises); this one owns a stream and hands it to every launch.
class GpuControl
{
public:
    GpuControl() = default;
    ~GpuControl();
    int init(int device);                      // GpuControl.cpp:351-436
    void setAsCurrent();                       // GpuControl.cpp:311-327
    static GpuControl* getCurrentCuda() { return current_gpu_; }
    int getDeviceID() const { return device_; }
    cudaStream_t stream() const { return stream_; }
    void* malloc(size_t bytes);                // GpuControl.cpp:459-516: tracked allocations
    void free(void* p);
    size_t allocatedBytes() const { return allocated_; }
    void synchronize() const;
    std::unique_ptr<Cublas> cublas_;

private:
    static thread_local GpuControl* current_gpu_;    // GpuControl.cpp:18
    int device_ = -1;
    cudaStream_t stream_ = nullptr;
    std::map<void*, size_t> allocs_;
    size_t allocated_ = 0;
};

// Column-major tensor with dims (width, height, channel, number); row_ = width*height*channel.
class Matrix
{
public:
    Matrix() = default;
    Matrix(int w, int h, int c, int n, DataType dt, GpuControl* gpu);
    // A view of memory the caller owns (weights loaded elsewhere).
    static Matrix view(void* data, int w, int h, int c, int n, DataType dt, GpuControl* gpu);
    ~Matrix();
    Matrix(const Matrix&) = delete;
    Matrix& operator=(const Matrix&) = delete;
    Matrix(Matrix&& o) noexcept;

    int width_ = 0, height_ = 0, channel_ = 0, number_ = 0, row_ = 0;
    void* data() const { return data_; }
    DataType getDataType() const { return dt_; }
    size_t getDataSize() const { return (size_t)row_ * number_; }                // elements
    size_t getDataSizeInByte() const;                                             // FP4: ceil(n/2), MatrixData.h:159
    float getQuantScale() const { return quant_scale_; }                         // a DEQUANT multiplier (Matrix.cpp:346)
    void setQuantScale(float s) { quant_scale_ = s; }
    float getInputScale() const { return input_scale_; }
    void* getBlockScaleData() const { return block_scale_; }
    void setBlockScaleData(void* p) { block_scale_ = p; }
    static int fp4BlockSize() { return 16; }                                      // MatrixData.h:23
    GpuControl* gpu() const { return gpu_; }
    bool isCuda() const { return gpu_ != nullptr; }

    // R = a*op(A)*op(B) + r*R (Matrix.cpp:1107-1157)
    static void mul(const Matrix& A, const Matrix& B, Matrix& R, float a = 1, float r = 0, MatrixTransType ta = MATRIX_NO_TRANS,
        MatrixTransType tb = MATRIX_NO_TRANS);
    // batch = A.number_ independent products (Matrix.cpp:1162-1268); every LLM linear is
    // mulBatched(W, X, Y, MATRIX_TRANS, MATRIX_NO_TRANS, 1, 0) with batch 1.
    static void mulBatched(const Matrix& A, const Matrix& B, Matrix& R, MatrixTransType ta, MatrixTransType tb, float a = 1,
        float r = 0);
    // In-place weight quantisation with the reference's rules (Matrix.cpp:301-355): FP8 per-tensor
    // scale maxval/absmax with the stored multiplier absmax/maxval; FP4 block 16 with E4M3 scales.
    // The matrix must hold FLOAT or BFLOAT16 data it owns.  combine_absmax (optional) maps this matrix's absmax to
    // the one to use: a tensor-parallel shard passes its value in and gets the whole tensor's back, because the
    // per-tensor FP8 scale is shared by the shards.
    void quantizeWeights(DataType target, const std::function<float(float)>& combine_absmax = {});
    // Upload pre-quantised bytes (Matrix.cpp:357-375).
    void loadQuantizedDirect(const void* host_bytes, size_t n_bytes, DataType dt, float quant_scale);

private:
    void* data_ = nullptr;
    void* block_scale_ = nullptr;
    bool owns_ = false, owns_scale_ = false;
    DataType dt_ = FLOAT;
    float quant_scale_ = 1.0f, input_scale_ = 0.0f;
    GpuControl* gpu_ = nullptr;
};

}    // namespace cccc
