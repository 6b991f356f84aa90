#include "cccc_host.h"

#include <algorithm>

#include "../../../include/cccc_cuda_b200.h"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#define LOG_ERR(...) fprintf(stderr, __VA_ARGS__)

namespace cccc
{

// ---------------------------------------------------------------------------------- Cublas
size_t Cublas::elemBytes(DataType dt)
{
    switch (dt)
    {
    case FLOAT: return 4;
    case DOUBLE: return 8;
    case HALF:
    case BFLOAT16: return 2;
    default: return 1;
    }
}

cublasStatus_t Cublas::init(cudaStream_t stream)
{
    stream_ = stream;
    cublasStatus_t r = cublasCreate(&handle_);
    if (r != CUBLAS_STATUS_SUCCESS) { return r; }
    cublasSetMathMode(handle_, CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION);    // cublas_real.h:49
    return cublasSetStream(handle_, stream_);
}

void Cublas::destroy()
{
    if (handle_)
    {
        cublasDestroy(handle_);
        handle_ = nullptr;
    }
    if (ws_)
    {
        cudaFree(ws_);
        ws_ = nullptr;
        ws_cap_ = 0;
    }
}

void* Cublas::ensureWS(size_t bytes)
{
    if (bytes <= ws_cap_) { return ws_; }
    if (ws_)
    {
        cudaStreamSynchronize(stream_);
        cudaFree(ws_);
        ws_ = nullptr;
        ws_cap_ = 0;
    }
    if (cudaMalloc(&ws_, bytes) != cudaSuccess)
    {
        cudaGetLastError();
        ws_ = nullptr;
        return nullptr;    // the reference silently skips the GEMM in this case (cublas_real.h:948-951)
    }
    ws_cap_ = bytes;
    return ws_;
}

static cudaDataType cuda_type(DataType t)
{
    switch (t)
    {
    case HALF: return CUDA_R_16F;
    case BFLOAT16: return CUDA_R_16BF;
    case DOUBLE: return CUDA_R_64F;
    default: return CUDA_R_32F;
    }
}

void Cublas::gemm(MatrixTransType TransA, MatrixTransType TransB, int M, int N, int K, float alpha, const void* A, DataType typeA,
    int lda, float invScaleA, const void* B, DataType typeB, int ldb, float invScaleB, float beta, void* C, DataType typeC,
    int ldc, float act_scale, const uint8_t* blk_scA, const uint8_t* blk_scB)
{
    const bool aQ = isQuantized(typeA), bQ = isQuantized(typeB);
    const cublasOperation_t opA = TransA == MATRIX_NO_TRANS ? CUBLAS_OP_N : CUBLAS_OP_T;
    const cublasOperation_t opB = TransB == MATRIX_NO_TRANS ? CUBLAS_OP_N : CUBLAS_OP_T;
    if (aQ && bQ)
    {
        // Both operands E4M3 (cublas_real.h:883-897 -> :754-834): weight as op(A) = A^T, activations as B; BF16 or E4M3 out.
        if (typeA == FP8_E4M3 && typeB == FP8_E4M3 && (typeC == BFLOAT16 || typeC == FP8_E4M3) && TransA == MATRIX_TRANS && TransB == MATRIX_NO_TRANS
            && cuda_gemm_fp8_fp8(A, invScaleA, B, invScaleB, C, (int)typeC, (unsigned)M, (unsigned)N, (unsigned)K, (unsigned)lda, (unsigned)ldb,
                   (unsigned)ldc, 1u, alpha, beta, stream_, 0)
                == 0)
        {
            fused_calls_++;
            return;
        }
        LOG_ERR("Cublas::gemm: both operands quantised is served for E4M3 x E4M3 with the weight transposed and aligned operands only\n");
        return;
    }
    if (aQ || bQ)
    {
        const DataType typeW = aQ ? typeA : typeB;
        const DataType typeX = aQ ? typeB : typeA;
        const uint8_t* blk = aQ ? blk_scA : blk_scB;
        const float inv = aQ ? invScaleA : invScaleB;
        if (typeX != BFLOAT16 || typeC != BFLOAT16)
        {
            LOG_ERR("Cublas::gemm: quantised weights need BF16 activations and output here (got %d, %d)\n", (int)typeX, (int)typeC);
            return;
        }
        // W8A8 (cublas_real.h:619-666, :692-739): E4M3 weights with the activation type set to FP8_E4M3, one call at any
        // token count; anything it does not serve (unaligned operands, K % 128) continues as W8A16, which is also where
        // the reference ends up when its cublasLt call fails.
        if (typeW == FP8_E4M3 && act_data_type_ == FP8_E4M3 && TransA == MATRIX_TRANS && TransB == MATRIX_NO_TRANS)
        {
            const int r = aQ ? cuda_gemm_w8a8_bf16(A, inv, B, act_scale, C, (unsigned)M, (unsigned)N, (unsigned)K, (unsigned)lda, (unsigned)ldb,
                                   (unsigned)ldc, 1u, alpha, beta, stream_, 0)
                             : cuda_gemm_w8a8_bf16(B, inv, A, act_scale, C, (unsigned)N, (unsigned)M, (unsigned)K, (unsigned)ldb, (unsigned)lda, 1u,
                                   (unsigned)ldc, alpha, beta, stream_, 0);
            if (r == 0)
            {
                fused_calls_++;
                return;
            }
        }
        // Fused path: the weight's K runs contiguously when it is op(A) = A^T (weight as A) or
        // op(B) = B (weight as B), and the activations' K is contiguous for the other operand.
        if (aQ && TransA == MATRIX_TRANS && TransB == MATRIX_NO_TRANS)
        {
            // C(M x N, ldc): M = out features, N = tokens
            if (cuda_gemm_wq_bf16((int)typeA, A, blk, inv, B, C, (unsigned)M, (unsigned)N, (unsigned)K, (unsigned)lda, (unsigned)ldb,
                    (unsigned)ldc, 1u, alpha, beta, stream_, 0)
                == 0)
            {
                fused_calls_++;
                return;
            }
        }
        if (bQ && TransA == MATRIX_TRANS && TransB == MATRIX_NO_TRANS)
        {
            // C(M x N, ldc): M = tokens, N = out features
            if (cuda_gemm_wq_bf16((int)typeB, B, blk, inv, A, C, (unsigned)N, (unsigned)M, (unsigned)K, (unsigned)ldb, (unsigned)lda,
                    1u, (unsigned)ldc, alpha, beta, stream_, 0)
                == 0)
            {
                fused_calls_++;
                return;
            }
        }
        // Reference behaviour for every other layout (cublas_real.h:943-964, :1066-1087): dequantise
        // the whole weight into the workspace, then a BF16 GEMM.
        const int ldw = aQ ? lda : ldb;
        const int colsW = aQ ? (TransA == MATRIX_NO_TRANS ? K : M) : (TransB == MATRIX_NO_TRANS ? N : K);
        const size_t sz = (size_t)ldw * colsW;
        void* ws = ensureWS(sz * 2);
        if (!ws) { return; }
        cudaStreamSynchronize(stream_);    // the conversion entry points run on the default stream and synchronise
        if (typeW == FP4_E2M1 && blk) { cuda_fp4_blockscale_to_bf16(aQ ? A : B, blk, ws, (unsigned)sz, 16); }
        else { cuda_convert(aQ ? A : B, (int)typeW, ws, (int)BFLOAT16, (unsigned)sz, inv); }
        const float fa = alpha, fb = beta;
        cublasGemmEx(handle_, opA, opB, M, N, K, &fa, aQ ? ws : A, CUDA_R_16BF, lda, aQ ? B : ws, CUDA_R_16BF, ldb, &fb, C,
            CUDA_R_16BF, ldc, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
        fallback_calls_++;
        return;
    }
    // plain types: a library GEMM, as in the reference (cublas_real.h:1150-1165)
    if (typeC == DOUBLE)
    {
        const double da = alpha, db = beta;
        cublasDgemm(handle_, opA, opB, M, N, K, &da, (const double*)A, lda, (const double*)B, ldb, &db, (double*)C, ldc);
        return;
    }
    const float fa = alpha, fb = beta;
    const cudaDataType ct = cuda_type(typeC);
    cublasGemmEx(handle_, opA, opB, M, N, K, &fa, A, ct, lda, B, ct, ldb, &fb, C, ct, ldc, CUBLAS_COMPUTE_32F,
        CUBLAS_GEMM_DEFAULT_TENSOR_OP);
}

// ------------------------------------------------------------------------------ GpuControl
thread_local GpuControl* GpuControl::current_gpu_ = nullptr;

int GpuControl::init(int device)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
    {
        cudaGetLastError();
        return 1;
    }
    device_ = device;
    if (cudaSetDevice(device_) != cudaSuccess) { return 1; }
    if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess) { return 1; }
    cublas_ = std::make_unique<Cublas>();
    if (cublas_->init(stream_) != CUBLAS_STATUS_SUCCESS) { return 1; }
    current_gpu_ = this;
    return 0;
}

GpuControl::~GpuControl()
{
    if (device_ < 0) { return; }
    cudaSetDevice(device_);
    cublas_.reset();
    for (auto& kv : allocs_) { cudaFree(kv.first); }
    allocs_.clear();
    if (stream_) { cudaStreamDestroy(stream_); }
    if (current_gpu_ == this) { current_gpu_ = nullptr; }
}

void GpuControl::setAsCurrent()
{
    if (current_gpu_ != this || true)
    {
        cudaSetDevice(device_);
        current_gpu_ = this;
    }
}

void* GpuControl::malloc(size_t bytes)
{
    setAsCurrent();
    void* p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess)
    {
        cudaGetLastError();
        LOG_ERR("GpuControl::malloc: %zu bytes failed on device %d\n", bytes, device_);
        return nullptr;
    }
    allocs_[p] = bytes;
    allocated_ += bytes;
    return p;
}

void GpuControl::free(void* p)
{
    auto it = allocs_.find(p);
    if (it == allocs_.end()) { return; }
    setAsCurrent();
    cudaStreamSynchronize(stream_);
    cudaFree(p);
    allocated_ -= it->second;
    allocs_.erase(it);
}

void GpuControl::synchronize() const { cudaStreamSynchronize(stream_); }

// ---------------------------------------------------------------------------------- Matrix
size_t Matrix::getDataSizeInByte() const
{
    const size_t n = getDataSize();
    return dt_ == FP4_E2M1 ? (n + 1) / 2 : n * Cublas::elemBytes(dt_);
}

Matrix::Matrix(int w, int h, int c, int n, DataType dt, GpuControl* gpu) :
    width_(w), height_(h), channel_(c), number_(n), row_(w * h * c), dt_(dt), gpu_(gpu)
{
    data_ = gpu_->malloc(getDataSizeInByte());
    owns_ = true;
}

Matrix Matrix::view(void* data, int w, int h, int c, int n, DataType dt, GpuControl* gpu)
{
    Matrix m;
    m.width_ = w;
    m.height_ = h;
    m.channel_ = c;
    m.number_ = n;
    m.row_ = w * h * c;
    m.dt_ = dt;
    m.gpu_ = gpu;
    m.data_ = data;
    return m;
}

Matrix::Matrix(Matrix&& o) noexcept :
    width_(o.width_), height_(o.height_), channel_(o.channel_), number_(o.number_), row_(o.row_), data_(o.data_),
    block_scale_(o.block_scale_), owns_(o.owns_), owns_scale_(o.owns_scale_), dt_(o.dt_), quant_scale_(o.quant_scale_),
    input_scale_(o.input_scale_), gpu_(o.gpu_)
{
    o.owns_ = o.owns_scale_ = false;
    o.data_ = o.block_scale_ = nullptr;
}

Matrix::~Matrix()
{
    if (owns_ && data_ && gpu_) { gpu_->free(data_); }
    if (owns_scale_ && block_scale_ && gpu_) { gpu_->free(block_scale_); }
}

void Matrix::mul(const Matrix& A, const Matrix& B, Matrix& R, float a, float r, MatrixTransType ta, MatrixTransType tb)
{
    // Matrix.cpp:1110-1118
    const int m = R.row_;
    const int n = R.number_;
    const int lda = A.row_;
    int k = A.number_;
    const int ldb = B.row_;
    if (ta == MATRIX_TRANS) { k = A.row_; }
    if (!R.isCuda()) { return; }
    R.gpu()->setAsCurrent();
    const uint8_t* blk_scA = (A.getDataType() == FP4_E2M1) ? (const uint8_t*)A.getBlockScaleData() : nullptr;
    const uint8_t* blk_scB = (B.getDataType() == FP4_E2M1) ? (const uint8_t*)B.getBlockScaleData() : nullptr;
    R.gpu()->cublas_->gemm(ta, tb, m, n, k, a, A.data(), A.getDataType(), lda, A.getQuantScale(), B.data(), B.getDataType(), ldb,
        B.getQuantScale(), r, R.data(), R.getDataType(), m, 0.0f, blk_scA, blk_scB);
}

void Matrix::mulBatched(const Matrix& A, const Matrix& B, Matrix& R, MatrixTransType ta, MatrixTransType tb, float a, float r)
{
    // Matrix.cpp:1166-1176
    const int M = (ta == MATRIX_NO_TRANS) ? A.width_ : A.height_;
    const int K = (ta == MATRIX_NO_TRANS) ? A.height_ : A.width_;
    const int N = (tb == MATRIX_NO_TRANS) ? B.height_ : B.width_;
    const int batch = A.number_;
    const int lda = (ta == MATRIX_NO_TRANS) ? M : K;
    const int ldb = (tb == MATRIX_NO_TRANS) ? K : N;
    const int ldc = M;
    const long long strideA = (long long)M * K, strideB = (long long)K * N, strideC = (long long)M * N;
    if (!R.isCuda()) { return; }
    R.gpu()->setAsCurrent();
    for (int b = 0; b < batch; b++)
    {
        // Matrix.cpp:1180-1203: byte strides (FP4 packs two per byte) and the per-batch scale offset
        const long long bsA = (A.getDataType() == FP4_E2M1) ? strideA / 2 : strideA * (long long)Cublas::elemBytes(A.getDataType());
        const long long bsB = (B.getDataType() == FP4_E2M1) ? strideB / 2 : strideB * (long long)Cublas::elemBytes(B.getDataType());
        const long long bsC = strideC * (long long)Cublas::elemBytes(R.getDataType());
        const uint8_t* blk_scA = nullptr;
        if (A.getDataType() == FP4_E2M1 && A.getBlockScaleData())
        {
            blk_scA = (const uint8_t*)A.getBlockScaleData() + (long long)b * strideA / fp4BlockSize();
        }
        const uint8_t* blk_scB = nullptr;
        if (B.getDataType() == FP4_E2M1 && B.getBlockScaleData())
        {
            blk_scB = (const uint8_t*)B.getBlockScaleData() + (long long)b * strideB / fp4BlockSize();
        }
        R.gpu()->cublas_->gemm(ta, tb, M, N, K, a, (const char*)A.data() + b * bsA, A.getDataType(), lda, A.getQuantScale(),
            (const char*)B.data() + b * bsB, B.getDataType(), ldb, B.getQuantScale(), r, (char*)R.data() + b * bsC, R.getDataType(),
            ldc, 0.0f, blk_scA, blk_scB);
    }
}

float Cublas::absmax(const float* x, size_t n)
{
    if (n == 0 || !handle_) { return 0.f; }
    float best = 0.f;
    // cublasIsamax takes an int count: larger tensors go in pieces
    for (size_t off = 0; off < n; off += (size_t)1 << 30)
    {
        const int len = (int)std::min(n - off, (size_t)1 << 30);
        int idx = 0;
        if (cublasIsamax(handle_, len, x + off, 1, &idx) != CUBLAS_STATUS_SUCCESS || idx < 1) { continue; }
        float v = 0.f;
        cudaMemcpyAsync(&v, x + off + (idx - 1), sizeof(float), cudaMemcpyDeviceToHost, stream_);
        cudaStreamSynchronize(stream_);
        best = std::fmax(best, std::fabs(v));
    }
    return best;
}

void Matrix::quantizeWeights(DataType target, const std::function<float(float)>& combine_absmax)
{
    if (!Cublas::isQuantized(target) || !owns_ || !gpu_) { return; }
    if (dt_ != FLOAT && dt_ != BFLOAT16) { return; }
    gpu_->setAsCurrent();
    gpu_->synchronize();
    const size_t n = getDataSize();
    // Matrix.cpp:310-318: work from a float copy
    float* fbuf = (float*)gpu_->malloc(n * sizeof(float));
    if (!fbuf)
    {
        // the other ranks wait in the combine: take part in it before giving up
        if (combine_absmax && target != FP4_E2M1) { combine_absmax(0.f); }
        return;
    }
    if (dt_ == FLOAT) { cudaMemcpy(fbuf, data_, n * sizeof(float), cudaMemcpyDeviceToDevice); }
    else { cuda_convert(data_, (int)dt_, fbuf, (int)FLOAT, (unsigned)n, 1.0f); }
    if (target == FP4_E2M1)
    {
        // Matrix.cpp:321-335: block 16, E4M3 dequant multipliers
        const size_t n_blocks = (n + 15) / 16;
        void* q = gpu_->malloc((n + 1) / 2);
        void* sc = gpu_->malloc(n_blocks);
        cuda_float_to_fp4_blockscale(fbuf, q, sc, (unsigned)n, 16);
        gpu_->free(data_);
        data_ = q;
        block_scale_ = sc;
        owns_scale_ = true;
        quant_scale_ = 1.0f;
    }
    else
    {
        // Matrix.cpp:340-350: absmax -> forward scale maxval/absmax, stored multiplier absmax/maxval
        float absmax = gpu_->cublas_->absmax(fbuf, n);
        if (combine_absmax) { absmax = combine_absmax(absmax); }
        const float maxval = target == FP8_E4M3 ? 448.f : 57344.f;
        float fwd = 1.f;
        quant_scale_ = 1.f;
        if (absmax > 0.f)
        {
            fwd = maxval / absmax;
            quant_scale_ = absmax / maxval;
        }
        void* q = gpu_->malloc(n);
        cuda_convert(fbuf, (int)FLOAT, q, (int)target, (unsigned)n, fwd);
        gpu_->free(data_);
        data_ = q;
    }
    gpu_->free(fbuf);
    dt_ = target;
}

void Matrix::loadQuantizedDirect(const void* host_bytes, size_t n_bytes, DataType dt, float quant_scale)
{
    if (!gpu_) { return; }
    gpu_->setAsCurrent();
    if (owns_ && data_) { gpu_->free(data_); }
    dt_ = dt;
    data_ = gpu_->malloc(n_bytes);
    owns_ = true;
    cudaMemcpy(data_, host_bytes, n_bytes, cudaMemcpyHostToDevice);
    quant_scale_ = quant_scale;
}

}    // namespace cccc
