// Host-side helpers that encode TMA tensor maps through the driver entry point (no link-time
// dependency on the driver library).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace b200
{

// ---- tensor maps -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
    CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    // initialised once, thread-safe (C++11 static initialisation)
    static const EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
        {
            return (EncodeTiledFn)sym;
        }
        cudaGetLastError();
        return nullptr;
    }();
    return fn;
}

// A 3-D view (inner run, rows, runs along k) of a row-major [rows, k] operand: dimension 1 walks
// the rows (stride = the leading dimension), dimension 2 walks the 'inner'-sized runs of one row.
// A box {inner, box_rows, box_runs} therefore lands in shared memory as [run][row][inner].
static bool make_map(CUtensorMap* map, CUtensorMapDataType dt, unsigned int elem_bytes, const void* base, unsigned int inner,
    unsigned long long rows, unsigned long long runs, unsigned long long row_stride_bytes, unsigned int box_rows,
    unsigned int box_runs, bool swizzle128, bool swizzle64 = false)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) { return false; }
    const cuuint64_t gdim[3] = { inner, rows, runs };
    const cuuint64_t gstride[2] = { row_stride_bytes, (cuuint64_t)inner * elem_bytes };
    const cuuint32_t box[3] = { inner, box_rows, box_runs };
    const cuuint32_t estr[3] = { 1, 1, 1 };
    const CUresult r = fn(map, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : (swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}


// A plain 2-D view [rows, cols] (cols contiguous) with a {box_cols, box_rows} box.
static bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, unsigned int elem_bytes, const void* base, unsigned long long cols,
    unsigned long long rows, unsigned long long row_stride_bytes, unsigned int box_cols, unsigned int box_rows, bool swizzle128)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) { return false; }
    (void)elem_bytes;
    const cuuint64_t gdim[2] = { cols, rows };
    const cuuint64_t gstride[1] = { row_stride_bytes };
    const cuuint32_t box[2] = { box_cols, box_rows };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}    // namespace b200
