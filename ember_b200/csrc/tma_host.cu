// Host-side construction of TMA tensor maps. The driver's encoder is reached through
// cudaGetDriverEntryPoint, so the library does not link against libcuda.
#include "kernels.cuh"
#include "ptx.cuh"

namespace ember {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A (batch, rows, inner) row-major bf16 tensor viewed as a 3-D TMA tensor; boxes of
// box_rows x box_inner elements with the 128-byte swizzle (box_inner * 2 bytes must be 128).
// Out-of-range parts of a box read as zero. batch_stride_rows > rows describes a tensor whose batch
// entries hold more rows than are valid (a cache with spare capacity): rows past `rows` read as zero.
int make_tensor_map_bf16_3d(CUtensorMap *map, const void *base, uint64_t inner, uint64_t rows,
                            uint64_t batch, uint32_t box_inner, uint32_t box_rows, uint64_t batch_stride_rows)
{
    if (batch_stride_rows == 0) batch_stride_rows = rows;  // dense: one batch entry right after the other
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return EMBER_ERR_CUDA;
    }
    cuuint64_t dims[3] = {inner, rows, batch};
    cuuint64_t strides[2] = {inner * 2, batch_stride_rows * inner * 2};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu rows=%llu batch=%llu)", (int)r,
                  (unsigned long long)inner, (unsigned long long)rows, (unsigned long long)batch);
        return EMBER_ERR_CUDA;
    }
    return EMBER_OK;
}

// A matrix view as a 5-D TMA tensor (innermost first): row-major (cols, rows, 1, 1, 1); head-major
// (dim, seq, heads, batch, parts). Boxes of box_rows x box_cols elements (box_cols * 2 bytes = 128)
// along the two innermost dimensions, 128-byte swizzle, zero fill outside.
int make_tensor_map_bf16_view(CUtensorMap *map, const MatView &v, uint32_t box_cols, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return EMBER_ERR_CUDA;
    }
    cuuint64_t dims[5], strides[4];
    if (v.heads == 0) {
        dims[0] = (cuuint64_t)v.cols;
        dims[1] = (cuuint64_t)v.rows;
        dims[2] = dims[3] = dims[4] = 1;
        strides[0] = (cuuint64_t)v.cols * 2;
        strides[1] = strides[2] = strides[3] = (cuuint64_t)v.cols * 2 * (cuuint64_t)v.rows;
    } else {
        const cuuint64_t batch = (cuuint64_t)(v.rows / v.seq), parts = (cuuint64_t)(v.cols / (v.heads * v.dim));
        dims[0] = (cuuint64_t)v.dim;
        dims[1] = (cuuint64_t)v.seq;
        dims[2] = (cuuint64_t)v.heads;
        dims[3] = batch;
        dims[4] = parts;
        strides[0] = (cuuint64_t)v.dim * 2;
        strides[1] = strides[0] * (cuuint64_t)v.seq;
        strides[2] = strides[1] * (cuuint64_t)v.heads;
        strides[3] = strides[2] * batch;
    }
    cuuint32_t box[5] = {box_cols, box_rows, 1, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void *>(v.ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (view rows=%lld cols=%d heads=%d)", (int)r,
                  v.rows, v.cols, v.heads);
        return EMBER_ERR_CUDA;
    }
    return EMBER_OK;
}

}  // namespace ember
