#include "tensormap.cuh"

#include <cudaTypedefs.h>
#include <mutex>

namespace df8 {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    });
    return fn;
}
}  // namespace

namespace {
df8_status pick_swizzle(int swizzle_bytes, CUtensorMapSwizzle* sw) {
    *sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    if (swizzle_bytes == 32) *sw = CU_TENSOR_MAP_SWIZZLE_32B;
    else if (swizzle_bytes == 64) *sw = CU_TENSOR_MAP_SWIZZLE_64B;
    else if (swizzle_bytes == 128) *sw = CU_TENSOR_MAP_SWIZZLE_128B;
    else if (swizzle_bytes != 0) return fail(DF8_ERR_INVALID, "unsupported TMA swizzle of %d bytes", swizzle_bytes);
    return DF8_OK;
}
}  // namespace

df8_status make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                            uint32_t box_rows, uint32_t box_cols, int swizzle_bytes) {
    EncodeFn fn = encode_fn();
    if (!fn) return fail(DF8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch_bytes & 15u))
        return fail(DF8_ERR_INVALID, "TMA operand must be 16-byte aligned with a row pitch that is a multiple of 16 "
                                     "(base %p, pitch %llu)", base, (unsigned long long)pitch_bytes);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapSwizzle sw;
    df8_status rc = pick_swizzle(swizzle_bytes, &sw);
    if (rc != DF8_OK) return rc;
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DF8_ERR_CUDA, "cuTensorMapEncodeTiled (fp32) failed with CUresult %d (rows %llu cols %llu pitch %llu box %ux%u)",
                    int(r), (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes,
                    box_rows, box_cols);
    return DF8_OK;
}

df8_status make_tmap_3d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t slab_cols, uint64_t slabs,
                           uint64_t pitch_bytes, uint64_t slab_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                           int swizzle_bytes) {
    EncodeFn fn = encode_fn();
    if (!fn) return fail(DF8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch_bytes & 15u) || (slab_stride_bytes & 15u))
        return fail(DF8_ERR_INVALID, "TMA operand must be 16-byte aligned with pitches that are multiples of 16 "
                                     "(base %p, row pitch %llu, slab stride %llu)", base,
                    (unsigned long long)pitch_bytes, (unsigned long long)slab_stride_bytes);
    cuuint64_t dims[3] = {slab_cols, rows, slabs};
    cuuint64_t strides[2] = {pitch_bytes, slab_stride_bytes};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapSwizzle sw;
    df8_status rc = pick_swizzle(swizzle_bytes, &sw);
    if (rc != DF8_OK) return rc;
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DF8_ERR_CUDA, "cuTensorMapEncodeTiled (3-d) failed with CUresult %d (rows %llu slab cols %llu slabs %llu)",
                    int(r), (unsigned long long)rows, (unsigned long long)slab_cols, (unsigned long long)slabs);
    return DF8_OK;
}

df8_status make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                           uint32_t box_rows, uint32_t box_cols, int swizzle_bytes) {
    EncodeFn fn = encode_fn();
    if (!fn) return fail(DF8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch_bytes & 15u))
        return fail(DF8_ERR_INVALID, "TMA operand must be 16-byte aligned with a row pitch that is a multiple of 16 "
                                     "(base %p, pitch %llu)", base, (unsigned long long)pitch_bytes);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
    else if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
    else if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
    else if (swizzle_bytes != 0) return fail(DF8_ERR_INVALID, "unsupported TMA swizzle of %d bytes", swizzle_bytes);
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DF8_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows %llu cols %llu pitch %llu box %ux%u)",
                    int(r), (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes,
                    box_rows, box_cols);
    return DF8_OK;
}

}  // namespace df8
