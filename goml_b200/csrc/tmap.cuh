// tmap.cuh — host-side construction of TMA tensor maps for raw device
// pointers handed over a C ABI.  cuTensorMapEncodeTiled is a driver-API
// symbol; it is fetched through the runtime (cudaGetDriverEntryPoint) so the
// shared libraries keep the reference libraries' link line (cudart only, no
// hard libcuda dependency).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>

namespace sm100 {

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline encode_tiled_fn get_encode_tiled() {
    static std::atomic<encode_tiled_fn> cached{nullptr};
    encode_tiled_fn f = cached.load(std::memory_order_acquire);
    if (f) return f;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !p)
        return nullptr;
    f = reinterpret_cast<encode_tiled_fn>(p);
    cached.store(f, std::memory_order_release);
    return f;
}

// 2-D map over a dense row-major byte matrix [rows, row_bytes] (u8 elements),
// box = [box_rows, box_bytes].  row_bytes must be a multiple of 16 and base
// 16-byte aligned (checked by the callers, which return an error code instead
// of letting the copy fault).
inline bool make_tmap_u8_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                            uint32_t box_bytes, CUtensorMapSwizzle swz) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_bytes, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D map over [outer, rows, row_bytes] u8 (e.g. [BH, S, D]); box covers
// [1, box_rows, box_bytes].  Rows beyond `rows` read as zero, so a tile never
// crosses into the next head.
inline bool make_tmap_u8_3d(CUtensorMap* m, const void* base, uint64_t outer, uint64_t rows, uint64_t row_bytes,
                            uint32_t box_rows, uint32_t box_bytes, CUtensorMapSwizzle swz) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[3] = {row_bytes, rows, outer};
    cuuint64_t strides[2] = {row_bytes, row_bytes * rows};
    cuuint32_t box[3] = {box_bytes, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D map over 16-bit elements [outer, rows, cols] for TMA stores of fp16 output tiles.
inline bool make_tmap_u16_3d(CUtensorMap* m, const void* base, uint64_t outer, uint64_t rows, uint64_t cols,
                             uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[3] = {cols, rows, outer};
    cuuint64_t strides[2] = {cols * 2, cols * 2 * rows};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D map over a dense row-major fp32 matrix [rows, cols]; box = [box_rows, box_cols].  cols * 4 must be a
// multiple of 16 and base 16-byte aligned.  Used by TMA reduce-add stores (out-of-range parts of a box are clipped).
inline bool make_tmap_f32_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                             uint32_t box_cols, CUtensorMapSwizzle swz) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 4};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D map over a dense row-major matrix of 16-bit elements [rows, cols] (fp16 or bf16: the copy does not interpret
// them); box = [box_rows, box_cols].  cols * 2 must be a multiple of 16 and base 16-byte aligned.  Used by TMA
// stores of an output tile (parts of a box outside the matrix are not written).
inline bool make_tmap_u16_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                             uint32_t box_cols, CUtensorMapSwizzle swz) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace sm100
