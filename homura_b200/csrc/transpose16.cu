// Host side of the transposing kernel for 2-byte elements: tensor maps, encoded through the driver entry point
// the runtime hands out (the library does not link the driver).
#include "map.cuh"

#include <mutex>

namespace hmc {

namespace {

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_entry() {
    static EncodeTiled entry = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) == cudaSuccess &&
            found == cudaDriverEntryPointSuccess) {
            entry = reinterpret_cast<EncodeTiled>(fn);
        } else {
            cudaGetLastError();
        }
    });
    return entry;
}

}  // namespace

bool t16_encode_map(CUtensorMap *map, const void *base, int64_t cols, int64_t rows, int64_t outer, int64_t row_stride_elems,
                    int64_t outer_stride_elems) {
    const EncodeTiled encode = encode_entry();
    if (encode == nullptr) return false;
    // what the copy engine asks of a layout: a 16-byte aligned base, strides that are multiples of 16 bytes and
    // below 2^40, extents below 2^32
    const int64_t row_bytes = row_stride_elems * 2, outer_bytes = outer > 1 ? outer_stride_elems * 2 : row_bytes * rows;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || row_bytes % 16 != 0 || outer_bytes % 16 != 0) return false;
    if (row_bytes <= 0 || outer_bytes <= 0 || row_bytes >= (int64_t{1} << 40) || outer_bytes >= (int64_t{1} << 40)) return false;
    if (cols < 1 || rows < 1 || outer < 1 || cols >= (int64_t{1} << 32) || rows >= (int64_t{1} << 32) || outer >= (int64_t{1} << 32)) {
        return false;
    }
    const cuuint64_t extent[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(outer_bytes)};
    const cuuint32_t box[3] = {kT16Tile, kT16Tile, 1};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), extent, strides, box, element_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace hmc
