// Tensor maps for TMA tile copies. cuTensorMapEncodeTiled is a driver entry point: it is looked up at run time
// (cudaGetDriverEntryPoint), so nothing links libcuda.
#pragma once

#include <cuda.h>  // CUtensorMap and its enums only
#include <cuda_runtime.h>

namespace tma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return (EncodeTiledFn)sym;
    }();
    return fn;
}

// A [rows, row_bytes] byte matrix, row-major, copied in boxes of box_rows x box_bytes with no swizzle. Bytes of a
// box that fall outside the matrix (past a row's end or past the last row) read as zero. row_bytes and box_bytes
// are multiples of 16; the base is 16-byte aligned.
inline bool bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[2] = {row_bytes, rows}, strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes, box_rows}, elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [seqs][rows][row_bytes] bytes: boxes of 128 bytes x box_rows rows of one sequence, 128-byte swizzle (16-byte chunks
// of a box row XORed with the row's low three bits). Rows and sequences outside the tensor read as zero.
inline bool bytes_3d_swizzled(CUtensorMap* map, const void* base, uint64_t seqs, uint64_t rows, uint64_t row_bytes, uint64_t seq_bytes,
                              uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[3] = {row_bytes, rows, seqs}, strides[2] = {row_bytes, seq_bytes};
    const cuuint32_t box[3] = {128, box_rows, 1}, elem[3] = {1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [rows][64] bf16 (rows of 128 bytes), boxes of box_rows whole rows, 128-byte swizzle: the K-major operand tiles of
// the tensor cores. Rows past the end read as zero.
inline bool bf16_rows64_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[2] = {64, rows}, strides[1] = {128};
    const cuuint32_t box[2] = {64, box_rows}, elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tma
