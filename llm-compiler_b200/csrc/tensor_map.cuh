// Host-side construction of TMA tensor maps. cuTensorMapEncodeTiled is resolved through
// the runtime (cudaGetDriverEntryPoint), so the library links against nothing but cudart
// and still loads on a machine without a GPU driver.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn encode = nullptr;
  static bool resolved = false;
  if (!resolved) {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query) ==
            cudaSuccess &&
        query == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<EncodeTiledFn>(entry);
    resolved = true;
  }
  return encode;
}

// bf16 row-major matrix [rows, cols] with a row pitch of `row_stride` elements, tiled in boxes
// of box_rows x 64 columns (128-byte rows) with the 128B swizzle; out-of-range reads give zeros.
inline bool make_bf16_matrix_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                                 int64_t row_stride, int box_rows) {
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr || box_rows > 256 || rows <= 0 || cols <= 0) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride * 2)};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bf16 tensor of logical shape [B, H, T, D] with element strides {sb, sh, st, 1}, read in boxes
// of `box_tokens` tokens x 64 elements of one (batch, head): a 4-D map whose dimensions are
// ordered by stride. *token_is_dim1 tells the kernel the coordinate order: {d, t, h, b} when
// true, {d, h, t, b} otherwise. Reads past T give zeros.
inline bool make_bf16_bhtd_map(CUtensorMap* map, const void* base, int64_t batch, int64_t heads,
                               int64_t tokens, int64_t dim, int64_t sb, int64_t sh, int64_t st,
                               int box_tokens, bool* token_is_dim1) {
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr || box_tokens > 256 || dim % 64 != 0) return false;
  *token_is_dim1 = st <= sh;
  const int64_t d1 = *token_is_dim1 ? tokens : heads, s1 = *token_is_dim1 ? st : sh;
  const int64_t d2 = *token_is_dim1 ? heads : tokens, s2 = *token_is_dim1 ? sh : st;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(dim), static_cast<cuuint64_t>(d1),
                              static_cast<cuuint64_t>(d2), static_cast<cuuint64_t>(batch)};
  // a dimension of extent 1 may come with any stride (0 included): give it a legal one
  const int64_t safe1 = d1 == 1 ? dim : s1, safe2 = d2 == 1 ? safe1 * d1 : s2;
  const int64_t safe3 = batch == 1 ? safe2 * d2 : sb;
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(safe1 * 2), static_cast<cuuint64_t>(safe2 * 2),
                                 static_cast<cuuint64_t>(safe3 * 2)};
  for (cuuint64_t stride : strides)
    if (stride % 16 != 0 || stride == 0) return false;
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(*token_is_dim1 ? box_tokens : 1),
                             static_cast<cuuint32_t>(*token_is_dim1 ? 1 : box_tokens), 1};
  const cuuint32_t element_strides[4] = {1, 1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace b200
