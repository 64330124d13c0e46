// Host side of TMA: tensor maps are encoded by the driver (cuTensorMapEncodeTiled), reached through
// the runtime's entry-point query so that the library does not link against libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace va {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tmap_encoder() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// Map of a (B, H, S, 128) tensor of 16-bit elements with element strides (sb, sh, ss) and unit
// inner stride, read in boxes of `box_rows` rows by 64 elements (128 bytes, the span of the
// 128-byte swizzle): coordinates are {element, row, head, batch}.  Rows past S read as zeros.
inline bool encode_rows_map(CUtensorMap* map, int is_bf16, const void* ptr, int batch, int heads, int64_t rows, int64_t sb,
                            int64_t sh, int64_t ss, int box_rows) {
  EncodeTiledFn enc = tmap_encoder();
  if (!enc) return false;
  const cuuint64_t dims[4] = {128, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t st_s = (cuuint64_t)ss * 2, st_h = (cuuint64_t)sh * 2, st_b = (cuuint64_t)sb * 2;
  // a dimension of extent 1 never advances: any legal stride will do where the caller's is not usable
  if (heads == 1 && (st_h == 0 || st_h % 16 != 0)) st_h = st_s * (cuuint64_t)rows;
  if (batch == 1 && (st_b == 0 || st_b % 16 != 0)) st_b = st_h * (cuuint64_t)heads;
  const cuuint64_t strides[3] = {st_s, st_h, st_b};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(ptr), dims,
             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace va
