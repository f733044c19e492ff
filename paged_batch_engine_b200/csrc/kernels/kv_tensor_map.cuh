// A layer's key or value pages as a tensor map for TMA tile loads: the cache tensor
// [pages, kv_heads, page_tokens, head_dim] read as a matrix [pages * kv_heads * page_tokens,
// head_dim] of bfloat16, fetched in boxes of box_rows rows (a page, or part of a larger page)
// by 64 columns with the 128-byte swizzle: in shared memory a box is box_rows rows of 128 bytes,
// the 16-byte chunk c of row r at chunk position c ^ (r & 7) (the destination 1024-byte aligned).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace pbe {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's encoder, through the runtime (no link against the driver library).
inline EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// 0, or a cudaError_t value.  head_dim must be a multiple of 64, the cache 16-byte aligned.
inline int make_kv_tensor_map(CUtensorMap* map, const void* cache, long long rows, int head_dim, int box_rows) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace pbe
