// Host side: build TMA tensor maps without linking libcuda (the encode entry point is looked up
// through the CUDA runtime, so the library also loads on machines that have no driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace fg {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 tensor [heads, rows, D] (contiguous) seen as a 3-D map (D, rows, heads) with a
// (64 elements = 128 bytes, box_rows, 1) box and the 128-byte swizzle.  Rows past `rows` read as
// zero, so ragged tails need no host-side padding.  Returns 0 on success.
inline int make_qkv_map(CUtensorMap* map, const void* base, int heads, int rows, int D, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return 1;
  cuuint64_t dims[3] = {cuuint64_t(D), cuuint64_t(rows), cuuint64_t(heads)};
  cuuint64_t strides[2] = {cuuint64_t(D) * 2, cuuint64_t(rows) * cuuint64_t(D) * 2};
  cuuint32_t box[3] = {64, cuuint32_t(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

}  // namespace fg
