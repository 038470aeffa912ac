// Host-side construction of TMA tensor maps (no link-time dependency on libcuda: the driver entry
// point is looked up through the runtime).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace qpam {

// ------------------------------------------------------------------ TMA descriptors
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Row-major bf16 matrix [outer][inner] with `row_stride` elements between rows; boxes of
// box_inner x box_outer elements, 128-byte swizzle, out-of-range elements read as zero.
static inline int make_map(CUtensorMap* m, const void* base, int64_t inner, int64_t outer, int64_t row_stride,
                    int box_inner, int box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return QPAM_ECUDA;
  }
  QPAM_REQUIRE(((uintptr_t)base & 15) == 0 && (row_stride * 2) % 16 == 0, "TMA operand is not 16-byte aligned");
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%lld outer=%lld stride=%lld box=%dx%d)", (int)r,
              (long long)inner, (long long)outer, (long long)row_stride, box_inner, box_outer);
    return QPAM_ECUDA;
  }
  return QPAM_OK;
}

}  // namespace qpam
