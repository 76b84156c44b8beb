// Host helpers that encode TMA tensor maps.  The driver entry point is looked
// up at run time so the library links without libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>

namespace grb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tmap_encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// bf16 row-major [outer, inner], leading dimension ld (elements).
// Box = box_inner x box_outer elements; swizzle128 selects the 128-byte swizzle (box_inner must be 64).
inline int make_tmap_2d_bf16(CUtensorMap* tm, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                             uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  EncodeTiledFn enc = tmap_encoder();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// As above with an explicit swizzle mode (used for TMA stores of 64-byte-wide bf16 tiles).
inline int make_tmap_2d_bf16_sw(CUtensorMap* tm, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                                uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
  EncodeTiledFn enc = tmap_encoder();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// bf16 [B, T, C] with row stride ld (elements) and batch stride T*ld; box = box_c x box_t x 1, no swizzle.
inline int make_tmap_btc_bf16(CUtensorMap* tm, const void* base, uint64_t C, uint64_t T, uint64_t B, uint64_t ld,
                              uint32_t box_c, uint32_t box_t) {
  EncodeTiledFn enc = tmap_encoder();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return -2;
  cuuint64_t dims[3] = {C, T, B};
  cuuint64_t strides[2] = {ld * 2, T * ld * 2};
  cuuint32_t box[3] = {box_c, box_t, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace grb
