// Host-side construction of TMA tensor maps. The driver entry point is resolved at run time
// through the runtime API so the library carries no link-time dependency on libcuda (it has to
// load on machines without a driver for the CPU-side build check).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Generic 2-D tiled map with the 128-byte swizzle. `inner`/`outer` are extents in elements,
// `row_stride_bytes` the byte distance between rows (multiple of 16), box_inner*elem_size must be
// exactly 128 bytes for the swizzle atom used by the tensor-core descriptors. Returns 0 or an
// error code (-3: driver entry point missing, -4: encode rejected the arguments).
inline int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_size, const void* base,
                        uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                        uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -3;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elem_size;
  return r == CUDA_SUCCESS ? 0 : -4;
}

inline int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                             uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, inner, outer,
                      row_stride_bytes, box_inner, box_outer);
}

}  // namespace rb
