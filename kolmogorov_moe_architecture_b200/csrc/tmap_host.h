// Host-side helper: encode a rank-4 bf16 TMA tensor map with 128-byte swizzle through the
// driver entry point (resolved at run time, so nothing links against libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

namespace kmoe {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
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

// dims/box innermost first; strides in bytes for dims 1..3.  Returns 0 or a negative code.
inline int encode_bf16_4d(CUtensorMap* out, const void* base, const cuuint64_t dims[4], const cuuint64_t strides[3],
                          const cuuint32_t box[4]) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -10;
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 != 0) return -12;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return -13;
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -14;
}

}  // namespace kmoe
