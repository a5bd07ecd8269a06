// Host-side encoding of TMA tensor maps through the driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace aidn {
namespace tmap {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn& encode_fn() {
  static EncodeTiledFn fn = nullptr;
  return fn;
}

inline cudaError_t resolve_encode() {
  if (encode_fn()) return cudaSuccess;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
  encode_fn() = reinterpret_cast<EncodeTiledFn>(fn);
  return cudaSuccess;
}

// [B, H, S, D] tensor viewed as a 4-D TMA tensor (D, S, H, B); box = box_cols x box_rows x 1 x 1.
inline bool encode_bhsd(CUtensorMap* tm, CUtensorMapDataType dt, int esz, CUtensorMapSwizzle swz, const void* base,
                        int64_t D, int64_t S, int64_t H, int64_t B, const int64_t* stride /*B,H,S in elements*/,
                        int box_cols, int box_rows) {
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  // A dimension of extent 1 never advances; give it a harmless valid stride.
  const int64_t s_s = stride[2];
  const int64_t s_h = H > 1 ? stride[1] : s_s * S;
  const int64_t s_b = B > 1 ? stride[0] : (s_h * H > s_s * S ? s_h * H : s_s * S);
  cuuint64_t strides[3] = {(cuuint64_t)(s_s * esz), (cuuint64_t)(s_h * esz), (cuuint64_t)(s_b * esz)};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUresult r = encode_fn()(tm, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace tmap
}  // namespace aidn
