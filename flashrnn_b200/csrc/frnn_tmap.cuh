// Host side of the tensor-map bulk copies: encodes a CUtensorMap over a tensor of 16-bit elements seen as 5-d.
// The driver entry point is looked up through the runtime, so the library needs no link against libcuda.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "frnn_elem.cuh"

namespace FRNN_NS {

// dims / strides innermost first (dims[0] contiguous elements, strides in bytes for dims 1..4), `box` = tile extents.
// 128-byte swizzle: the tile's innermost extent is 64 elements; out-of-range elements read as zero and are dropped on
// stores.  Returns false when the driver offers no encoder or rejects the description.
inline bool encode_tiles16(CUtensorMap* tm, const void* base, const uint64_t (&dims)[5], const uint64_t (&strides)[4],
                              const uint32_t (&box)[5]) {
  static const PFN_cuTensorMapEncodeTiled_v12000 encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }();
  if (!encode) return false;
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < 5; ++i) { gdim[i] = dims[i]; gbox[i] = box[i]; estr[i] = 1; }
  for (int i = 0; i < 4; ++i) gstr[i] = strides[i];
  return encode(tm, kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), gdim, gstr, gbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace FRNN_NS
