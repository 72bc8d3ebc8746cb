// The 16-bit element type of Wx, R, b, the gradients and (unless fp32) the states.  Every translation unit of the
// library is compiled twice: as is (bfloat16, namespace frnn) and with -DFRNN_F16 (float16, namespace frnn_f16); the
// C entry points pick the set that matches frnn_problem.dtype_io.  Arithmetic is fp32 in both; only operand formats,
// conversions and the tensor-map element type differ.  (The reference builds one extension per dtype from -D macros,
// flashrnn/flashrnn/flashrnn.py:339-383.)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#if defined(FRNN_NS_OVERRIDE)
#define FRNN_NS FRNN_NS_OVERRIDE  // a translation unit that instantiates the shared templates with other compile options
#elif defined(FRNN_F16)
#define FRNN_NS frnn_f16
#else
#define FRNN_NS frnn
#endif

namespace FRNN_NS {

#ifdef FRNN_F16
using elem_t = __half;
using elem2_t = __half2;
constexpr bool kF16 = true;
constexpr uint32_t kOneBits = 0x3C00u;  // 1.0
__host__ __device__ __forceinline__ elem2_t floats_to_elem2(float lo, float hi) { return __floats2half2_rn(lo, hi); }
__host__ __device__ __forceinline__ float2 elem2_to_floats(elem2_t v) { return __half22float2(v); }
__host__ __device__ __forceinline__ elem_t float_to_elem(float x) { return __float2half_rn(x); }
__host__ __device__ __forceinline__ float elem_to_float(elem_t x) { return __half2float(x); }
__device__ __forceinline__ uint32_t elem_bits(elem_t x) { return __half_as_ushort(x); }
#define FRNN_MMA_TYPE "f16"
#else
using elem_t = __nv_bfloat16;
using elem2_t = __nv_bfloat162;
constexpr bool kF16 = false;
constexpr uint32_t kOneBits = 0x3F80u;  // 1.0
__host__ __device__ __forceinline__ elem2_t floats_to_elem2(float lo, float hi) { return __floats2bfloat162_rn(lo, hi); }
__host__ __device__ __forceinline__ float2 elem2_to_floats(elem2_t v) { return __bfloat1622float2(v); }
__host__ __device__ __forceinline__ elem_t float_to_elem(float x) { return __float2bfloat16_rn(x); }
__host__ __device__ __forceinline__ float elem_to_float(elem_t x) { return __bfloat162float(x); }
__device__ __forceinline__ uint32_t elem_bits(elem_t x) { return __bfloat16_as_ushort(x); }
#define FRNN_MMA_TYPE "bf16"
#endif

}  // namespace FRNN_NS
