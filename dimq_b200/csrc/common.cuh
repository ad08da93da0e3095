// Shared device/host helpers of the dimq_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dimq_b200.h"

namespace dimq {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load element i of a tensor whose element type is only known at run time.
__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
  if (dtype == DIMQ_F32) return static_cast<const float*>(p)[i];
  if (dtype == DIMQ_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, int dtype, int64_t i, float v) {
  if (dtype == DIMQ_F32) static_cast<float*>(p)[i] = v;
  else if (dtype == DIMQ_F16) static_cast<__half*>(p)[i] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// clamp(rint(x / s) + z, 0, 15) with an IEEE divide and round-half-even; NaN -> 0.
__device__ __forceinline__ uint32_t quantize_u4(float x, float scale, int zp) {
  float q = rintf(__fdiv_rn(x, scale)) + static_cast<float>(zp);
  q = fminf(fmaxf(q, 0.0f), 15.0f);  // fmaxf(NaN, 0) == 0
  return static_cast<uint32_t>(q);
}

// Index e of a `bits`-wide little-endian bit stream (any alignment).  `nbytes`
// bounds the second byte read.
__device__ __forceinline__ uint32_t get_index(const uint8_t* __restrict__ packed, int64_t e, int bits,
                                              int64_t nbytes) {
  const int64_t bit = e * bits;
  const int64_t byte = bit >> 3;
  const int sh = static_cast<int>(bit & 7);
  uint32_t v = packed[byte];
  if (sh + bits > 8 && byte + 1 < nbytes) v |= static_cast<uint32_t>(packed[byte + 1]) << 8;
  return (v >> sh) & ((1u << bits) - 1u);
}

// erf(x) by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7): one reciprocal, one exp2, six FMAs.
__device__ __forceinline__ float fast_erf(float x) {
  const float z = fabsf(x);
  const float t = __fdividef(1.0f, fmaf(0.3275911f, z, 1.0f));
  float p = fmaf(t, 1.061405429f, -1.453152027f);
  p = fmaf(t, p, 1.421413741f);
  p = fmaf(t, p, -0.284496736f);
  p = fmaf(t, p, 0.254829592f);
  p *= t;
  const float e = __expf(-z * z);
  return copysignf(fmaf(-p, e, 1.0f), x);
}

__device__ __forceinline__ float apply_epilogue(float v, int epilogue) {
  if (epilogue == DIMQ_EPI_RELU) return fmaxf(v, 0.0f);
  if (epilogue == DIMQ_EPI_GELU) return 0.5f * v * (1.0f + fast_erf(v * 0.70710678118654752440f));
  return v;
}

// accumulator (+bias) -> output value.  DIMQ_EPI_ADD_RELU adds the residual before the ReLU; the
// other epilogues apply the activation first and add the residual after it.
__device__ __forceinline__ float finish_value(float v, int epilogue, bool has_res, float res) {
  if (epilogue == DIMQ_EPI_ADD_RELU) return fmaxf(has_res ? v + res : v, 0.0f);
  v = apply_epilogue(v, epilogue);
  return has_res ? v + res : v;
}

inline bool valid_dtype(int d) { return d == DIMQ_F32 || d == DIMQ_F16 || d == DIMQ_BF16; }
inline int dtype_size(int d) { return d == DIMQ_F32 ? 4 : 2; }
inline bool valid_bits(int b) { return b == 1 || b == 2 || b == 3 || b == 4 || b == 8; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DIMQ_OK : static_cast<int>(e);
}

}  // namespace dimq
