// Dense helper of the whole-model harness: (residual add +) LayerNorm over 16-bit rows.
// One warp per row, the row held in registers (8 elements per 16-byte load), statistics in fp32.
// Memory-bound: every element is read once and written once.
#include "common.cuh"

namespace dimq {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxVec = 4;  // 16-byte vectors per lane: rows of up to 32 * 4 * 8 = 1024 elements

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
add_layer_norm_kernel(const T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ gamma,
                      const T* __restrict__ beta, T* __restrict__ x_out, T* __restrict__ h_out, int64_t rows,
                      int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int vecs = cols / 8;  // vectors per row
  float v[kMaxVec][8];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int vi = i * 32 + lane;
    if (vi < vecs) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + row * cols) + vi);
      const T* e = reinterpret_cast<const T*>(&q);
      if (delta != nullptr) {
        const uint4 d = __ldg(reinterpret_cast<const uint4*>(delta + row * cols) + vi);
        const T* de = reinterpret_cast<const T*>(&d);
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          oe[j] = from_float<T>(to_float<T>(e[j]) + to_float<T>(de[j]));  // the sum is stored in T first
          v[i][j] = to_float<T>(oe[j]);
        }
        reinterpret_cast<uint4*>(x_out + row * cols)[vi] = o;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = to_float<T>(e[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[i][j];
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
  const float mean = sum / static_cast<float>(cols);
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    if (i * 32 + lane < vecs) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; sq = fmaf(d, d, sq); }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, off);
  const float rstd = rsqrtf(sq / static_cast<float>(cols) + eps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int vi = i * 32 + lane;
    if (vi < vecs) {
      const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(beta) + vi);
      const T* ge = reinterpret_cast<const T*>(&g);
      const T* be = reinterpret_cast<const T*>(&b);
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) oe[j] = from_float<T>(fmaf((v[i][j] - mean) * rstd, to_float<T>(ge[j]), to_float<T>(be[j])));
      reinterpret_cast<uint4*>(h_out + row * cols)[vi] = o;
    }
  }
}

}  // namespace
}  // namespace dimq

using namespace dimq;

extern "C" int dimq_add_layer_norm(const void* x, const void* delta, const void* gamma, const void* beta,
                                   void* x_out, void* h_out, int64_t rows, int64_t cols, float eps, int dtype,
                                   void* stream) {
  if (rows < 0 || cols <= 0) return DIMQ_ERR_BAD_SIZE;
  if (dtype != DIMQ_BF16 && dtype != DIMQ_F16) return DIMQ_ERR_BAD_DTYPE;
  if (cols % 8 != 0 || cols > 32 * kMaxVec * 8) return DIMQ_ERR_UNSUPPORTED;
  if (rows == 0) return DIMQ_OK;
  if (x == nullptr || gamma == nullptr || beta == nullptr || h_out == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (delta != nullptr && x_out == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (!aligned(x, 16) || !aligned(gamma, 16) || !aligned(beta, 16) || !aligned(h_out, 16) ||
      (delta != nullptr && (!aligned(delta, 16) || !aligned(x_out, 16))))
    return DIMQ_ERR_ALIGNMENT;
  const int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7FFFFFFFll) return DIMQ_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == DIMQ_BF16)
    add_layer_norm_kernel<__nv_bfloat16><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
        static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta),
        static_cast<__nv_bfloat16*>(x_out), static_cast<__nv_bfloat16*>(h_out), rows, static_cast<int>(cols), eps);
  else
    add_layer_norm_kernel<__half><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, st>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(delta), static_cast<const __half*>(gamma),
        static_cast<const __half*>(beta), static_cast<__half*>(x_out), static_cast<__half*>(h_out), rows,
        static_cast<int>(cols), eps);
  return launch_status();
}
