// W4A4 product-table linear and convolution on the tensor cores.
//
// The reference's lookup  y = bias + sum_k P[w_idx][a_idx],  P[w][a] = C[w] * (s * (a - z))
// (dimq_cuda_backend/csrc/dimq_gemm_lut.cu:14-56, dimq_conv2d_lut.cu:14-88) factors as
//     y = bias + sum_k (s * C[w_idx]) * (a_idx - z).
// (a - z) is an integer in [-15, 15]: exact in bf16.  s * C[w] goes through the weight-only kernel's
// hi + lo pair of bf16 values (about 2^-17 relative), so the result differs from the table lookup only
// by that operand rounding and the order of the fp32 accumulation.  Two launches:
//   1. centre_quantize_kernel: a = clamp(rint(x / s) + z, 0, 15) exactly as the reference's quantiser
//      (csrc/dimq_pack.cu:42-50), written as bf16 (a - z); thread block 0 also writes the 16 scaled
//      codewords (fp32);
//   2. the tcgen05 weight-only GEMM / implicit-GEMM convolution over those operands.
// Both need caller-owned scratch: this library allocates nothing.
#include "common.cuh"

namespace dimq {
bool tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K);
int launch_linear_wq_tc(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                        const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                        int precision, cudaStream_t st, void* workspace = nullptr, int64_t workspace_bytes = 0);
bool conv_tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, int y_dtype);
int launch_conv2d_wq_tc(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                        const void* residual, void* y, int y_dtype, const dimq_conv_geom* g, int epilogue,
                        cudaStream_t st);

namespace {

constexpr int kThreads = 256;
constexpr int64_t kCodebookBytes = 256;  // 16 fp32 codewords, padded so the next region stays 256-byte aligned

inline int64_t round_up_256(int64_t v) { return (v + 255) / 256 * 256; }

template <typename T>
__global__ void __launch_bounds__(kThreads)
centre_quantize_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out, int64_t n, float scale, int zp,
                       int vec_ok, const void* __restrict__ codebook, int cb_dtype, float* __restrict__ scaled_cb) {
  if (scaled_cb != nullptr && blockIdx.x == 0 && threadIdx.x < 16)
    scaled_cb[threadIdx.x] = __fmul_rn(scale, load_as_float(codebook, cb_dtype, threadIdx.x));
  const int64_t base = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) * 8;
  if (base >= n) return;
  if (vec_ok && base + 8 <= n) {
    float f[8];
    if constexpr (sizeof(T) == 4) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(x + base));
      const float4 b = __ldg(reinterpret_cast<const float4*>(x + base) + 1);
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + base));
      const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = to_float<T>(h[i]);
    }
    __align__(16) __nv_bfloat16 o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      o[i] = __float2bfloat16(static_cast<float>(static_cast<int>(quantize_u4(f[i], scale, zp)) - zp));
    *reinterpret_cast<uint4*>(out + base) = *reinterpret_cast<const uint4*>(o);
  } else {
    for (int i = 0; i < 8 && base + i < n; ++i)
      out[base + i] =
          __float2bfloat16(static_cast<float>(static_cast<int>(quantize_u4(to_float<T>(x[base + i]), scale, zp)) - zp));
  }
}

int launch_centre_quantize(const void* x, int x_dtype, int64_t n, float scale, int zp, const void* codebook,
                           int cb_dtype, float* scaled_cb, __nv_bfloat16* out, cudaStream_t st) {
  const int64_t blocks = ((n + 7) / 8 + kThreads - 1) / kThreads;
  if (blocks > 0x7FFFFFFFll) return DIMQ_ERR_TOO_LARGE;
  const int vec_ok = aligned(x, 16) && aligned(out, 16);
  const unsigned grid = static_cast<unsigned>(blocks);
  if (x_dtype == DIMQ_F32)
    centre_quantize_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<const float*>(x), out, n, scale, zp, vec_ok,
                                                             codebook, cb_dtype, scaled_cb);
  else if (x_dtype == DIMQ_F16)
    centre_quantize_kernel<__half><<<grid, kThreads, 0, st>>>(static_cast<const __half*>(x), out, n, scale, zp,
                                                              vec_ok, codebook, cb_dtype, scaled_cb);
  else
    centre_quantize_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), out, n,
                                                                     scale, zp, vec_ok, codebook, cb_dtype, scaled_cb);
  return launch_status();
}

int check_a4_args(int x_dtype, int cb_dtype, const void* bias, int bias_dtype, float act_scale, int act_zp) {
  if (!valid_dtype(x_dtype) || !valid_dtype(cb_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (!(act_scale > 0.0f) || act_zp < 0 || act_zp > 15) return DIMQ_ERR_BAD_QPARAMS;
  return DIMQ_OK;
}

}  // namespace
}  // namespace dimq

using namespace dimq;

extern "C" int dimq_centre_quantize_u4(const void* x, int x_dtype, int64_t numel, float act_scale, int act_zp,
                                       void* codes_bf16, void* stream) {
  if (numel < 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(x_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (!(act_scale > 0.0f) || act_zp < 0 || act_zp > 15) return DIMQ_ERR_BAD_QPARAMS;
  if (numel == 0) return DIMQ_OK;
  if (x == nullptr || codes_bf16 == nullptr) return DIMQ_ERR_NULL_POINTER;
  return launch_centre_quantize(x, x_dtype, numel, act_scale, act_zp, nullptr, DIMQ_F32, nullptr,
                                static_cast<__nv_bfloat16*>(codes_bf16), static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_a4_workspace_bytes(int64_t x_numel, int64_t conv_weight_numel, int64_t* bytes) {
  if (bytes == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (x_numel < 0 || conv_weight_numel < 0) return DIMQ_ERR_BAD_SIZE;
  *bytes = kCodebookBytes + round_up_256(x_numel * 2) + round_up_256((conv_weight_numel + 1) / 2);
  return DIMQ_OK;
}

extern "C" int dimq_linear_lut_tc(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook,
                                  int cb_dtype, float act_scale, int act_zp, const void* bias, int bias_dtype,
                                  float* y, int64_t M, int64_t N, int64_t K, void* workspace,
                                  int64_t workspace_bytes, void* stream) {
  if (M < 0 || N <= 0 || K <= 0) return DIMQ_ERR_BAD_SIZE;
  int rc = check_a4_args(x_dtype, cb_dtype, bias, bias_dtype, act_scale, act_zp);
  if (rc != DIMQ_OK) return rc;
  if (M == 0) return DIMQ_OK;
  if (x == nullptr || packed_w == nullptr || codebook == nullptr || y == nullptr || workspace == nullptr)
    return DIMQ_ERR_NULL_POINTER;
  if (!aligned(workspace, 256)) return DIMQ_ERR_ALIGNMENT;
  int64_t need = 0;
  dimq_a4_workspace_bytes(M * K, 0, &need);
  if (workspace_bytes < need) return DIMQ_ERR_SCRATCH_TOO_SMALL;
  float* scaled_cb = static_cast<float*>(workspace);
  __nv_bfloat16* xq = reinterpret_cast<__nv_bfloat16*>(static_cast<unsigned char*>(workspace) + kCodebookBytes);
  dimq_wq_weight w{packed_w, 4, scaled_cb, DIMQ_F32, 16, 1, N, nullptr};
  if (!tc_supported(xq, DIMQ_BF16, &w, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = launch_centre_quantize(x, x_dtype, M * K, act_scale, act_zp, codebook, cb_dtype, scaled_cb, xq, st);
  if (rc != DIMQ_OK) return rc;
  return launch_linear_wq_tc(xq, DIMQ_BF16, &w, bias, bias_dtype, nullptr, y, DIMQ_F32, M, N, K, DIMQ_EPI_NONE, 0, st);
}

extern "C" int dimq_conv2d_lut_tc(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook,
                                  int cb_dtype, float act_scale, int act_zp, const void* bias, int bias_dtype,
                                  float* y, const dimq_conv_geom* geom, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
  if (geom == nullptr) return DIMQ_ERR_NULL_POINTER;
  dimq_conv_geom g = *geom;
  int rc = dimq_conv_out_size(&g);
  if (rc != DIMQ_OK) return rc;
  if (g.out_h != geom->out_h || g.out_w != geom->out_w) return DIMQ_ERR_BAD_SHAPE;
  rc = check_a4_args(x_dtype, cb_dtype, bias, bias_dtype, act_scale, act_zp);
  if (rc != DIMQ_OK) return rc;
  if (static_cast<int64_t>(g.batch) * g.out_channels * g.out_h * g.out_w == 0) return DIMQ_OK;
  if (x == nullptr || packed_w == nullptr || codebook == nullptr || y == nullptr || workspace == nullptr)
    return DIMQ_ERR_NULL_POINTER;
  if (!aligned(workspace, 256)) return DIMQ_ERR_ALIGNMENT;
  const int64_t x_numel = static_cast<int64_t>(g.batch) * g.in_channels * g.in_h * g.in_w;
  const int64_t w_numel = static_cast<int64_t>(g.out_channels) * g.in_channels_per_group * g.kernel_h * g.kernel_w;
  int64_t need = 0;
  dimq_a4_workspace_bytes(x_numel, w_numel, &need);
  if (workspace_bytes < need) return DIMQ_ERR_SCRATCH_TOO_SMALL;
  unsigned char* base = static_cast<unsigned char*>(workspace);
  float* scaled_cb = reinterpret_cast<float*>(base);
  __nv_bfloat16* xq = reinterpret_cast<__nv_bfloat16*>(base + kCodebookBytes);
  uint8_t* khwc = base + kCodebookBytes + round_up_256(x_numel * 2);
  dimq_wq_weight w{packed_w, 4, scaled_cb, DIMQ_F32, 16, 1, g.out_channels, khwc};
  // the quantised copy keeps the storage order of x, which must be channels_last (checked here through
  // the strides in the geometry)
  if (!conv_tc_supported(xq, DIMQ_BF16, &w, &g, DIMQ_F32)) return DIMQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = dimq_conv_prepack(packed_w, 4, g.out_channels, g.in_channels_per_group, g.kernel_h, g.kernel_w, khwc, stream);
  if (rc != DIMQ_OK) return rc;
  rc = launch_centre_quantize(x, x_dtype, x_numel, act_scale, act_zp, codebook, cb_dtype, scaled_cb, xq, st);
  if (rc != DIMQ_OK) return rc;
  return launch_conv2d_wq_tc(xq, DIMQ_BF16, &w, bias, bias_dtype, nullptr, y, DIMQ_F32, &g, DIMQ_EPI_NONE, st);
}
