// Exact fp32 SIMT kernels: the W4A4 product-table GEMM / direct convolution with
// the reference's semantics, and weight-only GEMM / convolution for any shape,
// bit width, alignment and codebook grouping.  They are the correctness path for
// shapes the streaming and tcgen05 kernels do not take; accumulation is fp32 in
// ascending k (GEMM) or (ci, kh, kw) order (conv), like the reference kernels.
#include "common.cuh"

namespace dimq {
namespace {

constexpr int kTileM = 32;
constexpr int kTileN = 32;
constexpr int kTileK = 64;
constexpr int kThreads = 256;

// ---- W4A4 GEMM over the product table -------------------------------------
// Block = 32(m) x 32(n) outputs; thread (tx = n, ty) owns rows ty, ty+8, ty+16, ty+24.
// Activations are quantised once per tile (not once per output as in the
// reference kernel), weights nibbles staged through shared memory.
__global__ void __launch_bounds__(kThreads)
linear_lut_a4_kernel(const void* __restrict__ x, int x_dtype, const uint8_t* __restrict__ packed_w,
                     const void* __restrict__ codebook, int cb_dtype, float scale, int zp,
                     const void* __restrict__ bias, int bias_dtype, float* __restrict__ y, int64_t M, int64_t N,
                     int64_t K) {
  __shared__ float table_s[256];
  __shared__ uint8_t qa_s[kTileM][kTileK];
  __shared__ uint8_t wi_s[kTileN][kTileK + 4];
  const int tid = threadIdx.x;
  {
    const float c = load_as_float(codebook, cb_dtype, tid >> 4);
    const float a_hat = __fmul_rn(scale, static_cast<float>((tid & 15) - zp));
    table_s[tid] = __fmul_rn(c, a_hat);
  }
  const int tx = tid & 31, ty = tid >> 5;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTileM;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTileN;
  const int64_t wbytes = (N * K + 1) / 2;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int64_t k0 = 0; k0 < K; k0 += kTileK) {
    __syncthreads();
    for (int i = tid; i < kTileM * kTileK; i += kThreads) {
      const int r = i / kTileK, c = i % kTileK;
      const int64_t m = m0 + r, k = k0 + c;
      qa_s[r][c] = (m < M && k < K) ? static_cast<uint8_t>(quantize_u4(load_as_float(x, x_dtype, m * K + k), scale, zp)) : 0;
      const int64_t n = n0 + r;
      wi_s[r][c] = (n < N && k < K) ? static_cast<uint8_t>(get_index(packed_w, n * K + k, 4, wbytes)) : 0;
    }
    __syncthreads();
    const int kmax = static_cast<int>(K - k0 < kTileK ? K - k0 : kTileK);
    for (int k = 0; k < kmax; ++k) {
      const int wrow = static_cast<int>(wi_s[tx][k]) * 16;
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += table_s[wrow + qa_s[ty + 8 * j][k]];
    }
  }
  const int64_t n = n0 + tx;
  if (n >= N) return;
  const float b = bias != nullptr ? load_as_float(bias, bias_dtype, n) : 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t m = m0 + ty + 8 * j;
    if (m < M) y[m * N + n] = bias != nullptr ? acc[j] + b : acc[j];
  }
}

// ---- weight-only GEMM -------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
linear_wq_generic_kernel(const void* __restrict__ x, int x_dtype, dimq_wq_weight w, const void* __restrict__ bias,
                         int bias_dtype, const void* __restrict__ residual, void* __restrict__ y, int y_dtype,
                         int64_t M, int64_t N, int64_t K, int epilogue) {
  __shared__ float xs[kTileM][kTileK];
  __shared__ float ws[kTileN][kTileK + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 31, ty = tid >> 5;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTileM;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTileN;
  const int64_t wbytes = (N * K * w.bits + 7) / 8;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int64_t k0 = 0; k0 < K; k0 += kTileK) {
    __syncthreads();
    for (int i = tid; i < kTileM * kTileK; i += kThreads) {
      const int r = i / kTileK, c = i % kTileK;
      const int64_t m = m0 + r, k = k0 + c;
      xs[r][c] = (m < M && k < K) ? load_as_float(x, x_dtype, m * K + k) : 0.0f;
      const int64_t n = n0 + r;
      float wv = 0.0f;
      if (n < N && k < K) {
        const uint32_t idx = get_index(w.packed, n * K + k, w.bits, wbytes);
        wv = load_as_float(w.codebooks, w.cb_dtype, (n / w.group_rows) * w.entries + idx);
      }
      ws[r][c] = wv;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kTileK; ++k) {
      const float wv = ws[tx][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = fmaf(xs[ty + 8 * j][k], wv, acc[j]);
    }
  }
  const int64_t n = n0 + tx;
  if (n >= N) return;
  const float b = bias != nullptr ? load_as_float(bias, bias_dtype, n) : 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t m = m0 + ty + 8 * j;
    if (m < M) {
      const float res = residual != nullptr ? load_as_float(residual, y_dtype, m * N + n) : 0.0f;
      store_from_float(y, y_dtype, m * N + n, finish_value(acc[j] + b, epilogue, residual != nullptr, res));
    }
  }
}

// ---- direct convolution (A4 over the product table, or weight-only) -----------
// One thread per output element; consecutive threads walk the innermost
// (unit-stride) axis of y so stores coalesce for both NCHW and NHWC storage.
template <bool A4>
__global__ void __launch_bounds__(kThreads)
conv2d_direct_kernel(const void* __restrict__ x, int x_dtype, dimq_wq_weight w, float scale, int zp,
                     const void* __restrict__ bias, int bias_dtype, const void* __restrict__ residual,
                     void* __restrict__ y, int y_dtype, dimq_conv_geom g, int epilogue, int channels_inner) {
  __shared__ float table_s[256];
  if (A4) {
    const int tid = threadIdx.x;
    const float c = load_as_float(w.codebooks, w.cb_dtype, tid >> 4);
    table_s[tid] = __fmul_rn(c, __fmul_rn(scale, static_cast<float>((tid & 15) - zp)));
    __syncthreads();
  }
  const int64_t total = static_cast<int64_t>(g.batch) * g.out_channels * g.out_h * g.out_w;
  const int64_t lin = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (lin >= total) return;
  int ow, oh, co, b;
  if (channels_inner) {  // (b, oh, ow, co) order
    co = static_cast<int>(lin % g.out_channels);
    ow = static_cast<int>((lin / g.out_channels) % g.out_w);
    oh = static_cast<int>((lin / (static_cast<int64_t>(g.out_channels) * g.out_w)) % g.out_h);
    b = static_cast<int>(lin / (static_cast<int64_t>(g.out_channels) * g.out_w * g.out_h));
  } else {               // (b, co, oh, ow) order, as in the reference kernel
    ow = static_cast<int>(lin % g.out_w);
    oh = static_cast<int>((lin / g.out_w) % g.out_h);
    co = static_cast<int>((lin / (static_cast<int64_t>(g.out_w) * g.out_h)) % g.out_channels);
    b = static_cast<int>(lin / (static_cast<int64_t>(g.out_w) * g.out_h * g.out_channels));
  }
  const int ocg = g.out_channels / g.groups;
  const int grp = co / ocg;
  const int icg = g.in_channels_per_group;
  const int64_t wnumel = static_cast<int64_t>(g.out_channels) * icg * g.kernel_h * g.kernel_w;
  const int64_t wbytes = (wnumel * w.bits + 7) / 8;
  const int64_t wbase = static_cast<int64_t>(co) * icg * g.kernel_h * g.kernel_w;
  const int64_t cb_off = (co / w.group_rows) * w.entries;
  float acc = 0.0f;
  for (int cg = 0; cg < icg; ++cg) {
    const int ci = grp * icg + cg;
    for (int kh = 0; kh < g.kernel_h; ++kh) {
      const int ih = oh * g.stride_h + kh * g.dilation_h - g.pad_h;
      if (ih < 0 || ih >= g.in_h) continue;
      for (int kw = 0; kw < g.kernel_w; ++kw) {
        const int iw = ow * g.stride_w + kw * g.dilation_w - g.pad_w;
        if (iw < 0 || iw >= g.in_w) continue;
        const float xv = load_as_float(
            x, x_dtype, b * g.x_stride[0] + ci * g.x_stride[1] + ih * g.x_stride[2] + iw * g.x_stride[3]);
        const uint32_t wi =
            get_index(w.packed, wbase + (static_cast<int64_t>(cg) * g.kernel_h + kh) * g.kernel_w + kw, w.bits, wbytes);
        if (A4) acc += table_s[wi * 16 + quantize_u4(xv, scale, zp)];
        else acc = fmaf(xv, load_as_float(w.codebooks, w.cb_dtype, cb_off + wi), acc);
      }
    }
  }
  if (bias != nullptr) acc += load_as_float(bias, bias_dtype, co);
  const int64_t yo = b * g.y_stride[0] + co * g.y_stride[1] + oh * g.y_stride[2] + ow * g.y_stride[3];
  if (!A4) {
    const float res = residual != nullptr ? load_as_float(residual, y_dtype, yo) : 0.0f;
    acc = finish_value(acc, epilogue, residual != nullptr, res);
  }
  store_from_float(y, y_dtype, yo, acc);
}

// kcrs -> khwc re-ordering of a packed index stream: 8 output indices (= `bits` output bytes) per thread.
__global__ void __launch_bounds__(kThreads)
conv_prepack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int bits, int64_t oc, int64_t icg,
                    int64_t kh, int64_t kw) {
  const int64_t n = oc * icg * kh * kw;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t base = t * 8;
  if (base >= n) return;
  const int64_t src_bytes = (n * bits + 7) / 8;
  unsigned long long stream = 0ull;
  for (int i = 0; i < 8; ++i) {
    const int64_t o = base + i;              // position in [oc][kh][kw][ci]
    if (o >= n) break;
    const int64_t ci = o % icg;
    const int64_t tap = (o / icg) % (kh * kw);
    const int64_t co = o / (icg * kh * kw);
    const int64_t e = (co * icg + ci) * (kh * kw) + tap;   // position in [oc][ci][kh][kw]
    stream |= static_cast<unsigned long long>(get_index(src, e, bits, src_bytes)) << (i * bits);
  }
  const int64_t off = t * bits;
  for (int b = 0; b < bits; ++b)
    if (off + b < src_bytes) dst[off + b] = static_cast<uint8_t>(stream >> (8 * b));
}

}  // namespace

int check_wq_weight(const dimq_wq_weight* w, int64_t out_rows) {
  if (w == nullptr || w->packed == nullptr || w->codebooks == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (!(w->bits == 2 || w->bits == 3 || w->bits == 4 || w->bits == 8)) return DIMQ_ERR_BAD_BITS;
  if (!valid_dtype(w->cb_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (w->entries <= 0 || w->entries > (1 << w->bits)) return DIMQ_ERR_BAD_SIZE;
  if (w->groups <= 0 || w->group_rows <= 0) return DIMQ_ERR_BAD_SIZE;
  if (w->groups * w->group_rows < out_rows) return DIMQ_ERR_BAD_SHAPE;
  return DIMQ_OK;
}

int launch_linear_wq_generic(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                             const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                             int epilogue, cudaStream_t st) {
  dim3 grid((unsigned)((N + kTileN - 1) / kTileN), (unsigned)((M + kTileM - 1) / kTileM));
  if (grid.y > 65535) return DIMQ_ERR_TOO_LARGE;
  linear_wq_generic_kernel<<<grid, kThreads, 0, st>>>(x, x_dtype, *w, bias, bias_dtype, residual, y, y_dtype, M, N,
                                                     K, epilogue);
  return launch_status();
}

int launch_conv2d_direct(bool a4, const void* x, int x_dtype, const dimq_wq_weight* w, float scale, int zp,
                         const void* bias, int bias_dtype, const void* residual, void* y, int y_dtype,
                         const dimq_conv_geom* g, int epilogue, cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(g->batch) * g->out_channels * g->out_h * g->out_w;
  if (total == 0) return DIMQ_OK;
  const int64_t blocks = (total + kThreads - 1) / kThreads;
  if (blocks > 0x7FFFFFFFll) return DIMQ_ERR_TOO_LARGE;
  const int channels_inner = g->y_stride[1] == 1 && g->out_channels > 1;
  if (a4)
    conv2d_direct_kernel<true><<<(unsigned)blocks, kThreads, 0, st>>>(x, x_dtype, *w, scale, zp, bias, bias_dtype,
                                                                      residual, y, y_dtype, *g, epilogue,
                                                                      channels_inner);
  else
    conv2d_direct_kernel<false><<<(unsigned)blocks, kThreads, 0, st>>>(x, x_dtype, *w, scale, zp, bias, bias_dtype,
                                                                       residual, y, y_dtype, *g, epilogue,
                                                                       channels_inner);
  return launch_status();
}

}  // namespace dimq

using namespace dimq;

extern "C" int dimq_conv_prepack(const uint8_t* packed_kcrs, int bits, int64_t out_channels,
                                 int64_t in_channels_per_group, int64_t kernel_h, int64_t kernel_w,
                                 uint8_t* packed_khwc, void* stream) {
  if (!(bits == 2 || bits == 3 || bits == 4 || bits == 8)) return DIMQ_ERR_BAD_BITS;
  if (out_channels <= 0 || in_channels_per_group <= 0 || kernel_h <= 0 || kernel_w <= 0) return DIMQ_ERR_BAD_SIZE;
  if (packed_kcrs == nullptr || packed_khwc == nullptr) return DIMQ_ERR_NULL_POINTER;
  const int64_t n = out_channels * in_channels_per_group * kernel_h * kernel_w;
  const int64_t blocks = ((n + 7) / 8 + kThreads - 1) / kThreads;
  if (blocks > 0x7FFFFFFFll) return DIMQ_ERR_TOO_LARGE;
  conv_prepack_kernel<<<(unsigned)blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      packed_kcrs, packed_khwc, bits, out_channels, in_channels_per_group, kernel_h, kernel_w);
  return launch_status();
}

extern "C" int dimq_conv_out_size(dimq_conv_geom* g) {
  if (g == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (g->batch < 0 || g->in_channels <= 0 || g->in_h < 0 || g->in_w < 0) return DIMQ_ERR_BAD_SIZE;
  if (g->out_channels <= 0 || g->in_channels_per_group <= 0 || g->kernel_h <= 0 || g->kernel_w <= 0)
    return DIMQ_ERR_BAD_SIZE;
  if (g->stride_h <= 0 || g->stride_w <= 0 || g->dilation_h <= 0 || g->dilation_w <= 0 || g->groups <= 0)
    return DIMQ_ERR_BAD_SIZE;
  if (g->pad_h < 0 || g->pad_w < 0) return DIMQ_ERR_BAD_SIZE;
  if (g->in_channels != g->in_channels_per_group * g->groups) return DIMQ_ERR_BAD_SHAPE;
  if (g->out_channels % g->groups != 0) return DIMQ_ERR_BAD_SHAPE;
  // a dilated kernel larger than the padded input has no output position
  const int nh = g->in_h + 2 * g->pad_h - g->dilation_h * (g->kernel_h - 1) - 1;
  const int nw = g->in_w + 2 * g->pad_w - g->dilation_w * (g->kernel_w - 1) - 1;
  if (nh < 0 || nw < 0) return DIMQ_ERR_BAD_SHAPE;
  g->out_h = nh / g->stride_h + 1;
  g->out_w = nw / g->stride_w + 1;
  return DIMQ_OK;
}

extern "C" int dimq_linear_lut(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook,
                               int cb_dtype, float act_scale, int act_zp, const void* bias, int bias_dtype,
                               float* y, int64_t M, int64_t N, int64_t K, void* stream) {
  if (M < 0 || N <= 0 || K <= 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(x_dtype) || !valid_dtype(cb_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (!(act_scale > 0.0f) || act_zp < 0 || act_zp > 15) return DIMQ_ERR_BAD_QPARAMS;
  if (M == 0) return DIMQ_OK;
  if (x == nullptr || packed_w == nullptr || codebook == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  dim3 grid((unsigned)((N + kTileN - 1) / kTileN), (unsigned)((M + kTileM - 1) / kTileM));
  if (grid.y > 65535) return DIMQ_ERR_TOO_LARGE;
  linear_lut_a4_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      x, x_dtype, packed_w, codebook, cb_dtype, act_scale, act_zp, bias, bias_dtype, y, M, N, K);
  return launch_status();
}

extern "C" int dimq_conv2d_lut(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook,
                               int cb_dtype, float act_scale, int act_zp, const void* bias, int bias_dtype,
                               float* y, const dimq_conv_geom* geom, void* stream) {
  if (geom == nullptr) return DIMQ_ERR_NULL_POINTER;
  dimq_conv_geom g = *geom;
  const int rc = dimq_conv_out_size(&g);
  if (rc != DIMQ_OK) return rc;
  if (g.out_h != geom->out_h || g.out_w != geom->out_w) return DIMQ_ERR_BAD_SHAPE;
  if (!valid_dtype(x_dtype) || !valid_dtype(cb_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (!(act_scale > 0.0f) || act_zp < 0 || act_zp > 15) return DIMQ_ERR_BAD_QPARAMS;
  if (static_cast<int64_t>(g.batch) * g.out_channels * g.out_h * g.out_w == 0) return DIMQ_OK;
  if (x == nullptr || packed_w == nullptr || codebook == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  dimq_wq_weight w;
  w.packed = packed_w;
  w.bits = 4;
  w.codebooks = codebook;
  w.cb_dtype = cb_dtype;
  w.entries = 16;
  w.groups = 1;
  w.group_rows = g.out_channels;
  w.packed_khwc = nullptr;
  return launch_conv2d_direct(true, x, x_dtype, &w, act_scale, act_zp, bias, bias_dtype, nullptr, y, DIMQ_F32, &g,
                              DIMQ_EPI_NONE, static_cast<cudaStream_t>(stream));
}
