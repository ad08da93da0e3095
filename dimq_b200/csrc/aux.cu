// Dense helper of the whole-model harness: (residual add +) LayerNorm over 16-bit rows.
// One warp per row, the row held in registers (8 elements per 16-byte load), statistics in fp32.
// Memory-bound: every element is read once and written once.
#include <type_traits>
#include "common.cuh"

namespace dimq {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxVec = 4;  // 16-byte vectors per lane: rows of up to 32 * 4 * 8 = 1024 elements

// One warp per row.  The row stays in registers as packed 16-bit vectors (converted again in each of the
// three passes) rather than as floats: the kernel waits on memory latency, so what counts is how many
// warps - bytes in flight - an SM holds (48 with 40 registers per thread; 32 with the float copy).
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 6)
add_layer_norm_kernel(const T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ gamma,
                      const T* __restrict__ beta, T* __restrict__ x_out, T* __restrict__ h_out, int64_t rows,
                      int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int vecs = cols / 8;  // vectors per row
  uint4 q[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int vi = i * 32 + lane;
    if (vi < vecs) q[i] = __ldg(reinterpret_cast<const uint4*>(x + row * cols) + vi);
  }
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int vi = i * 32 + lane;
    if (vi < vecs) {
      T* e = reinterpret_cast<T*>(&q[i]);
      if (delta != nullptr) {
        const uint4 d = __ldg(reinterpret_cast<const uint4*>(delta + row * cols) + vi);
        const T* de = reinterpret_cast<const T*>(&d);
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = from_float<T>(to_float<T>(e[j]) + to_float<T>(de[j]));  // the sum is stored in T first
        reinterpret_cast<uint4*>(x_out + row * cols)[vi] = q[i];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += to_float<T>(e[j]);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
  const float mean = sum / static_cast<float>(cols);
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    if (i * 32 + lane < vecs) {
      const T* e = reinterpret_cast<const T*>(&q[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = to_float<T>(e[j]) - mean; sq = fmaf(d, d, sq); }
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
      const T* e = reinterpret_cast<const T*>(&q[i]);
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) oe[j] = from_float<T>(fmaf((to_float<T>(e[j]) - mean) * rstd, to_float<T>(ge[j]), to_float<T>(be[j])));
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

// ---------------------------------------------------------------------------------------------
// Explicit im2col for convolutions whose channel count does not fit the implicit-GEMM kernel (the
// 3-channel ResNet stem), and a 16-bit NHWC max-pool.  Both are streaming kernels: 16-byte stores,
// consecutive threads write consecutive vectors.
// ---------------------------------------------------------------------------------------------
namespace dimq {
namespace {

constexpr int kAuxThreads = 256;

// cols[(b, oh, ow)][k], k = (kh * KW + kw) * C + c for k < KH*KW*C, zero for the padding columns up
// to kp.  One thread writes 8 consecutive k of one output pixel.
template <typename T>
__global__ void __launch_bounds__(kAuxThreads)
im2col_kernel(const T* __restrict__ x, T* __restrict__ cols, dimq_conv_geom g, int kp) {
  // per column k: (kh * dilation, kw * dilation, c) packed as 8 | 8 | 16 bits, or -1 for a padding
  // column; built once per block so that the element loop has no divisions
  extern __shared__ int col_tbl[];
  const int C = g.in_channels, k_real = g.kernel_h * g.kernel_w * C;
  for (int k = threadIdx.x; k < kp; k += kAuxThreads) {
    int code = -1;
    if (k < k_real) {
      const int c = k % C, tap = k / C;
      code = ((tap / g.kernel_w) * g.dilation_h) | (((tap % g.kernel_w) * g.dilation_w) << 8) | (c << 16);
    }
    col_tbl[k] = code;
  }
  __syncthreads();
  const int vec_per_row = kp / 8;
  const int64_t total = static_cast<int64_t>(g.batch) * g.out_h * g.out_w * vec_per_row;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kAuxThreads + threadIdx.x;
  if (i >= total) return;
  const int v = static_cast<int>(i % vec_per_row);
  const int64_t pix = i / vec_per_row;
  const int ow = static_cast<int>(pix % g.out_w);
  const int oh = static_cast<int>((pix / g.out_w) % g.out_h);
  const int b = static_cast<int>(pix / (static_cast<int64_t>(g.out_w) * g.out_h));
  const int ih0 = oh * g.stride_h - g.pad_h, iw0 = ow * g.stride_w - g.pad_w;
  const T* xb = x + b * g.x_stride[0];
  uint4 out;
  T* o = reinterpret_cast<T*>(&out);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int code = col_tbl[v * 8 + e];
    const int ih = ih0 + (code & 0xFF), iw = iw0 + ((code >> 8) & 0xFF);
    T val = from_float<T>(0.0f);
    if (code >= 0 && ih >= 0 && ih < g.in_h && iw >= 0 && iw < g.in_w)
      val = xb[(code >> 16) * g.x_stride[1] + ih * g.x_stride[2] + iw * g.x_stride[3]];
    o[e] = val;
  }
  reinterpret_cast<uint4*>(cols)[i] = out;
}

// The same matrix through a shared-memory patch, persistent blocks.  Block (kp / 8, pixels per
// chunk); a block walks over output rows (b, oh) and, inside a row, over chunks of pixels: it loads the
// input window of the chunk ([C][KH][win_w], read along w, zeros outside the image), then every
// thread gathers its eight columns from the patch and writes 16 bytes.  Everything that needs a
// division (column -> patch offset, patch element -> (channel, kernel row, column)) is worked out once
// per block / thread, outside the loops.
constexpr int kPatchPerThread = 4;
constexpr int kPixelGroups = 1;  // pixel groups (of blockDim.y pixels) per chunk; more per barrier pair measured slower
template <typename T>
__global__ void __launch_bounds__(kAuxThreads)
im2col_patch_kernel(const T* __restrict__ x, T* __restrict__ cols, dimq_conv_geom g, int kp, int win_w) {
  extern __shared__ int col_tbl[];  // [kp] patch offset of column k (or -1), then the patch
  T* patch = reinterpret_cast<T*>(col_tbl + kp);
  const int C = g.in_channels, KH = g.kernel_h, KW = g.kernel_w, k_real = KH * KW * C;
  const int threads = blockDim.x * blockDim.y;
  const int tid = threadIdx.y * blockDim.x + threadIdx.x;
  for (int k = tid; k < kp; k += threads) {
    int off = -1;
    if (k < k_real) {
      const int c = k % C, tap = k / C;
      off = (c * KH + tap / KW) * win_w + (tap % KW) * g.dilation_w;
    }
    col_tbl[k] = off;
  }
  // this thread's patch elements: idx = tid + i * threads -> (channel, kernel row, column j)
  const int patch_elems = C * KH * win_w;
  int p_dh[kPatchPerThread], p_j[kPatchPerThread];
  int64_t p_off[kPatchPerThread];
#pragma unroll
  for (int i = 0; i < kPatchPerThread; ++i) {
    const int idx = tid + i * threads;
    p_dh[i] = -1;
    p_j[i] = 0;
    p_off[i] = 0;
    if (idx < patch_elems) {
      const int r = idx / win_w, j = idx - r * win_w;
      const int c = r / KH, kh = r - c * KH;
      p_dh[i] = kh * g.dilation_h;
      p_j[i] = j;
      p_off[i] = c * g.x_stride[1] + static_cast<int64_t>(p_dh[i]) * g.x_stride[2] + j * g.x_stride[3];
    }
  }
  const int px = blockDim.y * kPixelGroups, v = threadIdx.x;
  const int vec = kp / 8;
  const int64_t n_rows = static_cast<int64_t>(g.batch) * g.out_h;
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const int b = static_cast<int>(row / g.out_h), oh = static_cast<int>(row - static_cast<int64_t>(b) * g.out_h);
    const int ih0 = oh * g.stride_h - g.pad_h;
    const T* xr = x + static_cast<int64_t>(b) * g.x_stride[0] + static_cast<int64_t>(ih0) * g.x_stride[2];
    for (int ow0 = 0; ow0 < g.out_w; ow0 += px) {
      const int iw0 = ow0 * g.stride_w - g.pad_w;
      __syncthreads();  // the previous chunk's gathers are done (and, the first time, the table is written)
#pragma unroll
      for (int i = 0; i < kPatchPerThread; ++i) {
        if (p_dh[i] >= 0) {
          const int ih = ih0 + p_dh[i], iw = iw0 + p_j[i];
          T val = from_float<T>(0.0f);
          if (ih >= 0 && ih < g.in_h && iw >= 0 && iw < g.in_w) val = xr[p_off[i] + static_cast<int64_t>(iw0) * g.x_stride[3]];
          patch[tid + i * threads] = val;
        }
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < kPixelGroups; ++r) {
        const int pl = threadIdx.y + r * blockDim.y;  // pixel inside the chunk
        const int ow = ow0 + pl;
        if (ow < g.out_w) {
          const int shift = pl * g.stride_w;
          uint4 out;
          T* o = reinterpret_cast<T*>(&out);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int off = col_tbl[v * 8 + e];
            o[e] = off >= 0 ? patch[off + shift] : from_float<T>(0.0f);
          }
          reinterpret_cast<uint4*>(cols)[(row * g.out_w + ow) * vec + v] = out;
        }
      }
    }
  }
}

// y[b][oh][ow][c] = max over the window of x[b][ih][iw][c], NHWC 16-bit, 8 channels per thread.
template <typename T>
__global__ void __launch_bounds__(kAuxThreads)
max_pool_nhwc_kernel(const T* __restrict__ x, T* __restrict__ y, int B, int H, int W, int C, int OH, int OW, int k,
                     int stride, int pad) {
  // grid = (chunks of one image's OH * OW * C / 8 vectors, B): 32-bit index arithmetic only (the kernel was bound
  // by its instruction count - 64-bit divisions per thread - at half the DRAM rate)
  const int cv = C / 8, row_v = OW * cv;
  const int t = static_cast<int>(blockIdx.x) * kAuxThreads + static_cast<int>(threadIdx.x);
  if (t >= OH * row_v) return;
  const int oh = t / row_v, r = t - oh * row_v;
  const int ow = r / cv, c8 = r - ow * cv;
  const int b = static_cast<int>(blockIdx.y);
  // packed 16-bit maxima, two channels per instruction (no conversions); -inf in both halves to start
  using T2 = typename std::conditional<std::is_same<T, __nv_bfloat16>::value, __nv_bfloat162, __half2>::type;
  const uint32_t ninf = std::is_same<T, __nv_bfloat16>::value ? 0xFF80FF80u : 0xFC00FC00u;
  uint32_t m[4] = {ninf, ninf, ninf, ninf};
  const uint4* img = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(b) * H * W * C);   // 32-bit offsets inside an image
  auto take = [&](const uint4& q) {
    const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const T2 r = __hmax2(*reinterpret_cast<const T2*>(&m[e]), *reinterpret_cast<const T2*>(&w4[e]));
      m[e] = *reinterpret_cast<const uint32_t*>(&r);
    }
  };
  if (k == 3) {
    // the usual window: all nine vectors requested before the first maximum (positions outside the image read -inf)
    uint4 q[9];
#pragma unroll
    for (int dy = 0; dy < 3; ++dy) {
      const int ih = oh * stride + dy - pad;
#pragma unroll
      for (int dx = 0; dx < 3; ++dx) {
        const int iw = ow * stride + dx - pad;
        const bool in = static_cast<unsigned>(ih) < static_cast<unsigned>(H) && static_cast<unsigned>(iw) < static_cast<unsigned>(W);
        q[dy * 3 + dx] = in ? __ldg(img + (ih * W + iw) * cv + c8) : make_uint4(ninf, ninf, ninf, ninf);
      }
    }
#pragma unroll
    for (int i = 0; i < 9; ++i) take(q[i]);
  } else {
    for (int dy = 0; dy < k; ++dy) {
      const int ih = oh * stride + dy - pad;
      if (ih < 0 || ih >= H) continue;
      for (int dx = 0; dx < k; ++dx) {
        const int iw = ow * stride + dx - pad;
        if (iw < 0 || iw >= W) continue;
        take(__ldg(img + (ih * W + iw) * cv + c8));
      }
    }
  }
  const uint4 out = make_uint4(m[0], m[1], m[2], m[3]);
  reinterpret_cast<uint4*>(y + ((static_cast<int64_t>(b) * OH + oh) * OW + ow) * C)[c8] = out;
}

}  // namespace
}  // namespace dimq

extern "C" int dimq_im2col(const void* x, int dtype, const dimq_conv_geom* geom, int64_t padded_k, void* cols,
                           void* stream) {
  if (geom == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (dtype != DIMQ_BF16 && dtype != DIMQ_F16) return DIMQ_ERR_BAD_DTYPE;
  dimq_conv_geom g = *geom;
  const int rc = dimq_conv_out_size(&g);
  if (rc != DIMQ_OK) return rc;
  if (g.groups != 1) return DIMQ_ERR_UNSUPPORTED;
  const int64_t k_real = static_cast<int64_t>(g.kernel_h) * g.kernel_w * g.in_channels;
  if (padded_k < k_real || padded_k % 8 != 0 || padded_k > 8192) return DIMQ_ERR_BAD_SIZE;
  if (g.kernel_h * g.dilation_h > 255 || g.kernel_w * g.dilation_w > 255 || g.in_channels > 32767) return DIMQ_ERR_UNSUPPORTED;
  const int64_t total = static_cast<int64_t>(g.batch) * g.out_h * g.out_w * (padded_k / 8);
  if (total == 0) return DIMQ_OK;
  if (x == nullptr || cols == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (!aligned(cols, 16)) return DIMQ_ERR_ALIGNMENT;
  const int64_t blocks = (total + kAuxThreads - 1) / kAuxThreads;
  if (blocks > 0x7FFFFFFFll) return DIMQ_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    // shared-memory patch variant when the launch geometry can carry the output position and the
    // window of a block's pixels is small
    const int vec = static_cast<int>(padded_k / 8);
    if (vec <= kAuxThreads) {
      const int px = kAuxThreads / vec;
      const int64_t win_w = static_cast<int64_t>(px * kPixelGroups - 1) * g.stride_w + static_cast<int64_t>(g.kernel_w - 1) * g.dilation_w + 1;
      const int64_t patch_elems = static_cast<int64_t>(g.in_channels) * g.kernel_h * win_w;
      if (patch_elems <= static_cast<int64_t>(kPatchPerThread) * vec * px) {
        const int64_t n_rows = static_cast<int64_t>(g.batch) * g.out_h;
        const int64_t want = static_cast<int64_t>(kNumSMs) * 8;
        const dim3 block(vec, px), grid(static_cast<unsigned>(n_rows < want ? n_rows : want));
        const size_t smem = padded_k * sizeof(int) + static_cast<size_t>(patch_elems) * 2;
        if (dtype == DIMQ_BF16)
          im2col_patch_kernel<__nv_bfloat16><<<grid, block, smem, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                                        static_cast<__nv_bfloat16*>(cols), g,
                                                                        static_cast<int>(padded_k), static_cast<int>(win_w));
        else
          im2col_patch_kernel<__half><<<grid, block, smem, st>>>(static_cast<const __half*>(x),
                                                                 static_cast<__half*>(cols), g,
                                                                 static_cast<int>(padded_k), static_cast<int>(win_w));
        return launch_status();
      }
    }
  }
  if (dtype == DIMQ_BF16)
    im2col_kernel<__nv_bfloat16><<<(unsigned)blocks, kAuxThreads, padded_k * sizeof(int), st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(cols), g, static_cast<int>(padded_k));
  else
    im2col_kernel<__half><<<(unsigned)blocks, kAuxThreads, padded_k * sizeof(int), st>>>(static_cast<const __half*>(x),
                                                                   static_cast<__half*>(cols), g,
                                                                   static_cast<int>(padded_k));
  return launch_status();
}

namespace dimq {
namespace {

// y[b][p][c] = T(x[b][c][p]) for the 3 channels of an image batch (p = pixel index): NCHW fp32 / 16-bit in,
// NHWC 16-bit out.  One thread = 8 consecutive pixels: two 16-byte loads per channel plane (one for 16-bit
// input), three 16-byte stores of the 24 interleaved values.
template <typename TI, typename TO>
__global__ void __launch_bounds__(kAuxThreads)
images_to_nhwc_kernel(const TI* __restrict__ x, TO* __restrict__ y, int64_t batch, int64_t pixels) {
  const int64_t per_image = pixels / 8;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kAuxThreads + threadIdx.x;
  if (i >= batch * per_image) return;
  const int64_t b = i / per_image, p0 = (i - b * per_image) * 8;
  float v[3][8];
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const TI* src = x + (b * 3 + c) * pixels + p0;
    if constexpr (sizeof(TI) == 4) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(src));
      const float4 d = __ldg(reinterpret_cast<const float4*>(src) + 1);
      v[c][0] = a.x; v[c][1] = a.y; v[c][2] = a.z; v[c][3] = a.w; v[c][4] = d.x; v[c][5] = d.y; v[c][6] = d.z; v[c][7] = d.w;
    } else {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(src));
      const TI* h = reinterpret_cast<const TI*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[c][j] = to_float<TI>(h[j]);
    }
  }
  __align__(16) TO o[24];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int c = 0; c < 3; ++c) o[3 * j + c] = from_float<TO>(v[c][j]);
  uint4* dst = reinterpret_cast<uint4*>(y + (b * pixels + p0) * 3);
#pragma unroll
  for (int k = 0; k < 3; ++k) dst[k] = reinterpret_cast<const uint4*>(o)[k];
}

}  // namespace
}  // namespace dimq

extern "C" int dimq_images_to_nhwc(const void* x, int x_dtype, void* y, int y_dtype, int64_t batch, int64_t height,
                                   int64_t width, void* stream) {
  if (!valid_dtype(x_dtype) || (y_dtype != DIMQ_BF16 && y_dtype != DIMQ_F16)) return DIMQ_ERR_BAD_DTYPE;
  if (batch < 0 || height <= 0 || width <= 0) return DIMQ_ERR_BAD_SIZE;
  const int64_t pixels = height * width;
  if (pixels % 8 != 0) return DIMQ_ERR_UNSUPPORTED;
  if (batch == 0) return DIMQ_OK;
  if (x == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (!aligned(x, 16) || !aligned(y, 16)) return DIMQ_ERR_ALIGNMENT;
  const int64_t total = batch * (pixels / 8);
  const int64_t blocks = (total + kAuxThreads - 1) / kAuxThreads;
  if (blocks > 0x7FFFFFFFll) return DIMQ_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(blocks);
#define DIMQ_IMG(TI, TO) images_to_nhwc_kernel<TI, TO><<<grid, kAuxThreads, 0, st>>>(static_cast<const TI*>(x), static_cast<TO*>(y), batch, pixels)
  if (y_dtype == DIMQ_BF16) {
    if (x_dtype == DIMQ_F32) DIMQ_IMG(float, __nv_bfloat16);
    else if (x_dtype == DIMQ_F16) DIMQ_IMG(__half, __nv_bfloat16);
    else DIMQ_IMG(__nv_bfloat16, __nv_bfloat16);
  } else {
    if (x_dtype == DIMQ_F32) DIMQ_IMG(float, __half);
    else if (x_dtype == DIMQ_F16) DIMQ_IMG(__half, __half);
    else DIMQ_IMG(__nv_bfloat16, __half);
  }
#undef DIMQ_IMG
  return launch_status();
}

extern "C" int dimq_max_pool_nhwc(const void* x, void* y, int dtype, int64_t batch, int64_t height, int64_t width,
                                  int64_t channels, int kernel, int stride, int pad, void* stream) {
  if (dtype != DIMQ_BF16 && dtype != DIMQ_F16) return DIMQ_ERR_BAD_DTYPE;
  if (batch < 0 || height <= 0 || width <= 0 || channels <= 0 || kernel <= 0 || stride <= 0 || pad < 0 || 2 * pad > kernel)
    return DIMQ_ERR_BAD_SIZE;
  if (channels % 8 != 0) return DIMQ_ERR_UNSUPPORTED;
  const int64_t oh = (height + 2 * pad - kernel) / stride + 1, ow = (width + 2 * pad - kernel) / stride + 1;
  if (oh <= 0 || ow <= 0) return DIMQ_ERR_BAD_SHAPE;
  const int64_t total = batch * oh * ow * (channels / 8);
  if (total == 0) return DIMQ_OK;
  if (x == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (!aligned(x, 16) || !aligned(y, 16)) return DIMQ_ERR_ALIGNMENT;
  const int64_t per_image = oh * ow * (channels / 8);
  if (per_image > 0x7FFFFFFFll - kAuxThreads || height * width * channels > 0x7FFFFFFFll || batch > 65535) return DIMQ_ERR_TOO_LARGE;
  const dim3 blocks(static_cast<unsigned>((per_image + kAuxThreads - 1) / kAuxThreads), static_cast<unsigned>(batch));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == DIMQ_BF16)
    max_pool_nhwc_kernel<__nv_bfloat16><<<blocks, kAuxThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), (int)batch, (int)height, (int)width,
        (int)channels, (int)oh, (int)ow, kernel, stride, pad);
  else
    max_pool_nhwc_kernel<__half><<<blocks, kAuxThreads, 0, st>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), (int)batch, (int)height, (int)width, (int)channels,
        (int)oh, (int)ow, kernel, stride, pad);
  return launch_status();
}
