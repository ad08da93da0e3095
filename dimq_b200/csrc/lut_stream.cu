// Small-M weight-only LUT GEMM (the HBM-bound regime, M <= 8).
//
// One warp owns one output row n at a time and streams that row's packed
// indices from HBM exactly once: lane l loads unit (it*32 + l) of 32 indices with
// one vector load (16 B at 4 bits, 8 B at 2 bits, 3 x 4 B at 3 bits, 2 x 16 B at
// 8 bits), so a warp covers a contiguous span per iteration.  Codebooks of every
// group sit in shared memory as fp32 (a 16-entry table maps to 16 distinct banks,
// so lookups never conflict), the activations sit in shared memory as fp32 in a
// lane-transposed order that makes the float4 reads conflict-free, and the M
// partial sums per lane are reduced with shuffles.
#include "common.cuh"

namespace dimq {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr size_t kMaxSmem = 200 * 1024;

template <int BITS>
struct Unit {
  static constexpr int kWords = BITS;  // 32 indices * BITS bits = BITS 32-bit words
  __device__ static void load(const uint8_t* p, uint32_t (&w)[BITS]) {
    if constexpr (BITS == 4) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
      w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
    } else if constexpr (BITS == 2) {
      const uint2 q = __ldg(reinterpret_cast<const uint2*>(p));
      w[0] = q.x; w[1] = q.y;
    } else if constexpr (BITS == 8) {
      const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(p));
      const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(p) + 1);
      w[0] = q0.x; w[1] = q0.y; w[2] = q0.z; w[3] = q0.w; w[4] = q1.x; w[5] = q1.y; w[6] = q1.z; w[7] = q1.w;
    } else {
#pragma unroll
      for (int i = 0; i < BITS; ++i) w[i] = __ldg(reinterpret_cast<const uint32_t*>(p) + i);
    }
  }
  // index i (0..31) of the unit; i is a compile-time constant after unrolling
  __device__ static uint32_t get(const uint32_t (&w)[BITS], int i) {
    const int bit = i * BITS;
    const int word = bit >> 5, sh = bit & 31;
    uint32_t v = w[word] >> sh;
    if (sh + BITS > 32) v |= w[word + 1] << (32 - sh);
    return v & ((1u << BITS) - 1u);
  }
};

template <int BITS, int MT>
__global__ void __launch_bounds__(kThreads)
linear_wq_stream_kernel(const void* __restrict__ x, int x_dtype, dimq_wq_weight w, const void* __restrict__ bias,
                        int bias_dtype, const void* __restrict__ residual, void* __restrict__ y, int y_dtype,
                        int M, int64_t N, int64_t K, int epilogue) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* cb_s = reinterpret_cast<float*>(smem_raw);
  const int cb_total = static_cast<int>(w.groups) * w.entries;
  const int cb_pad = (cb_total + 3) & ~3;
  float* x_s = cb_s + cb_pad;  // [MT][Kp] in lane-transposed order, Kp = K rounded up to 1024
  const int64_t Kp = (K + 1023) & ~static_cast<int64_t>(1023);
  const int tid = threadIdx.x;
  for (int i = tid; i < cb_total; i += kThreads) cb_s[i] = load_as_float(w.codebooks, w.cb_dtype, i);
  // element k = ((it*32 + lane)*8 + q)*4 + e  ->  position ((it*8 + q)*32 + lane)*4 + e:
  // four consecutive k stay together, so x moves as float4 groups
  const bool x_vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  for (int m = 0; m < MT; ++m) {
    float* xm = x_s + m * Kp;
    for (int64_t k4 = static_cast<int64_t>(tid) * 4; k4 < K; k4 += kThreads * 4) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < M) {
        const int64_t src = static_cast<int64_t>(m) * K + k4;
        if (x_dtype == DIMQ_F32) {
          if (x_vec) v = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(x) + src));
          else { const float* xp = static_cast<const float*>(x) + src; v = make_float4(xp[0], xp[1], xp[2], xp[3]); }
        } else {
          uint2 raw;
          if (x_vec) raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(x) + src));
          else { const uint16_t* xp = static_cast<const uint16_t*>(x) + src; raw = make_uint2(xp[0] | (uint32_t(xp[1]) << 16), xp[2] | (uint32_t(xp[3]) << 16)); }
          if (x_dtype == DIMQ_BF16) {
            v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                            __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u));
          } else {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            v = make_float4(a.x, a.y, c.x, c.y);
          }
        }
      }
      const int q = static_cast<int>((k4 >> 2) & 7);
      const int64_t unit = k4 >> 5;
      const int ln = static_cast<int>(unit & 31);
      const int64_t it = unit >> 5;
      *reinterpret_cast<float4*>(xm + ((it * 8 + q) * 32 + ln) * 4) = v;
    }
  }
  __syncthreads();

  const int warp = tid >> 5, lane = tid & 31;
  const int64_t units = K >> 5;
  const int64_t row_bytes = K * BITS / 8;
  const int64_t warp_stride = static_cast<int64_t>(gridDim.x) * kWarps;
  for (int64_t n = static_cast<int64_t>(blockIdx.x) * kWarps + warp; n < N; n += warp_stride) {
    const float* cb = cb_s + (n / w.group_rows) * w.entries;
    const uint8_t* row = w.packed + n * row_bytes;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    for (int64_t u0 = 0; u0 < units; u0 += 32) {
      const int64_t u = u0 + lane;
      if (u < units) {
        uint32_t wd[BITS];
        Unit<BITS>::load(row + u * (4 * BITS), wd);
        const float* xb = x_s + ((u0 >> 5) * 8 * 32 + lane) * 4;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float wv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) wv[e] = cb[Unit<BITS>::get(wd, q * 4 + e)];
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const float4 xv = *reinterpret_cast<const float4*>(xb + m * Kp + q * 128);
            acc[m] = fmaf(xv.x, wv[0], acc[m]);
            acc[m] = fmaf(xv.y, wv[1], acc[m]);
            acc[m] = fmaf(xv.z, wv[2], acc[m]);
            acc[m] = fmaf(xv.w, wv[3], acc[m]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc[m] += __shfl_xor_sync(0xFFFFFFFFu, acc[m], off);
    }
    float mine = 0.0f;
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (lane == m) mine = acc[m];
    if (lane < M) {
      float v = mine + (bias != nullptr ? load_as_float(bias, bias_dtype, n) : 0.0f);
      const int64_t o = static_cast<int64_t>(lane) * N + n;
      const float res = residual != nullptr ? load_as_float(residual, y_dtype, o) : 0.0f;
      store_from_float(y, y_dtype, o, finish_value(v, epilogue, residual != nullptr, res));
    }
  }
}

template <int BITS>
int launch_bits(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                const void* residual, void* y, int y_dtype, int M, int64_t N, int64_t K, int epilogue,
                cudaStream_t st) {
  const int mt = M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
  const size_t cb_pad = (static_cast<size_t>(w->groups) * w->entries + 3) & ~size_t(3);
  const size_t kp = (static_cast<size_t>(K) + 1023) & ~size_t(1023);
  const size_t smem = sizeof(float) * (cb_pad + static_cast<size_t>(mt) * kp);
  if (smem > kMaxSmem) return DIMQ_ERR_UNSUPPORTED;
  // one CTA per SM; rows are dealt to warps round-robin
  int64_t blocks = (N + kWarps - 1) / kWarps;
  if (blocks > kNumSMs) blocks = kNumSMs;
#define DIMQ_STREAM_CASE(MT_)                                                                                   \
  case MT_: {                                                                                                   \
    auto kern = linear_wq_stream_kernel<BITS, MT_>;                                                             \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem);     \
    if (e != cudaSuccess) return static_cast<int>(e);                                                           \
    kern<<<(unsigned)blocks, kThreads, smem, st>>>(x, x_dtype, *w, bias, bias_dtype, residual, y, y_dtype, M, N, \
                                                   K, epilogue);                                                \
    break;                                                                                                      \
  }
  switch (mt) {
    DIMQ_STREAM_CASE(1)
    DIMQ_STREAM_CASE(2)
    DIMQ_STREAM_CASE(4)
    DIMQ_STREAM_CASE(8)
  }
#undef DIMQ_STREAM_CASE
  return launch_status();
}

}  // namespace

// Whether the streaming kernel takes this problem (otherwise the caller picks another path).
bool stream_supported(const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K) {
  if (M < 1 || M > 8 || N < 1) return false;
  if (K % 32 != 0) return false;
  if (!aligned(w->packed, 16)) return false;
  const int mt = M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
  const size_t cb_pad = (static_cast<size_t>(w->groups) * w->entries + 3) & ~size_t(3);
  const size_t kp = (static_cast<size_t>(K) + 1023) & ~size_t(1023);
  return sizeof(float) * (cb_pad + static_cast<size_t>(mt) * kp) <= kMaxSmem;
}

int launch_linear_wq_stream(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                            const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                            int epilogue, cudaStream_t st) {
  if (!stream_supported(w, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  switch (w->bits) {
    case 2: return launch_bits<2>(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, (int)M, N, K, epilogue, st);
    case 3: return launch_bits<3>(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, (int)M, N, K, epilogue, st);
    case 4: return launch_bits<4>(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, (int)M, N, K, epilogue, st);
    case 8: return launch_bits<8>(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, (int)M, N, K, epilogue, st);
    default: return DIMQ_ERR_BAD_BITS;
  }
}

}  // namespace dimq
