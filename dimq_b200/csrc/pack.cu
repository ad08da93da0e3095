// Index bit-packing, activation quantiser, product table and the hard-quantise
// (+pack) export kernel.  All are byte/integer streaming kernels bound by HBM:
// every thread moves 16-byte vectors where alignment allows, a warp covers a
// contiguous span, and nothing is read twice.
#include "common.cuh"

namespace dimq {
namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------
// pack: 16 indices per thread -> 2*BITS bytes
// ---------------------------------------------------------------------------
template <int BITS>
__global__ void __launch_bounds__(kThreads)
pack_bits_kernel(const uint8_t* __restrict__ idx, uint8_t* __restrict__ packed, int64_t n, int vec_ok) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t base = t * 16;
  if (base >= n) return;
  uint32_t v[16];
  const bool full = base + 16 <= n;
  if (full && vec_ok) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(idx + base));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (w[i >> 2] >> ((i & 3) * 8)) & 0xFFu;
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (base + i < n) ? idx[base + i] : 0u;
  }
  constexpr uint32_t mask = (1u << BITS) - 1u;
  unsigned long long lo = 0ull, hi = 0ull;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const unsigned long long val = v[i] & mask;
    const int bit = i * BITS;
    if (bit < 64) {
      lo |= val << bit;
      if (bit + BITS > 64) hi |= val >> (64 - bit);
    } else {
      hi |= val << (bit - 64);
    }
  }
  const int64_t out_off = t * (2 * BITS);
  const int64_t total_bytes = (n * BITS + 7) / 8;
  if (full && vec_ok) {
    if constexpr (BITS == 8) {
      *reinterpret_cast<uint4*>(packed + out_off) =
          make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
    } else if constexpr (BITS == 4) {
      *reinterpret_cast<uint2*>(packed + out_off) = make_uint2((uint32_t)lo, (uint32_t)(lo >> 32));
    } else if constexpr (BITS == 2) {
      *reinterpret_cast<uint32_t*>(packed + out_off) = (uint32_t)lo;
    } else if constexpr (BITS == 1) {
      *reinterpret_cast<uint16_t*>(packed + out_off) = (uint16_t)lo;
    } else {  // BITS == 3: 6 bytes, 2-byte aligned
      uint16_t* o = reinterpret_cast<uint16_t*>(packed + out_off);
      o[0] = (uint16_t)lo;
      o[1] = (uint16_t)(lo >> 16);
      o[2] = (uint16_t)(lo >> 32);
    }
    return;
  }
#pragma unroll
  for (int b = 0; b < 2 * BITS; ++b) {
    if (out_off + b < total_bytes) {
      const unsigned long long word = b < 8 ? lo : hi;
      packed[out_off + b] = static_cast<uint8_t>(word >> ((b & 7) * 8));
    }
  }
}

// ---------------------------------------------------------------------------
// unpack: 2*BITS bytes -> 16 indices per thread
// ---------------------------------------------------------------------------
template <int BITS>
__global__ void __launch_bounds__(kThreads)
unpack_bits_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ idx, int64_t n, int vec_ok) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t base = t * 16;
  if (base >= n) return;
  const int64_t in_off = t * (2 * BITS);
  const int64_t total_bytes = (n * BITS + 7) / 8;
  const bool full = base + 16 <= n;
  unsigned long long lo = 0ull, hi = 0ull;
  if (full && vec_ok && BITS == 4) {
    const uint2 q = __ldg(reinterpret_cast<const uint2*>(packed + in_off));
    lo = (unsigned long long)q.x | ((unsigned long long)q.y << 32);
  } else if (full && vec_ok && BITS == 8) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(packed + in_off));
    lo = (unsigned long long)q.x | ((unsigned long long)q.y << 32);
    hi = (unsigned long long)q.z | ((unsigned long long)q.w << 32);
  } else if (full && vec_ok && BITS == 2) {
    lo = __ldg(reinterpret_cast<const uint32_t*>(packed + in_off));
  } else {
#pragma unroll
    for (int b = 0; b < 2 * BITS; ++b) {
      if (in_off + b < total_bytes) {
        const unsigned long long byte = packed[in_off + b];
        if (b < 8) lo |= byte << (b * 8);
        else hi |= byte << ((b - 8) * 8);
      }
    }
  }
  constexpr unsigned long long mask = (1ull << BITS) - 1ull;
  uint32_t v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int bit = i * BITS;
    unsigned long long val;
    if (bit < 64) {
      val = lo >> bit;
      if (bit + BITS > 64) val |= hi << (64 - bit);
    } else {
      val = hi >> (bit - 64);
    }
    v[i] = static_cast<uint32_t>(val & mask);
  }
  if (full && vec_ok) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = v[4 * j] | (v[4 * j + 1] << 8) | (v[4 * j + 2] << 16) | (v[4 * j + 3] << 24);
    *reinterpret_cast<uint4*>(idx + base) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (base + i < n) idx[base + i] = static_cast<uint8_t>(v[i]);
  }
}

// ---------------------------------------------------------------------------
// activation quantiser: 8 elements per thread
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
quantize_activation_u4_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, int64_t n, float scale, int zp,
                              int vec_ok) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t base = t * 8;
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
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w0 |= quantize_u4(f[i], scale, zp) << (8 * i);
      w1 |= quantize_u4(f[4 + i], scale, zp) << (8 * i);
    }
    *reinterpret_cast<uint2*>(out + base) = make_uint2(w0, w1);
  } else {
    for (int i = 0; i < 8 && base + i < n; ++i)
      out[base + i] = static_cast<uint8_t>(quantize_u4(to_float<T>(x[base + i]), scale, zp));
  }
}

// ---------------------------------------------------------------------------
// product table: one thread per entry of [groups, entries, 16]
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
product_table_kernel(const void* __restrict__ codebook, int cb_dtype, int64_t total, float scale, int zp,
                     float* __restrict__ table) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= total) return;
  const int a = static_cast<int>(i & 15);
  const float c = load_as_float(codebook, cb_dtype, i >> 4);
  const float a_hat = __fmul_rn(scale, static_cast<float>(a - zp));
  table[i] = __fmul_rn(c, a_hat);
}

// ---------------------------------------------------------------------------
// hard quantise (+ pack): 8 consecutive weights per thread
// ---------------------------------------------------------------------------
constexpr int kHqSmemEntries = 8192;  // codebook entries staged in shared memory (32 KB)

template <typename T>
__global__ void __launch_bounds__(kThreads)
hard_quantize_kernel(const T* __restrict__ w, int64_t n, int64_t cols, const float* __restrict__ codebooks,
                     int entries, int64_t groups, int64_t group_rows, uint8_t* __restrict__ idx_out,
                     uint8_t* __restrict__ packed, int bits, int use_smem, int vec_ok, T* __restrict__ fake_out) {
  extern __shared__ float cb_s[];
  // sorted_s[g] != 0: codebook g is finite and non-decreasing, so the nearest codeword of a finite weight
  // is found by bisection (see below) instead of K distance evaluations
  unsigned char* sorted_s = reinterpret_cast<unsigned char*>(cb_s + (use_smem ? groups * entries : 0));
  if (use_smem) {
    const int total = static_cast<int>(groups) * entries;
    for (int i = threadIdx.x; i < total; i += kThreads) cb_s[i] = codebooks[i];
    __syncthreads();
    for (int g = threadIdx.x; g < groups; g += kThreads) {
      const float* c = cb_s + g * entries;
      bool ok = isfinite(c[0]);
      for (int k = 1; k < entries; ++k) ok = ok && isfinite(c[k]) && c[k - 1] <= c[k];
      sorted_s[g] = ok ? 1 : 0;
    }
    __syncthreads();
  }
  const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t base = t * 8;
  if (base >= n) return;
  const bool full = base + 8 <= n;
  float f[8];
  if (full && vec_ok) {
    if constexpr (sizeof(T) == 4) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(w + base));
      const float4 b = __ldg(reinterpret_cast<const float4*>(w + base) + 1);
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(w + base));
      const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = to_float<T>(h[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = (base + i < n) ? to_float<T>(w[base + i]) : 0.0f;
  }
  // the 8 weights of a thread share a codebook unless they straddle a group boundary
  const int64_t g_first = (base / cols) / group_rows;
  const int64_t last = (base + 7 < n ? base + 7 : n - 1);
  const int64_t g_last = (last / cols) / group_rows;
  uint32_t r[8];
  // From 9 to 16 codewords the position of w is counted with one comparison per codeword (the
  // codeword is a broadcast read shared by the thread's eight weights); above, by bisection; up to 8
  // codewords the plain scan below is faster (measured).
  if (g_first == g_last && use_smem && entries > 8 && sorted_s[g_first]) {
    // Sorted finite codebook.  d(k) = fl(fl(w - c[k])^2) does not increase up to the last c[k] < w and
    // does not decrease from the first c[k] >= w on (rounding is monotone), so the minimum is at one of
    // the two entries around w; equal distances form a contiguous run, and the scan's "first minimum"
    // is the lowest index of that run.  A non-finite weight has the same distance (inf or NaN) to every
    // finite codeword: index 0, as the scan gives.
    const float* cb = cb_s + g_first * entries;
    const int top = 1 << (31 - __clz(entries));
    int below[8];  // number of codewords below the weight
#pragma unroll
    for (int i = 0; i < 8; ++i) below[i] = 0;
    if (entries <= 16) {
#pragma unroll 4
      for (int k = 0; k < entries; ++k) {
        const float c = cb[k];
#pragma unroll
        for (int i = 0; i < 8; ++i) below[i] += c < f[i] ? 1 : 0;
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float wv = f[i];
      uint32_t bi = 0u;
      if (isfinite(wv)) {
        int pos = below[i];
        if (entries > 16) {
          for (int step = top; step > 0; step >>= 1) {
            const int q = pos + step;
            if (q <= entries && cb[q - 1] < wv) pos = q;
          }
        }
        const int lo = pos > 0 ? pos - 1 : 0;
        const int hi = pos < entries ? pos : entries - 1;
        float d = __fsub_rn(wv, cb[lo]);
        const float dlo = __fmul_rn(d, d);
        d = __fsub_rn(wv, cb[hi]);
        const float dhi = __fmul_rn(d, d);
        int b = dhi < dlo ? hi : lo;
        const float db = dhi < dlo ? dhi : dlo;
        while (b > 0) {
          d = __fsub_rn(wv, cb[b - 1]);
          if (__fmul_rn(d, d) == db) --b;
          else break;
        }
        bi = static_cast<uint32_t>(b);
      }
      r[i] = bi;
    }
  } else if (g_first == g_last) {
    const float* cb = use_smem ? cb_s + g_first * entries : codebooks + g_first * entries;
    float best[8];
    const float c0 = cb[0];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float d = __fsub_rn(f[i], c0);
      best[i] = __fmul_rn(d, d);
      r[i] = 0u;
    }
    for (int k = 1; k < entries; ++k) {
      const float c = cb[k];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = __fsub_rn(f[i], c);
        const float dd = __fmul_rn(d, d);
        // first minimum wins; a NaN distance beats any number, the first NaN stays
        if (dd < best[i] || (dd != dd && best[i] == best[i])) { best[i] = dd; r[i] = k; }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t e = base + i < n ? base + i : n - 1;
      const int64_t g = (e / cols) / group_rows;
      const float* cb = use_smem ? cb_s + g * entries : codebooks + g * entries;
      float d = __fsub_rn(f[i], cb[0]);
      float best = __fmul_rn(d, d);
      uint32_t bi = 0u;
      for (int k = 1; k < entries; ++k) {
        d = __fsub_rn(f[i], cb[k]);
        const float dd = __fmul_rn(d, d);
        if (dd < best || (dd != dd && best == best)) { best = dd; bi = k; }
      }
      r[i] = bi;
    }
  }
  if (idx_out != nullptr) {
    if (full && vec_ok) {
      const uint32_t w0 = r[0] | (r[1] << 8) | (r[2] << 16) | (r[3] << 24);
      const uint32_t w1 = r[4] | (r[5] << 8) | (r[6] << 16) | (r[7] << 24);
      *reinterpret_cast<uint2*>(idx_out + base) = make_uint2(w0, w1);
    } else {
      for (int i = 0; i < 8 && base + i < n; ++i) idx_out[base + i] = static_cast<uint8_t>(r[i]);
    }
  }
  if (fake_out != nullptr) {
    // straight-through fake quantisation, value of  w + (c[idx].to(w.dtype) - w)  with every operation
    // rounded to the weight's type, as PyTorch evaluates quant/dimq_wrapper.py:72-75
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (base + i < n) {
        const int64_t g = ((base + i) / cols) / group_rows;
        const float* cb = use_smem ? cb_s + g * entries : codebooks + g * entries;
        const float c = to_float<T>(from_float<T>(cb[r[i]]));
        const float diff = to_float<T>(from_float<T>(__fsub_rn(c, f[i])));
        fake_out[base + i] = from_float<T>(__fadd_rn(f[i], diff));
      }
    }
  }
  if (packed != nullptr) {
    // 8 indices -> `bits` bytes at byte offset t*bits of the flattened stream
    const uint32_t mask = (1u << bits) - 1u;
    unsigned long long s = 0ull;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (base + i < n) s |= static_cast<unsigned long long>(r[i] & mask) << (i * bits);
    const int64_t off = t * bits;
    const int64_t total_bytes = (n * bits + 7) / 8;
    for (int b = 0; b < bits; ++b)
      if (off + b < total_bytes) packed[off + b] = static_cast<uint8_t>(s >> (8 * b));
  }
}

inline int64_t blocks_for(int64_t items) { return (items + kThreads - 1) / kThreads; }

template <template <int> class Launcher, typename... Args>
int dispatch_bits(int bits, Args... args) {
  switch (bits) {
    case 1: return Launcher<1>::run(args...);
    case 2: return Launcher<2>::run(args...);
    case 3: return Launcher<3>::run(args...);
    case 4: return Launcher<4>::run(args...);
    case 8: return Launcher<8>::run(args...);
    default: return DIMQ_ERR_BAD_BITS;
  }
}

template <int BITS>
struct PackLauncher {
  static int run(const uint8_t* idx, uint8_t* packed, int64_t n, cudaStream_t st) {
    const int vec_ok = aligned(idx, 16) && aligned(packed, 16);
    pack_bits_kernel<BITS><<<(unsigned)blocks_for((n + 15) / 16), kThreads, 0, st>>>(idx, packed, n, vec_ok);
    return launch_status();
  }
};

template <int BITS>
struct UnpackLauncher {
  static int run(const uint8_t* packed, uint8_t* idx, int64_t n, cudaStream_t st) {
    const int vec_ok = aligned(idx, 16) && aligned(packed, 16);
    unpack_bits_kernel<BITS><<<(unsigned)blocks_for((n + 15) / 16), kThreads, 0, st>>>(packed, idx, n, vec_ok);
    return launch_status();
  }
};

}  // namespace
}  // namespace dimq

using namespace dimq;

extern "C" int dimq_pack_bits(const uint8_t* indices, int64_t numel, int bits, uint8_t* packed, void* stream) {
  if (numel < 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_bits(bits)) return DIMQ_ERR_BAD_BITS;
  if (numel == 0) return DIMQ_OK;
  if (indices == nullptr || packed == nullptr) return DIMQ_ERR_NULL_POINTER;
  return dispatch_bits<PackLauncher>(bits, indices, packed, numel, static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_unpack_bits(const uint8_t* packed, int64_t numel, int bits, uint8_t* indices, void* stream) {
  if (numel < 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_bits(bits)) return DIMQ_ERR_BAD_BITS;
  if (numel == 0) return DIMQ_OK;
  if (indices == nullptr || packed == nullptr) return DIMQ_ERR_NULL_POINTER;
  return dispatch_bits<UnpackLauncher>(bits, packed, indices, numel, static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_pack_u4(const uint8_t* indices, int64_t numel, uint8_t* packed, void* stream) {
  return dimq_pack_bits(indices, numel, 4, packed, stream);
}

extern "C" int dimq_unpack_u4(const uint8_t* packed, int64_t numel, uint8_t* indices, void* stream) {
  return dimq_unpack_bits(packed, numel, 4, indices, stream);
}

extern "C" int dimq_quantize_activation_u4(const void* x, int x_dtype, int64_t numel, float act_scale, int act_zp,
                                           uint8_t* out, void* stream) {
  if (numel < 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(x_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (!(act_scale > 0.0f) || act_zp < 0 || act_zp > 15) return DIMQ_ERR_BAD_QPARAMS;
  if (numel == 0) return DIMQ_OK;
  if (x == nullptr || out == nullptr) return DIMQ_ERR_NULL_POINTER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)blocks_for((numel + 7) / 8);
  const int vec_ok = aligned(x, 16) && aligned(out, 8);
  if (x_dtype == DIMQ_F32)
    quantize_activation_u4_kernel<float><<<blocks, kThreads, 0, st>>>(static_cast<const float*>(x), out, numel,
                                                                      act_scale, act_zp, vec_ok);
  else if (x_dtype == DIMQ_F16)
    quantize_activation_u4_kernel<__half><<<blocks, kThreads, 0, st>>>(static_cast<const __half*>(x), out, numel,
                                                                       act_scale, act_zp, vec_ok);
  else
    quantize_activation_u4_kernel<__nv_bfloat16><<<blocks, kThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), out, numel, act_scale, act_zp, vec_ok);
  return launch_status();
}

extern "C" int dimq_build_product_table(const void* codebook, int cb_dtype, int64_t groups, int entries,
                                        float act_scale, int act_zp, float* table, void* stream) {
  if (groups <= 0 || entries <= 0 || entries > 256) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(cb_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (!(act_scale > 0.0f) || act_zp < 0 || act_zp > 15) return DIMQ_ERR_BAD_QPARAMS;
  if (codebook == nullptr || table == nullptr) return DIMQ_ERR_NULL_POINTER;
  const int64_t total = groups * entries * 16;
  product_table_kernel<<<(unsigned)blocks_for(total), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      codebook, cb_dtype, total, act_scale, act_zp, table);
  return launch_status();
}

static int hard_quantize_launch(const void* w, int w_dtype, int64_t rows, int64_t cols, const float* codebooks,
                                int entries, int64_t group_rows, uint8_t* indices, uint8_t* packed, int bits,
                                void* fake_out, void* stream) {
  if (rows < 0 || cols < 0 || group_rows <= 0) return DIMQ_ERR_BAD_SIZE;
  if (entries <= 0 || entries > 256) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(w_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (packed != nullptr) {
    if (!valid_bits(bits)) return DIMQ_ERR_BAD_BITS;
    if (entries > (1 << bits)) return DIMQ_ERR_BAD_BITS;
  }
  const int64_t n = rows * cols;
  if (n == 0) return DIMQ_OK;
  if (w == nullptr || codebooks == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (indices == nullptr && packed == nullptr && fake_out == nullptr) return DIMQ_ERR_NULL_POINTER;
  const int64_t groups = (rows + group_rows - 1) / group_rows;
  const int use_smem = groups * entries <= kHqSmemEntries;
  const size_t smem = use_smem ? sizeof(float) * static_cast<size_t>(groups * entries) + static_cast<size_t>(groups) : 0;
  const int vec_ok = aligned(w, 16) && (indices == nullptr || aligned(indices, 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)blocks_for((n + 7) / 8);
  const int pbits = packed != nullptr ? bits : 8;
  if (w_dtype == DIMQ_F32)
    hard_quantize_kernel<float><<<blocks, kThreads, smem, st>>>(static_cast<const float*>(w), n, cols, codebooks,
                                                                entries, groups, group_rows, indices, packed, pbits,
                                                                use_smem, vec_ok, static_cast<float*>(fake_out));
  else if (w_dtype == DIMQ_F16)
    hard_quantize_kernel<__half><<<blocks, kThreads, smem, st>>>(static_cast<const __half*>(w), n, cols, codebooks,
                                                                 entries, groups, group_rows, indices, packed, pbits,
                                                                 use_smem, vec_ok, static_cast<__half*>(fake_out));
  else
    hard_quantize_kernel<__nv_bfloat16><<<blocks, kThreads, smem, st>>>(
        static_cast<const __nv_bfloat16*>(w), n, cols, codebooks, entries, groups, group_rows, indices, packed,
        pbits, use_smem, vec_ok, static_cast<__nv_bfloat16*>(fake_out));
  return launch_status();
}

extern "C" int dimq_hard_quantize(const void* w, int w_dtype, int64_t rows, int64_t cols, const float* codebooks,
                                  int entries, int64_t group_rows, uint8_t* indices, uint8_t* packed, int bits,
                                  void* stream) {
  if (indices == nullptr && packed == nullptr && rows * cols != 0) return DIMQ_ERR_NULL_POINTER;
  return hard_quantize_launch(w, w_dtype, rows, cols, codebooks, entries, group_rows, indices, packed, bits, nullptr,
                              stream);
}

extern "C" int dimq_fake_quantize_ste(const void* w, int w_dtype, int64_t rows, int64_t cols, const float* codebooks,
                                      int entries, int64_t group_rows, void* out, uint8_t* indices, void* stream) {
  if (out == nullptr && rows * cols != 0) return DIMQ_ERR_NULL_POINTER;
  return hard_quantize_launch(w, w_dtype, rows, cols, codebooks, entries, group_rows, indices, nullptr, 8, out, stream);
}
