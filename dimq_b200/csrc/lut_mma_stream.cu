// Small-M weight-only LUT GEMM for 16-bit activations (M <= 32): the index-streaming regime.
//
// The packed indices are read from HBM exactly once with coalesced vector loads and never touch
// shared memory; the work per weight is one table lookup for every TWO weights (four at 2 bits) and
// a share of a warp-level mma.sync, which stands in for the M fused multiply-adds per weight that a
// SIMT kernel cannot issue fast enough beyond M = 2.  The tensor pipe is nowhere near busy here: the
// kernel is bound by HBM and by shared-memory lookups, so the warp-level MMA is the right tool and
// the tcgen05 path (which would need the weights staged as operands) is not.
//
// Work unit: 16 output rows x 128 k.  Lane (g = lane / 4, t = lane % 4) of a warp loads, for rows g
// and g + 8 of the block, the 32 consecutive indices k = 32 t .. 32 t + 31 of the chunk (16 B at
// 4 bits, 12 B at 3 bits, 8 B at 2 bits; a quad covers a contiguous span of the row).  Because a dot
// product does not care about the order of k, MMA step s (of 8) takes from every lane its indices
// 4 s .. 4 s + 3: the A fragment registers a0/a2 (row g) and a1/a3 (row g + 8) each hold two
// k-adjacent codewords, which is exactly one entry of a PAIR table indexed by the two packed indices
// (one byte of a 4-bit stream, six bits of a 3-bit stream; at 2 bits one byte gives a0 and a2
// together).  The pair table is stored once per lane ([entry][lane]), so a lookup never has a bank
// conflict whatever the indices are.  The matching B fragment is x[m = g][32 t + 4 s .. + 3]: one
// 8-byte read of the activations, staged in shared memory in an order ([chunk][s][t][4]) and with a
// row stride (2 K + 32 bytes) that put the 16 lanes of a half-warp on distinct banks.
//
// A CTA (16 warps) works on G row blocks at a time and deals their (block, chunk) units round-robin
// to its warps; partial sums meet in a double-buffered shared-memory accumulator with one
// __syncthreads per iteration, after which bias / epilogue / residual are applied and y is stored.
// Index loads run PF units ahead of the arithmetic in a register ring.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"

namespace dimq {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kChunkK = 128;
constexpr size_t kSmemLimit = 220 * 1024;

struct MsParams {
  const void* x;
  const uint8_t* packed;
  const void* codebooks;
  int cb_dtype, entries;
  int64_t group_rows;
  const void* bias;
  int bias_dtype;
  const void* residual;
  void* y;
  int y_dtype;
  int M;
  int64_t N, K;
  int epilogue;
  int G;         // row blocks a CTA works on at a time
  int chunks;    // K / 128
  int units;     // G * chunks
  int upw;       // units per warp and iteration
  int total_it;  // ceil(ceil(N / 16) / G)
  int ipc;       // iterations per CTA
  int xs;        // activation row stride in shared memory, elements
  int dbg;       // measurement only: 1 skip the MMAs, 2 skip the table lookups, 4 skip the activation reads
};

template <int BITS>
struct Cfg {
  static constexpr int kWords = BITS;                                   // 32 indices per lane, row and unit
  static constexpr int kPrefetch = BITS == 4 ? 6 : (BITS == 3 ? 8 : 12);  // units in flight per warp (48 registers)
  static constexpr int kTableEntries = BITS == 3 ? 64 : 256;
  static constexpr int kEntryWords = BITS == 2 ? 2 : 1;
  static constexpr int kTableBytes = kTableEntries * 32 * 4 * kEntryWords;
};

template <bool F16>
__device__ __forceinline__ uint32_t to_operand(float c) {
  if constexpr (F16) return __half_as_ushort(__float2half_rn(c));
  else return __bfloat16_as_ushort(__float2bfloat16_rn(c));
}

template <bool F16>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if constexpr (F16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// Position of a warp in its sequence of units: iteration `it` (global numbering) and the i-th unit of
// the warp inside it.  `u = warp + 16 i` is the unit, `slot = u / chunks` the row block of the
// iteration it belongs to, `chunk = u % chunks` its k chunk.
struct Cursor {
  int it, i, slot, chunk;
  __device__ __forceinline__ void reset(int warp, int chunks) {
    i = 0;
    slot = warp / chunks;
    chunk = warp - slot * chunks;
  }
  __device__ __forceinline__ void advance(int upw, int warp, int chunks) {
    if (++i == upw) {
      ++it;
      reset(warp, chunks);
    } else {
      chunk += kWarps;
      while (chunk >= chunks) { chunk -= chunks; ++slot; }
    }
  }
};

template <int BITS>
__device__ __forceinline__ void load_row_words(const uint8_t* p, uint32_t (&w)[BITS]) {
  if constexpr (BITS == 4) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
    w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
  } else if constexpr (BITS == 2) {
    const uint2 q = __ldg(reinterpret_cast<const uint2*>(p));
    w[0] = q.x; w[1] = q.y;
  } else {
#pragma unroll
    for (int i = 0; i < BITS; ++i) w[i] = __ldg(reinterpret_cast<const uint32_t*>(p) + i);
  }
}

// compile-time loop: f(std::integral_constant<int, I>) for I in [0, N) - every index a constant
template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

template <int BITS, int NB, bool F16>
__global__ void __launch_bounds__(kThreads, 1) linear_wq_mma_stream_kernel(const MsParams p) {
  using C = Cfg<BITS>;
  constexpr int W = C::kWords;
  constexpr int PF = C::kPrefetch;
  constexpr int MR = 8 * NB;  // activation rows held (M rounded up)
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* table = reinterpret_cast<uint32_t*>(smem);
  uint16_t* x_s = reinterpret_cast<uint16_t*>(smem + C::kTableBytes);
  const uint32_t x_bytes = (static_cast<uint32_t>(MR) * p.xs * 2 + 15) & ~15u;
  float* slots = reinterpret_cast<float*>(smem + C::kTableBytes + x_bytes);  // [2][G][MR][16]
  float* cb_s = slots + 2 * p.G * MR * 16;                                     // codewords of the current group

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int it_begin = blockIdx.x * p.ipc;
  const int it_end = min(it_begin + p.ipc, p.total_it);
  const int my_iters = it_end - it_begin;
  if (my_iters <= 0) return;

  // ---- one-time staging: activations (zero rows beyond M), accumulator slots ----
  {
    const int vec_per_row = static_cast<int>(p.K >> 2);  // 4 elements = 8 bytes
    const uint2* xg = static_cast<const uint2*>(p.x);
    // group v = k / 4 of a row is [chunk | t (2 bits) | s (3 bits)]; it is stored at [chunk | s | t], so
    // that MMA step s finds the four lanes of a quad in adjacent 8-byte slots
    for (int m = 0; m < MR; ++m) {
      uint2* dst = reinterpret_cast<uint2*>(x_s + static_cast<size_t>(m) * p.xs);
      if (m < p.M) {
        const uint2* src = xg + static_cast<int64_t>(m) * vec_per_row;
        for (int v = tid; v < vec_per_row; v += kThreads)
          dst[(v & ~31) | ((v & 7) << 2) | ((v >> 3) & 3)] = __ldg(src + v);
      } else {
        for (int v = tid; v < vec_per_row; v += kThreads) dst[v] = make_uint2(0u, 0u);
      }
    }
    for (int idx = tid; idx < 2 * p.G * MR * 16; idx += kThreads) slots[idx] = 0.0f;
  }

  // pair table of one codebook group, one copy per lane: word (entry * 32 + lane)
  auto build_table = [&](int64_t group) {
    if (tid < (1 << BITS))
      cb_s[tid] = tid < p.entries ? load_as_float(p.codebooks, p.cb_dtype, group * p.entries + tid) : 0.0f;
    __syncthreads();
    for (int wi = tid; wi < C::kTableEntries * 32; wi += kThreads) {
      const int e = wi >> 5;
      if constexpr (BITS == 2) {
        uint32_t h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = to_operand<F16>(cb_s[(e >> (2 * j)) & 3]);
        reinterpret_cast<uint2*>(table)[wi] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
      } else {
        table[wi] = to_operand<F16>(cb_s[e & ((1 << BITS) - 1)]) | (to_operand<F16>(cb_s[e >> BITS]) << 16);
      }
    }
  };
  auto group_of_iteration = [&](int it) -> int64_t {
    return (static_cast<int64_t>(it) * p.G * 16) / p.group_rows;
  };
  int64_t cur_group = group_of_iteration(it_begin);
  build_table(cur_group);
  __syncthreads();

  const int64_t row_bytes = p.K * BITS / 8;
  constexpr int kLaneBytes = 4 * BITS;             // 32 indices
  constexpr int kChunkBytes = kChunkK * BITS / 8;  // per row
  // shared-window addresses (32-bit arithmetic from here on)
  const uint32_t tbl_addr = static_cast<uint32_t>(__cvta_generic_to_shared(table)) + lane * (4 * C::kEntryWords);
  const uint32_t x_addr = static_cast<uint32_t>(__cvta_generic_to_shared(x_s)) + g * p.xs * 2 + 8 * t;
  const uint32_t x_nb_stride = 8u * p.xs * 2u;
  const uint8_t* lane_base = p.packed + static_cast<int64_t>(g) * row_bytes + t * kLaneBytes;
  const int64_t half_stride = 8 * row_bytes;

  uint32_t ring[PF][2][W];

  // the unit at cursor (it, i): u = warp + 16 i -> (slot, chunk); loads rows g and g + 8
  auto load_unit = [&](const Cursor& c, uint32_t (&buf)[2][W]) {
    const bool ok = c.it < it_end && c.slot < p.G;
    const int slot = ok ? c.slot : 0, chunk = ok ? c.chunk : 0;
    const int64_t r0 = (static_cast<int64_t>(c.it) * p.G + slot) * 16;
    const uint8_t* src = lane_base + r0 * row_bytes + chunk * kChunkBytes;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (ok && r0 + g + 8 * h < p.N) {
        load_row_words<BITS>(src + h * half_stride, buf[h]);
      } else {
#pragma unroll
        for (int j = 0; j < W; ++j) buf[h][j] = 0u;
      }
    }
  };

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[nb][j] = 0.0f;
  int acc_slot = -1;

  auto flush = [&](int it) {
    float* s = slots + (static_cast<size_t>(it & 1) * p.G + acc_slot) * (MR * 16);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int m = nb * 8 + 2 * t;
      atomicAdd(s + m * 16 + g, acc[nb][0]);
      atomicAdd(s + (m + 1) * 16 + g, acc[nb][1]);
      atomicAdd(s + m * 16 + g + 8, acc[nb][2]);
      atomicAdd(s + (m + 1) * 16 + g + 8, acc[nb][3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[nb][j] = 0.0f;
    }
    acc_slot = -1;
  };

  // eight MMA steps over the 128 k of one unit
  auto process = [&](const Cursor& c, const uint32_t (&buf)[2][W]) {
    if (c.slot >= p.G) return;
    const int slot = c.slot, chunk = c.chunk;
    if (acc_slot >= 0 && acc_slot != slot) flush(c.it);
    acc_slot = slot;
    const uint32_t xb = x_addr + chunk * (kChunkK * 2);
    static_for<0, 8>([&](auto sc) {
      constexpr int s = decltype(sc)::value;
      uint32_t a0, a1, a2, a3;
      if (p.dbg & 2) {
        a0 = buf[0][s % W]; a1 = buf[1][s % W]; a2 = a0 >> 3; a3 = a1 >> 5;
      } else if constexpr (BITS == 4) {
        // two bytes of each row: entry * 128 bytes, taken straight out of the word with a mask
        constexpr int word = s / 2, sh = (2 * s % 4) * 8;
        const uint32_t wg = buf[0][word], wh = buf[1][word];
        // byte b at bit sh: (w >> sh & 0xFF) * 128 == (w << 7 >> sh) & 0x7F80 (for sh >= 8: w >> (sh - 7))
        const uint32_t g0 = sh == 0 ? (wg << 7) & 0x7F80u : (wg >> (sh - 7)) & 0x7F80u;
        const uint32_t g1 = (wg >> (sh + 1)) & 0x7F80u;
        const uint32_t h0 = sh == 0 ? (wh << 7) & 0x7F80u : (wh >> (sh - 7)) & 0x7F80u;
        const uint32_t h1 = (wh >> (sh + 1)) & 0x7F80u;
        a0 = lds_u32(tbl_addr + g0);
        a2 = lds_u32(tbl_addr + g1);
        a1 = lds_u32(tbl_addr + h0);
        a3 = lds_u32(tbl_addr + h1);
      } else if constexpr (BITS == 3) {
        constexpr int bit = 12 * s, word = bit >> 5, sh = bit & 31;
        uint32_t vg, vh;
        if constexpr (sh + 12 > 32) {
          vg = __funnelshift_r(buf[0][word], buf[0][word + 1], sh);
          vh = __funnelshift_r(buf[1][word], buf[1][word + 1], sh);
        } else {
          vg = buf[0][word] >> sh;
          vh = buf[1][word] >> sh;
        }
        a0 = lds_u32(tbl_addr + ((vg << 7) & 0x1F80u));
        a2 = lds_u32(tbl_addr + ((vg << 1) & 0x1F80u));
        a1 = lds_u32(tbl_addr + ((vh << 7) & 0x1F80u));
        a3 = lds_u32(tbl_addr + ((vh << 1) & 0x1F80u));
      } else {
        // one byte -> four codewords (a0 and a2 of its row): entry * 256 bytes
        constexpr int word = s / 4, sh = (s % 4) * 8;
        const uint32_t wg = buf[0][word], wh = buf[1][word];
        const uint32_t og = sh == 0 ? (wg << 8) & 0xFF00u : (wg >> (sh - 8)) & 0xFF00u;
        const uint32_t oh = sh == 0 ? (wh << 8) & 0xFF00u : (wh >> (sh - 8)) & 0xFF00u;
        const uint2 eg = lds_u64(tbl_addr + og), eh = lds_u64(tbl_addr + oh);
        a0 = eg.x; a2 = eg.y; a1 = eh.x; a3 = eh.y;
      }
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        uint2 b = make_uint2(a0, a1);
        if (!(p.dbg & 4)) b = lds_u64(xb + nb * x_nb_stride + 32 * s);
        if (!(p.dbg & 1)) mma_16816<F16>(acc[nb], a0, a1, a2, a3, b.x, b.y);
        else acc[nb][0] += __uint_as_float(a0 ^ a1 ^ a2 ^ a3 ^ b.x ^ b.y);
      }
    });
  };

  // after the iteration's __syncthreads: bias, epilogue, residual, store; then clear the slot
  auto write_iteration = [&](int it) {
    float* s = slots + static_cast<size_t>(it & 1) * p.G * (MR * 16);
    const int total = p.G * MR * 16;
    for (int idx = tid; idx < total; idx += kThreads) {
      const int r = idx & 15;
      const int m = (idx >> 4) % MR;
      const int slot = idx / (MR * 16);
      const float v = s[idx];
      s[idx] = 0.0f;
      const int64_t n = (static_cast<int64_t>(it) * p.G + slot) * 16 + r;
      if (m < p.M && n < p.N) {
        const float vb = v + (p.bias != nullptr ? load_as_float(p.bias, p.bias_dtype, n) : 0.0f);
        const int64_t o = static_cast<int64_t>(m) * p.N + n;
        const float res = p.residual != nullptr ? load_as_float(p.residual, p.y_dtype, o) : 0.0f;
        store_from_float(p.y, p.y_dtype, o, finish_value(vb, p.epilogue, p.residual != nullptr, res));
      }
    }
  };

  Cursor ld, pr;
  ld.it = pr.it = it_begin;
  ld.reset(warp, p.chunks);
  pr.reset(warp, p.chunks);
  static_for<0, PF>([&](auto qc) {
    load_unit(ld, ring[decltype(qc)::value]);
    ld.advance(p.upw, warp, p.chunks);
  });
  const int total = my_iters * p.upw;
  for (int seq = 0; seq < total; seq += PF) {
    static_for<0, PF>([&](auto qc) {
      constexpr int q = decltype(qc)::value;
      if (seq + q < total) {
        process(pr, ring[q]);
        load_unit(ld, ring[q]);
        ld.advance(p.upw, warp, p.chunks);
        if (pr.i == p.upw - 1) {  // the iteration ends here for every warp of the CTA
          if (acc_slot >= 0) flush(pr.it);
          __syncthreads();
          write_iteration(pr.it);
          if (pr.it + 1 < it_end) {
            const int64_t ng = group_of_iteration(pr.it + 1);
            if (ng != cur_group) {  // uniform over the CTA: nobody reads the table between the barriers
              cur_group = ng;
              build_table(ng);
              __syncthreads();
            }
          }
        }
        pr.advance(p.upw, warp, p.chunks);
      }
    });
  }
}

struct Plan {
  int G, chunks, units, upw, total_it, ipc, ctas, nb;
  size_t smem;
};

template <int BITS>
bool make_plan(const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K, Plan* out) {
  const int nb = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  const int chunks = static_cast<int>(K / kChunkK);
  const int64_t row_blocks = (N + 15) / 16;
  double best = 1e30;
  Plan bp{};
  for (int G = 1; G <= 8; G *= 2) {
    if (w->groups > 1 && w->group_rows % (16 * G) != 0) continue;
    const int64_t units = static_cast<int64_t>(G) * chunks;
    if (units > (1 << 20)) continue;
    const int upw = static_cast<int>((units + kWarps - 1) / kWarps);
    const int64_t total_it = (row_blocks + G - 1) / G;
    if (total_it > 0x3FFFFFFF) continue;
    const int64_t ctas0 = total_it < kNumSMs ? total_it : kNumSMs;
    const int64_t ipc = (total_it + ctas0 - 1) / ctas0;
    const double cost = static_cast<double>(ipc) * (upw + 0.4);  // 0.4: barrier + write-back per iteration
    if (cost < best) {
      best = cost;
      bp.G = G; bp.chunks = chunks; bp.units = static_cast<int>(units); bp.upw = upw;
      bp.total_it = static_cast<int>(total_it); bp.ipc = static_cast<int>(ipc);
      bp.ctas = static_cast<int>((total_it + ipc - 1) / ipc);
    }
  }
  if (best >= 1e30) return false;
  bp.nb = nb;
  const size_t xs = static_cast<size_t>(K) + 16;
  const size_t x_bytes = (static_cast<size_t>(8 * nb) * xs * 2 + 15) & ~size_t(15);
  bp.smem = Cfg<BITS>::kTableBytes + x_bytes + sizeof(float) * (2 * bp.G * 8 * nb * 16 + 16);
  if (bp.smem > kSmemLimit) return false;
  *out = bp;
  return true;
}

bool plan_for(const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K, Plan* plan) {
  switch (w->bits) {
    case 2: return make_plan<2>(w, M, N, K, plan);
    case 3: return make_plan<3>(w, M, N, K, plan);
    case 4: return make_plan<4>(w, M, N, K, plan);
    default: return false;
  }
}

template <int BITS, int NB, bool F16>
int launch_one(const MsParams& p, const Plan& plan, cudaStream_t st) {
  auto kern = linear_wq_mma_stream_kernel<BITS, NB, F16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit);
  if (e != cudaSuccess) return static_cast<int>(e);
  kern<<<plan.ctas, kThreads, plan.smem, st>>>(p);
  return launch_status();
}

template <int BITS>
int launch_bits(const MsParams& p, const Plan& plan, bool f16, cudaStream_t st) {
  switch (plan.nb) {
    case 1: return f16 ? launch_one<BITS, 1, true>(p, plan, st) : launch_one<BITS, 1, false>(p, plan, st);
    case 2: return f16 ? launch_one<BITS, 2, true>(p, plan, st) : launch_one<BITS, 2, false>(p, plan, st);
    default: return f16 ? launch_one<BITS, 4, true>(p, plan, st) : launch_one<BITS, 4, false>(p, plan, st);
  }
}

}  // namespace

// 16-bit activations whose format the codewords can take without a second term (fp16 activations, or
// bf16 activations with a bf16 codebook), M <= 32, K a multiple of 128, 2-, 3- or 4-bit indices.
bool mma_stream_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K) {
  if (x_dtype != DIMQ_F16 && x_dtype != DIMQ_BF16) return false;
  if (x_dtype == DIMQ_BF16 && w->cb_dtype != DIMQ_BF16) return false;
  if (M < 1 || M > 32 || N < 1 || K < kChunkK || K % kChunkK != 0) return false;
  if (w->bits != 2 && w->bits != 3 && w->bits != 4) return false;
  if (w->groups > 1 && w->group_rows % 16 != 0) return false;
  if (!aligned(x, 8) || !aligned(w->packed, 16)) return false;
  if (N > (int64_t(1) << 34)) return false;
  Plan plan;
  return plan_for(w, M, N, K, &plan);
}

int launch_linear_wq_mma_stream(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                int bias_dtype, const void* residual, void* y, int y_dtype, int64_t M, int64_t N,
                                int64_t K, int epilogue, cudaStream_t st) {
  if (!mma_stream_supported(x, x_dtype, w, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  Plan plan;
  if (!plan_for(w, M, N, K, &plan)) return DIMQ_ERR_UNSUPPORTED;
  MsParams p{};
  p.x = x; p.packed = w->packed; p.codebooks = w->codebooks; p.cb_dtype = w->cb_dtype; p.entries = w->entries;
  p.group_rows = w->groups > 1 ? w->group_rows : (N + 15) / 16 * 16 + 16;
  p.bias = bias; p.bias_dtype = bias_dtype; p.residual = residual; p.y = y; p.y_dtype = y_dtype;
  p.M = static_cast<int>(M); p.N = N; p.K = K; p.epilogue = epilogue;
  p.G = plan.G; p.chunks = plan.chunks; p.units = plan.units; p.upw = plan.upw; p.total_it = plan.total_it;
  p.ipc = plan.ipc; p.xs = static_cast<int>(K) + 16;
  { const char* e = getenv("DIMQ_B200_MS_DEBUG"); p.dbg = e ? atoi(e) : 0; }
  const bool f16 = x_dtype == DIMQ_F16;
  switch (w->bits) {
    case 2: return launch_bits<2>(p, plan, f16, st);
    case 3: return launch_bits<3>(p, plan, f16, st);
    default: return launch_bits<4>(p, plan, f16, st);
  }
}

}  // namespace dimq
