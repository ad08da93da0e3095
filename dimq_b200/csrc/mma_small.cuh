// Pieces shared by the two small-M weight-only kernels (warp-level MMAs fed by pair-table lookups):
// the table geometry, the operand conversion, the m16n8k16 MMA, the index loads and the lookups.
#pragma once

#include <type_traits>

#include "common.cuh"

namespace dimq {
namespace small_m {

constexpr uint32_t kSmemWindow = 227 * 1024;  // dynamic shared memory a CTA may ask for
constexpr uint32_t kLowStart = 1024;          // the dynamic window starts at or below this shared address

// Pair table of one codebook group: entry e (two packed indices; four at 2 bits) holds the 16-bit
// codewords of those indices in MMA fragment order.  One copy per lane ([entry][lane]): a lookup never
// has a bank conflict whatever the indices are.  The table sits at an absolute shared address that is a
// multiple of its size, so a lookup address is (index bits, masked in place) | (base | lane offset).
template <int BITS>
struct PairTable {
  static constexpr int kEntries = BITS == 3 ? 64 : 256;
  static constexpr int kEntryWords = BITS == 2 ? 2 : 1;
  static constexpr uint32_t kBytes = kEntries * 32 * 4 * kEntryWords;
  static constexpr uint32_t kAddr = BITS == 2 ? 65536u : 32768u;
  static constexpr uint32_t kEnd = kAddr + kBytes;
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
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// the 32 indices of one lane, row and unit: BITS words
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

// Table lookups: their addresses depend on index words the thread has just read, so the compiler
// cannot move them ahead of the data they need, and the table only changes between two barriers that
// no lookup can cross for the same reason.  Not volatile: the scheduler is free to issue the lookups of
// later MMA steps early.
__device__ __forceinline__ uint32_t lookup_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lookup_u64(uint32_t addr) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// A fragments of MMA step s (of 8) of a unit: the lane's indices 4 s .. 4 s + 3 of rows g (wg) and
// g + 8 (wh), looked up in the pair table at `tbl` (= table address | lane offset).
template <int BITS, int S>
__device__ __forceinline__ void lookup_step(const uint32_t (&wg)[BITS], const uint32_t (&wh)[BITS], uint32_t tbl,
                                            uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
  if constexpr (BITS == 4) {
    // byte b of the word, times 128 bytes per entry: (w >> (8 b - 7)) & 0x7F80
    constexpr int word = S / 2, b = 2 * S % 4;
    const uint32_t g0 = b == 0 ? (wg[word] << 7) : (wg[word] >> (8 * b - 7));
    const uint32_t h0 = b == 0 ? (wh[word] << 7) : (wh[word] >> (8 * b - 7));
    a0 = lookup_u32((g0 & 0x7F80u) | tbl);
    a2 = lookup_u32(((wg[word] >> (8 * b + 1)) & 0x7F80u) | tbl);
    a1 = lookup_u32((h0 & 0x7F80u) | tbl);
    a3 = lookup_u32(((wh[word] >> (8 * b + 1)) & 0x7F80u) | tbl);
  } else if constexpr (BITS == 3) {
    constexpr int bit = 12 * S, word = bit >> 5, sh = bit & 31;
    uint32_t vg, vh;
    if constexpr (sh + 12 > 32) {
      vg = __funnelshift_r(wg[word], wg[word + 1], sh);
      vh = __funnelshift_r(wh[word], wh[word + 1], sh);
    } else {
      vg = wg[word] >> sh;
      vh = wh[word] >> sh;
    }
    a0 = lookup_u32(((vg << 7) & 0x1F80u) | tbl);
    a2 = lookup_u32(((vg << 1) & 0x1F80u) | tbl);
    a1 = lookup_u32(((vh << 7) & 0x1F80u) | tbl);
    a3 = lookup_u32(((vh << 1) & 0x1F80u) | tbl);
  } else {
    // one byte -> four codewords (a0 and a2 of its row), 256 bytes per entry: the byte drops into
    // byte 1 of the table address with one permute
    constexpr int word = S / 4, b = S % 4;
    constexpr uint32_t sel = 0x7604u | (b << 4);
    const uint2 eg = lookup_u64(__byte_perm(wg[word], tbl, sel));
    const uint2 eh = lookup_u64(__byte_perm(wh[word], tbl, sel));
    a0 = eg.x; a2 = eg.y; a1 = eh.x; a3 = eh.y;
  }
}

// Pair table of the codewords in cb[0 .. 2^BITS) (floats in shared memory), written by `threads`
// threads of which the caller is number `tid`: 16 bytes per store, four lanes' copies of an entry (two
// at 2 bits, where an entry is 8 bytes).
template <int BITS, bool F16>
__device__ __forceinline__ void fill_pair_table(uint4* table4, const float* cb, int tid, int threads) {
  using T = PairTable<BITS>;
  if constexpr (BITS == 2) {
#pragma unroll 2
    for (int wi = tid; wi < T::kEntries * 16; wi += threads) {
      const int e = wi >> 4;
      uint32_t h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = to_operand<F16>(cb[(e >> (2 * j)) & 3]);
      const uint32_t a = h[0] | (h[1] << 16), b = h[2] | (h[3] << 16);
      table4[wi] = make_uint4(a, b, a, b);
    }
  } else {
#pragma unroll 2
    for (int wi = tid; wi < T::kEntries * 8; wi += threads) {
      const int e = wi >> 3;
      const uint32_t v = to_operand<F16>(cb[e & ((1 << BITS) - 1)]) | (to_operand<F16>(cb[e >> BITS]) << 16);
      table4[wi] = make_uint4(v, v, v, v);
    }
  }
}

}  // namespace small_m
}  // namespace dimq
