// Small-M weight-only LUT GEMM (M <= 16, 16-bit activations) for weights large enough to be bound by
// the index stream: the activations stay in REGISTERS and the indices go from HBM straight into
// registers, so the shared-memory pipe carries the table lookups and little else.
//
// Same arithmetic as the index-streaming kernel (pair-table lookups feeding warp-level m16n8k16 MMAs,
// work unit = 16 output rows x 128 k, lane (g, t) takes 32 consecutive indices of rows g and g + 8), but
// the loops are turned inside out: a warp owns ONE 128-k range and walks down the row blocks.  Its B
// fragments - x[m = g (+8)][32 t .. 32 t + 31] of that k range, 16 registers per eight activation
// rows - are loaded once; per unit it issues two index loads (4-bit: 16 bytes per lane), kDepth units
// ahead, 32 lookups and 8 (16 at M > 8) MMAs.  No ring, no mbarrier, no activation reads.
//
// Index layout.  From the canonical [N][K] stream a warp's load touches eight rows (sixteen 16-byte
// pieces).  dimq_linear_prepack re-orders the stream once per layer into tiles of 16 rows x 128 k, every
// unit contiguous; the kernel then reads one run of 512 bytes per load, which is what its bound - the
// load / store data pipe - rewards (12.9 against 14.4 us at M = 8 on 8192 x 8192).
//
// The price is a reduction over the k ranges.  A CTA's 16 warps cover 2048 consecutive k of the same row
// blocks; each keeps the 16 x M partial sums of every unit in a buffer of its own in shared memory - as
// many units as fit beside the table (a "chunk": all of a CTA's row blocks at the sizes this kernel is
// chosen for), so the warps run freely, without a barrier per row block.  After a chunk one barrier, then
// all threads add the sixteen tiles of every unit into a per-CTA array `fin`, and a second barrier.  K / 2048
// CTAs (k slices) share a range of row blocks - several passes when K / 2048 has no divisor <= 8; each
// writes its `fin` to a slice of the caller's workspace ([k slice][M][N] floats) and a second, tiny kernel
// adds the slices and finishes the outputs (bias, epilogue, residual, store).  Nothing waits for another
// CTA, there are no atomics, and the sums are added in a fixed order.  (One kernel in which the CTA that
// arrives last does the adding was 1.5-7 us slower: its memory fence and the L2 reads of one CTA per range
// sit at the very end, where a separate kernel spreads them over all SMs.)  With K = 2048 there is one
// slice: no workspace, no second kernel.
//
// bf16 activations with an fp16 / fp32 codebook are converted to fp16 in registers.  A lane's 32
// elements of a row are exact in fp16 for 6.1e-5 <= |x| <= 65504; a (row, k range) whose largest finite
// magnitude exceeds 2^15, or is non-zero but below 2^-10, is scaled by a power of two into [2^14, 2^15)
// and the warp's partial sums are scaled back before they leave the warp.
#include <cuda.h>

#include "common.cuh"
#include "mma_small.cuh"

namespace dimq {
namespace {

using namespace small_m;

constexpr int kCtaK = 2048;   // k of a CTA's warps together; a warp owns KR = 128 of them (16 warps) or 64 (32 warps)
constexpr int kDepth = 3;     // units of indices in flight per warp (four: 7 % slower)
constexpr uint32_t kLowPart = 2048;   // shared address where the partial tiles below the table start
constexpr int kMaxSlices = 8;   // k slices worked on at a time (CTAs sharing a range of row blocks)

struct RgParams {
  const void* x;
  const uint8_t* packed;
  const void* codebooks;
  int cb_dtype, entries;
  int group_rbs;   // row blocks per codebook group
  const void* bias;
  int bias_dtype;
  const void* residual;
  void* y;
  int y_dtype;
  int M;
  int64_t N, K;
  int64_t row_bytes;  // of the packed index matrix
  int tiled;          // 1: `packed` is the output of dimq_linear_prepack ([row block][128-k range][16 rows][16 * bits bytes])
  int epilogue;
  int cvt;       // 1: x is bf16 and is converted to fp16 in registers
  int nrb;       // row blocks (N / 16)
  int ks;        // k slices of 2048 worked on at a time = CTAs per range of row blocks
  int passes;    // slices / ks
  int nk;        // 128-k ranges of the weight (K / 128): warps of the last slice beyond it have nothing to do
  int ranges;    // ranges of row blocks (each worked on by ks CTAs)
  float* partial;  // ks > 1: [ks][M][N] sums of the k slices
  int chunk;       // units a warp runs through between two reductions
  int chunk_low;   // of which so many have their partial tiles below the table
  uint32_t fin_bytes;  // size of `fin`: the partial tiles above the table start behind it
  uint32_t* status;
#ifdef DIMQ_B200_DIAG
  uint32_t* trace;   // host-mapped clock samples, [CTA][32]
#endif
};

static __device__ uint32_t g_rg_status;

// diagnostic builds: warps 0, 7 and 15 of every CTA record the SM clock at eight
// points (the words live in pinned host memory): [CTA][warp 0 / 7 / 15][point]
#ifdef DIMQ_B200_DIAG
#define RG_MARK(k)                                                                                      \
  do {                                                                                                  \
    const int w_ = threadIdx.x >> 5;                                                                    \
    if (p.trace != nullptr && (threadIdx.x & 31) == 0 && (w_ == 0 || w_ == 7 || w_ == 15))             \
      p.trace[blockIdx.x * 32 + (w_ == 0 ? 0 : (w_ == 7 ? 8 : 16)) + (k)] = static_cast<uint32_t>(clock64()); \
  } while (0)
#else
#define RG_MARK(k) do {} while (0)
#endif

__device__ __forceinline__ void st_shared_f2(uint32_t addr, float a, float b) {
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}

// Table geometry of this kernel.  At 4 bits an entry takes 256 bytes (32 lanes x 4 bytes, the rest unused)
// so that, as at 2 bits, one byte permute drops an index byte into byte 1 of the lookup address.
template <int BITS>
struct Tbl {
  static constexpr uint32_t kAddr = BITS == 3 ? PairTable<3>::kAddr : 65536u;
  static constexpr uint32_t kBytes = BITS == 3 ? PairTable<3>::kBytes : 65536u;
  static constexpr uint32_t kEnd = kAddr + kBytes;
  static constexpr int kLaneBytes = BITS == 2 ? 8 : 4;
};

template <int BITS, bool F16>
__device__ __forceinline__ void fill_table(uint4* table4, const float* cb, int tid, int threads) {
  if constexpr (BITS == 4) {
#pragma unroll 2
    for (int wi = tid; wi < 256 * 8; wi += threads) {
      const int e = wi >> 3;
      const uint32_t v = to_operand<F16>(cb[e & 15]) | (to_operand<F16>(cb[e >> 4]) << 16);
      table4[e * 16 + (wi & 7)] = make_uint4(v, v, v, v);
    }
  } else {
    fill_pair_table<BITS, F16>(table4, cb, tid, threads);
  }
}

// A fragments of MMA step S: the lane's indices 4 S .. 4 S + 3 of rows g (wg) and g + 8 (wh)
template <int BITS, int WL, int S>
__device__ __forceinline__ void lookup_a(const uint32_t (&wg)[WL], const uint32_t (&wh)[WL], uint32_t tbl,
                                         uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
  if constexpr (BITS == 4) {
    constexpr int word = S / 2, b = 2 * S % 4;
    constexpr uint32_t sel0 = 0x7604u | (b << 4), sel1 = 0x7604u | ((b + 1) << 4);
    a0 = lookup_u32(__byte_perm(wg[word], tbl, sel0));
    a2 = lookup_u32(__byte_perm(wg[word], tbl, sel1));
    a1 = lookup_u32(__byte_perm(wh[word], tbl, sel0));
    a3 = lookup_u32(__byte_perm(wh[word], tbl, sel1));
  } else if constexpr (BITS == 2) {
    // one byte -> four codewords (a0 and a2 of its row)
    constexpr int word = S / 4, b = S % 4;
    constexpr uint32_t sel = 0x7604u | (b << 4);
    const uint2 eg = lookup_u64(__byte_perm(wg[word], tbl, sel));
    const uint2 eh = lookup_u64(__byte_perm(wh[word], tbl, sel));
    a0 = eg.x; a2 = eg.y; a1 = eh.x; a3 = eh.y;
  } else {
    lookup_step<BITS, S>(wg, wh, tbl, a0, a1, a2, a3);   // 3 bits: WL == 3
  }
}

// d = a * b (no accumulator input: the first step of a unit)
template <bool F16>
__device__ __forceinline__ void mma_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
  if constexpr (F16) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
  }
}

// the lane's indices of one row of a unit: KR / 4 of them, WL words
template <int WL>
__device__ __forceinline__ void load_lane_words(const uint8_t* p, uint32_t (&w)[WL]) {
  if constexpr (WL == 4) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
    w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
  } else if constexpr (WL == 2) {
    const uint2 q = __ldg(reinterpret_cast<const uint2*>(p));
    w[0] = q.x; w[1] = q.y;
  } else {
#pragma unroll
    for (int i = 0; i < WL; ++i) w[i] = __ldg(reinterpret_cast<const uint32_t*>(p) + i);
  }
}

// KR: k of one warp.  128 (16 warps of up to 128 registers) is what runs.  64 (32 warps of 64 registers,
// diagnostic builds only) was 30 % slower at 8192 x 8192: the kernel is not short of warps to hide latency
// behind, it is bound by the load / store pipe - per unit 32 lookups, 16 wavefronts of index loads (a
// warp's 16-byte pieces lie in eight different rows), the partial tile - and halving a warp's k doubles
// the loads and tiles per k.
// MR: columns kept of a unit's 16 x 8 (M > 8: 16 x 16) accumulator tile - M rounded up to 2, 4, 8 or 16.
// The MMAs always compute eight (sixteen) columns; only the lanes that hold one of the first MR columns
// store their part of the partial tile, so the tile costs one shared-memory wavefront per store instead
// of two at M <= 4, and its reduction shrinks with it.
template <int BITS, int MR, bool F16, int KR>
__global__ void __launch_bounds__(kCtaK / KR * 32, 1) linear_wq_mma_regs_kernel(const RgParams p) {
  constexpr int NB = MR == 16 ? 2 : 1;   // 8-column MMA tiles
  using T = Tbl<BITS>;
  constexpr int kKWarps = kCtaK / KR;
  constexpr int TH = kKWarps * 32;
  constexpr int W = KR / 4 * BITS / 32;   // words of a lane's indices of one row of a unit
  constexpr int kSteps = KR / 16;         // MMA steps of a unit
  constexpr int XW = KR / 8;              // registers of a lane's activations of one row
  constexpr int kTile = 16 * MR;      // floats of one row block's sums
  extern __shared__ __align__(16) unsigned char smem[];
  const uint32_t s0 = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  if (s0 > kLowStart) {  // same for every CTA of the grid: the fixed layout below would not fit, do nothing
    if (threadIdx.x == 0) atomicOr(p.status, 0x80000A01u);
    return;
  }
  unsigned char* const abs0 = smem - s0;  // generic address of shared address 0
  float* cb_s = reinterpret_cast<float*>(abs0 + kLowStart);
  uint4* table4 = reinterpret_cast<uint4*>(abs0 + T::kAddr);
  // [kLowPart, table): partial tiles of the first chunk_low units of a chunk, [unit][warp][16 rows][MR];
  // [table end, +fin_bytes): fin, [row block of this CTA][16 rows][MR]; behind it the other units' tiles
  constexpr uint32_t kUnitBytes = kKWarps * kTile * 4;
  constexpr uint32_t kFinAddr = T::kEnd;
  float* fin = reinterpret_cast<float*>(abs0 + kFinAddr);
  const uint32_t part_high = kFinAddr + p.fin_bytes;
  auto part_addr = [&](int slot) -> uint32_t {   // shared address of the sixteen tiles of unit `slot` of a chunk
    return slot < p.chunk_low ? kLowPart + slot * kUnitBytes : part_high + (slot - p.chunk_low) * kUnitBytes;
  };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int range = blockIdx.x / p.ks;
  const int rank = blockIdx.x - range * p.ks;   // which k slice
  const int rb0 = static_cast<int>(static_cast<int64_t>(p.nrb) * range / p.ranges);
  const int rb1 = static_cast<int>(static_cast<int64_t>(p.nrb) * (range + 1) / p.ranges);
  const int n_it = rb1 - rb0;          // >= 1: there are no more ranges than row blocks

  RG_MARK(0);
  // the kernel that follows in the stream may start its own prologue now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  int cur_group = rb0 / p.group_rbs;
  int group_end = (cur_group + 1) * p.group_rbs - rb0;   // first iteration of the next codebook group
  float first_cb = 0.0f;
  if (tid < (1 << BITS) && tid < p.entries)
    first_cb = load_as_float(p.codebooks, p.cb_dtype, static_cast<int64_t>(cur_group) * p.entries + tid);

  // byte offsets into the packed matrix fit 32 bits (checked on the host)
  const uint32_t row_bytes = static_cast<uint32_t>(p.row_bytes);
  // canonical layout: the lane's pieces of rows g and g + 8 lie 8 rows apart and a warp's load touches eight
  // rows; tiled layout: the 16 row pieces of a unit are contiguous, a warp's load is one run of 512 bytes
  constexpr uint32_t kPiece = KR * BITS / 8;   // bytes of one row of a unit
  const uint32_t it_stride = 16u * row_bytes;  // the same unit of the next row block (either layout)
  const uint32_t half_stride = p.tiled ? 8u * kPiece : 8u * row_bytes;
  auto unit_off = [&](int pass) -> uint32_t {
    const int kr = (pass * p.ks + rank) * kKWarps + warp;
    if (p.tiled) return static_cast<uint32_t>(rb0) * it_stride + (kr * 16u + g) * kPiece + t * (4 * W);
    return (static_cast<uint32_t>(rb0) * 16u + g) * row_bytes + kr * kPiece + t * (4 * W);
  };
  // K need not fill the last slice: a warp whose range lies beyond K loads nothing, keeps zero activations and
  // so contributes tiles of zeros (its lookups read the table at whatever its zeroed index words say)
  auto live = [&](int pass) -> bool { return (pass * p.ks + rank) * kKWarps + warp < p.nk; };
  bool live_now = live(0);
  uint32_t buf[kDepth][2][W] = {};
  auto load_unit = [&](uint32_t (&b)[2][W], uint32_t off) {
    if (!live_now) return;   // uniform over the warp
    load_lane_words<W>(p.packed + off, b[0]);
    load_lane_words<W>(p.packed + off + half_stride, b[1]);
  };
  uint32_t off0 = unit_off(0);
  static_for<0, kDepth>([&](auto dc) {
    constexpr int d = decltype(dc)::value;
    if (d < n_it) load_unit(buf[d], off0 + d * it_stride);
  });

  auto build_table = [&](bool preloaded) {
    if (tid < (1 << BITS)) {
      if (preloaded) cb_s[tid] = first_cb;
      else cb_s[tid] = tid < p.entries ? load_as_float(p.codebooks, p.cb_dtype, static_cast<int64_t>(cur_group) * p.entries + tid) : 0.0f;
    }
    __syncthreads();
    fill_table<BITS, F16>(table4, cb_s, tid, TH);
    __syncthreads();
  };
  build_table(true);
  RG_MARK(1);

  // the activations may be the output of the kernel before this one in the stream: wait for it
  asm volatile("griddepcontrol.wait;" ::: "memory");
  RG_MARK(2);

  const uint32_t tbl = T::kAddr + lane * T::kLaneBytes;
  int seq = 0;
  for (int pass = 0; pass < p.passes; ++pass) {
    if (pass > 0) {
      live_now = live(pass);
      off0 = unit_off(pass);
      static_for<0, kDepth>([&](auto dc) {
        constexpr int d = decltype(dc)::value;
        if (d < n_it) load_unit(buf[d], off0 + d * it_stride);
      });
      if (cur_group != rb0 / p.group_rbs) {   // back to the first row block's codebook
        cur_group = rb0 / p.group_rbs;
        __syncthreads();
        build_table(false);
      }
      group_end = (cur_group + 1) * p.group_rbs - rb0;
    }
    // ---- B fragments of this warp's k range: x[m = nb * 8 + g][32 t .. 32 t + 31], kept for all row blocks ----
    uint32_t xb[NB][XW];
    float inv[NB][2];   // what the sums of columns 2 t, 2 t + 1 are multiplied by (converting mode)
    const int kr = (pass * p.ks + rank) * kKWarps + warp;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int m = nb * 8 + g;
      uint4 q[XW / 4];
      if (m < p.M && live_now) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) +
                                                          static_cast<int64_t>(m) * p.K + kr * KR + (KR / 4) * t);
#pragma unroll
        for (int j = 0; j < XW / 4; ++j) q[j] = __ldg(src + j);
      } else {
#pragma unroll
        for (int j = 0; j < XW / 4; ++j) q[j] = make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < XW / 4; ++j) {
        xb[nb][4 * j] = q[j].x; xb[nb][4 * j + 1] = q[j].y; xb[nb][4 * j + 2] = q[j].z; xb[nb][4 * j + 3] = q[j].w;
      }
      float back = 1.0f;
      if constexpr (F16) {
        if (p.cvt) {
          float a = 0.0f;   // largest finite magnitude of the row within this k range
#pragma unroll
          for (int j = 0; j < XW; ++j) {
            const float2 xy = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xb[nb][j]));
            if (fabsf(xy.x) < 3.0e38f) a = fmaxf(a, fabsf(xy.x));
            if (fabsf(xy.y) < 3.0e38f) a = fmaxf(a, fabsf(xy.y));
          }
          a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, 1));
          a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, 2));
          float f = 1.0f;
          if (a > 32768.0f || (a > 0.0f && a < 0.0009765625f)) {
            int e;
            frexpf(a, &e);               // a = frac * 2^e, frac in [0.5, 1)
            e = max(e, -111);            // the factor stays a finite float for the smallest bf16 subnormals
            f = ldexpf(1.0f, 15 - e);    // a * f in [2^14, 2^15)
            back = ldexpf(1.0f, e - 15);
          }
#pragma unroll
          for (int j = 0; j < XW; ++j) {
            float2 xy = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xb[nb][j]));
            xy.x *= f; xy.y *= f;
            const __half2 h = __float22half2_rn(xy);
            xb[nb][j] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
      }
      // column 2 t (+1) of the accumulator tile is activation row 2 t (+1): its factor sits with lane g = 2 t (+1)
      inv[nb][0] = __shfl_sync(0xFFFFFFFFu, back, 8 * t);
      inv[nb][1] = __shfl_sync(0xFFFFFFFFu, back, 8 * t + 4);
    }
    if (pass == 0) RG_MARK(3);

    int c0 = 0, c_end = min(n_it, p.chunk);   // the chunk being worked on: units [c0, c_end)
    for (int it0 = 0; it0 < n_it; it0 += kDepth) {
      static_for<0, kDepth>([&](auto dc) {
        constexpr int d = decltype(dc)::value;
        const int it = it0 + d;
        if (it < n_it) {   // uniform over the CTA
          if (it == group_end) {   // nobody looks anything up between the barriers of the rebuild
            ++cur_group;
            group_end += p.group_rbs;
            __syncthreads();
            build_table(false);
          }
          // the lookups below take the table address from here, after a rebuild's barriers: nothing
          // else orders them against it (they are not volatile, so that the scheduler may interleave them)
          uint32_t tbl_it = tbl;
          asm volatile("" : "+r"(tbl_it)::"memory");
          uint32_t cur[2][W];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < W; ++j) cur[h][j] = buf[d][h][j];
          if (it + kDepth < n_it) load_unit(buf[d], off0 + static_cast<uint32_t>(it + kDepth) * it_stride);

          // M <= 8: two accumulator sets (even / odd MMA steps) halve the dependent chain through the
          // MMAs; at M > 8 the two column tiles already are two chains
          constexpr int E = NB == 1 ? 2 : 1;
          float acc[E][NB][4];
          static_for<0, kSteps>([&](auto sc) {
            constexpr int s = decltype(sc)::value;
            uint32_t a0, a1, a2, a3;
            lookup_a<BITS, W, s>(cur[0], cur[1], tbl_it, a0, a1, a2, a3);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              if constexpr (s < E) mma_16816_first<F16>(acc[s % E][nb], a0, a1, a2, a3, xb[nb][2 * s], xb[nb][2 * s + 1]);
              else mma_16816<F16>(acc[s % E][nb], a0, a1, a2, a3, xb[nb][2 * s], xb[nb][2 * s + 1]);
            }
          });

          // the warp's partial tile of this unit
          const uint32_t dst = part_addr(it - c0) + static_cast<uint32_t>(warp * kTile) * 4u;
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            float c[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) c[j] = E == 2 ? acc[0][nb][j] + acc[E - 1][nb][j] : acc[0][nb][j];
            const int m = nb * 8 + 2 * t;
            if (MR >= 8 || m < MR) {   // only the lanes that hold a kept column
              st_shared_f2(dst + (g * MR + m) * 4, c[0] * inv[nb][0], c[1] * inv[nb][1]);
              st_shared_f2(dst + ((g + 8) * MR + m) * 4, c[2] * inv[nb][0], c[3] * inv[nb][1]);
            }
          }
          if (it + 1 == c_end) {
            // end of a chunk: all threads add the sixteen tiles of each of its units into `fin`
            __syncthreads();
            const int outs = (c_end - c0) * kTile;
            for (int o = tid; o < outs; o += TH) {
              const int slot = o / kTile, e = o - slot * kTile;   // consecutive lanes: consecutive words
              const float* src = reinterpret_cast<const float*>(abs0 + part_addr(slot)) + e;
              float sum = src[0];
#pragma unroll
              for (int wi = 1; wi < kKWarps; ++wi) sum += src[wi * kTile];
              float* f = fin + static_cast<size_t>(c0 + slot) * kTile + e;
              *f = pass > 0 ? *f + sum : sum;
            }
            __syncthreads();
            c0 = c_end;
            c_end = min(n_it, c0 + p.chunk);
          }
          if (seq == 0) RG_MARK(4);
          ++seq;
        }
      });
    }
  }

  // ---- one k slice: finish the outputs here; several: this CTA's sums go to its slice of the workspace ----
  RG_MARK(5);
  __syncthreads();
  RG_MARK(6);
  const int n_rows = n_it * 16;
  const int total_out = p.M * n_rows;
  const int64_t n0 = static_cast<int64_t>(rb0) * 16;
  if (p.ks > 1) {
    float* dst = p.partial + static_cast<int64_t>(rank) * p.M * p.N + n0;
    for (int o = tid; o < total_out; o += TH) {
      const int m = o / n_rows, nl = o - m * n_rows;   // consecutive threads: consecutive output columns
      dst[static_cast<int64_t>(m) * p.N + nl] = fin[nl * MR + m];
    }
  } else {
    for (int o = tid; o < total_out; o += TH) {
      const int m = o / n_rows, nl = o - m * n_rows;
      const int64_t n = n0 + nl;
      const float vb = fin[nl * MR + m] + (p.bias != nullptr ? load_as_float(p.bias, p.bias_dtype, n) : 0.0f);
      const int64_t at = static_cast<int64_t>(m) * p.N + n;
      const float res = p.residual != nullptr ? load_as_float(p.residual, p.y_dtype, at) : 0.0f;
      store_from_float(p.y, p.y_dtype, at, finish_value(vb, p.epilogue, p.residual != nullptr, res));
    }
  }
  RG_MARK(7);
}

// y = finish(sum of the k slices' partial sums + bias): one thread per four consecutive output columns
constexpr int kFinishThreads = 256;
__global__ void __launch_bounds__(kFinishThreads) mma_regs_finish_kernel(const RgParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // the partial sums are the output of the kernel before
  const int64_t quads = p.N / 4;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kFinishThreads + threadIdx.x;
  if (i >= p.M * quads) return;
  const int64_t m = i / quads, n = (i - m * quads) * 4;
  const float4* src = reinterpret_cast<const float4*>(p.partial + m * p.N + n);
  const int64_t slice = p.M * quads;   // float4 per k slice
  float4 s = src[0];
  for (int q = 1; q < p.ks; ++q) {
    const float4 v = src[q * slice];
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  const float v4[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float vb = v4[j] + (p.bias != nullptr ? load_as_float(p.bias, p.bias_dtype, n + j) : 0.0f);
    const int64_t at = m * p.N + n + j;
    const float res = p.residual != nullptr ? load_as_float(p.residual, p.y_dtype, at) : 0.0f;
    store_from_float(p.y, p.y_dtype, at, finish_value(vb, p.epilogue, p.residual != nullptr, res));
  }
}

// canonical [N][K] index stream -> tiles of 16 rows x 128 k, [row block][128-k range][row][16 * bits bytes]:
// one 32-bit word per thread
__global__ void linear_prepack_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int bits,
                                      int64_t row_words, int64_t ranges, int64_t total_words) {
  const int64_t wo = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (wo >= total_words) return;
  const int piece = 4 * bits;                  // words of one row of a unit
  const int64_t tile = wo / (16 * piece);
  const int within = static_cast<int>(wo - tile * (16 * piece));
  const int r = within / piece, cw = within - r * piece;
  const int64_t rb = tile / ranges, kr = tile - rb * ranges;
  dst[wo] = src[(rb * 16 + r) * row_words + kr * piece + cw];
}

struct RgPlan {
  int mr, kr, ks, passes, ranges, chunk, chunk_low;
  uint32_t fin_bytes;
  size_t smem;
};

#ifdef DIMQ_B200_DIAG
int g_force_ks = 0;   // k slices at a time, when it divides K / 2048
int g_force_kr = 0;   // k per warp (64 or 128)
uint32_t* g_trace = nullptr;
#endif

template <int BITS>
bool make_rg_plan(int64_t M, int64_t N, int64_t K, RgPlan* out) {
  using T = Tbl<BITS>;
  RgPlan pl{};
  pl.mr = M <= 2 ? 2 : (M <= 4 ? 4 : (M <= 8 ? 8 : 16));   // columns kept of the accumulator tiles
  pl.kr = 128;
#ifdef DIMQ_B200_DIAG
  if (g_force_kr == 64 && BITS != 3 && pl.mr == 8) pl.kr = 64;   // 32 warps of 64 k: measured 30 % slower
#endif
  const int slices = static_cast<int>((K + kCtaK - 1) / kCtaK);   // the last one may be partly empty
  // k slices at a time: the largest divisor of the slice count up to 4, else up to 8, else passes
  int ks = 1;
  for (int d = 1; d <= 4; ++d) if (slices % d == 0) ks = d;
  if (ks == 1) for (int d = 5; d <= kMaxSlices; ++d) if (slices % d == 0) ks = d;
#ifdef DIMQ_B200_DIAG
  if (g_force_ks > 0 && g_force_ks <= kMaxSlices && slices % g_force_ks == 0) ks = g_force_ks;
#endif
  pl.ks = ks;
  pl.passes = slices / ks;
  const int64_t nrb = N / 16;
  const int64_t cl = kNumSMs / ks;
  pl.ranges = static_cast<int>(nrb < cl ? nrb : cl);
  const int64_t max_it = (nrb + pl.ranges - 1) / pl.ranges;
  // shared memory: fin behind the table, the units' partial tiles below the table and behind fin
  const size_t unit = static_cast<size_t>(kCtaK / pl.kr) * 16 * pl.mr * sizeof(float);
  const size_t fin_bytes = static_cast<size_t>(max_it) * 16 * pl.mr * sizeof(float);
  if (T::kEnd + fin_bytes > kSmemWindow) return false;
  const int64_t low = (T::kAddr - kLowPart) / unit;
  const int64_t high = (kSmemWindow - T::kEnd - fin_bytes) / unit;
  if (low + high < 1) return false;
  pl.chunk = static_cast<int>(low + high < max_it ? low + high : max_it);
  pl.chunk_low = static_cast<int>(low < pl.chunk ? low : pl.chunk);
  pl.fin_bytes = static_cast<uint32_t>(fin_bytes);
  pl.smem = T::kEnd + fin_bytes + static_cast<size_t>(pl.chunk - pl.chunk_low) * unit;   // counted from shared address 0
  *out = pl;
  return true;
}

bool rg_plan_for(int bits, int64_t M, int64_t N, int64_t K, RgPlan* plan) {
  switch (bits) {
    case 2: return make_rg_plan<2>(M, N, K, plan);
    case 3: return make_rg_plan<3>(M, N, K, plan);
    case 4: return make_rg_plan<4>(M, N, K, plan);
    default: return false;
  }
}

template <int BITS, int MR, bool F16, int KR>
int launch_rg(RgParams& p, const RgPlan& plan, cudaStream_t st) {
  auto kern = linear_wq_mma_regs_kernel<BITS, MR, F16, KR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemWindow);
  if (e != cudaSuccess) return static_cast<int>(e);
  void* status = nullptr;
  e = cudaGetSymbolAddress(&status, g_rg_status);
  if (e != cudaSuccess) return static_cast<int>(e);
  p.status = static_cast<uint32_t*>(status);
#ifdef DIMQ_B200_DIAG
  p.trace = g_trace;
#endif
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.ranges * plan.ks));   // no CTA waits for another: any order will do
  cfg.blockDim = dim3(kCtaK / KR * 32);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  // programmatic dependent launch: the prologue (first index loads, table) may overlap the tail of the
  // kernel before this one; the kernel waits before it reads the activations or writes anything
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (plan.ks > 1) {
    const int64_t quads = static_cast<int64_t>(p.M) * (p.N / 4);
    cfg.gridDim = dim3(static_cast<unsigned>((quads + kFinishThreads - 1) / kFinishThreads));
    cfg.blockDim = dim3(kFinishThreads);
    cfg.dynamicSmemBytes = 0;
    e = cudaLaunchKernelEx(&cfg, mma_regs_finish_kernel, p);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return launch_status();
}

template <int BITS, bool F16>
int launch_rg_cols(RgParams& p, const RgPlan& plan, cudaStream_t st) {
#ifdef DIMQ_B200_DIAG
  if constexpr (BITS != 3) {
    if (plan.mr == 8 && plan.kr == 64) return launch_rg<BITS, 8, F16, 64>(p, plan, st);
  }
#endif
  switch (plan.mr) {
    case 2: return launch_rg<BITS, 2, F16, 128>(p, plan, st);
    case 4: return launch_rg<BITS, 4, F16, 128>(p, plan, st);
    case 8: return launch_rg<BITS, 8, F16, 128>(p, plan, st);
    default: return launch_rg<BITS, 16, F16, 128>(p, plan, st);
  }
}

template <int BITS>
int launch_rg_bits(RgParams& p, const RgPlan& plan, bool f16, cudaStream_t st) {
  return f16 ? launch_rg_cols<BITS, true>(p, plan, st) : launch_rg_cols<BITS, false>(p, plan, st);
}

}  // namespace

#ifdef DIMQ_B200_DIAG
void set_mma_regs_slices(int ks) { g_force_ks = ks & 0xFF; g_force_kr = ks >> 8; }   // slices | k per warp << 8
void set_mma_regs_trace(uint32_t* trace) { g_trace = trace; }
#endif

// 16-bit activations, M <= 16, N a multiple of 16, K a multiple of 128 and at least 2048, 2-, 3- or 4-bit indices; the
// sums of one CTA's row blocks must fit its shared memory beside the table.
bool mma_regs_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K) {
  if (x_dtype != DIMQ_F16 && x_dtype != DIMQ_BF16) return false;
  if (M < 1 || M > 16 || N < 16 || N % 16 != 0 || K < kCtaK || K % 128 != 0) return false;
  if (w->bits != 2 && w->bits != 3 && w->bits != 4) return false;
  if (w->groups > 1 && w->group_rows % 16 != 0) return false;
  if (!aligned(x, 16) || !aligned(w->packed, 16)) return false;
  if (N > 0x3FFFFFFF || K > 0x3FFFFFFF || N * K * w->bits / 8 > 0x7FFFFFFF) return false;   // 32-bit byte offsets
  RgPlan plan;
  return rg_plan_for(w->bits, M, N, K, &plan);
}

// From 2 MB of indices on this kernel is the faster of the two small-M kernels (4096 -> 1024 at 4 bits:
// 3.6 against 5.4 us at M = 4); below that neither has been seen to win and the older one stays.
bool mma_regs_pays(const dimq_wq_weight* w, int64_t N, int64_t K) {
  return N * K * w->bits >= (int64_t{1} << 24);
}

// bytes of scratch a call needs: the k slices' partial sums, [slices][M][N] floats (0 with one slice)
int64_t mma_regs_workspace_bytes(const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K) {
  RgPlan plan;
  if (!rg_plan_for(w->bits, M, N, K, &plan) || plan.ks == 1) return 0;
  return static_cast<int64_t>(plan.ks) * M * N * static_cast<int64_t>(sizeof(float));
}

int launch_linear_wq_mma_regs(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                              const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                              int epilogue, void* workspace, int64_t workspace_bytes, cudaStream_t st) {
  if (!mma_regs_supported(x, x_dtype, w, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  RgPlan plan;
  if (!rg_plan_for(w->bits, M, N, K, &plan)) return DIMQ_ERR_UNSUPPORTED;
  const int64_t need = mma_regs_workspace_bytes(w, M, N, K);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need)) return DIMQ_ERR_SCRATCH_TOO_SMALL;
  if (need > 0 && !aligned(workspace, 16)) return DIMQ_ERR_ALIGNMENT;
  RgParams p{};
  p.x = x; p.codebooks = w->codebooks;
  p.tiled = (w->packed_khwc != nullptr && aligned(w->packed_khwc, 16)) ? 1 : 0;   // the output of dimq_linear_prepack
  p.packed = p.tiled ? w->packed_khwc : w->packed;
#ifdef DIMQ_B200_DIAG
  if (plan.kr != 128) { p.tiled = 0; p.packed = w->packed; }   // the tiles are cut for 128 k per warp
#endif
  p.cb_dtype = w->cb_dtype; p.entries = w->entries;
  p.group_rbs = w->groups > 1 ? static_cast<int>(w->group_rows / 16) : static_cast<int>(N / 16) + 1;
  p.bias = bias; p.bias_dtype = bias_dtype; p.residual = residual; p.y = y; p.y_dtype = y_dtype;
  p.M = static_cast<int>(M); p.N = N; p.K = K; p.epilogue = epilogue;
  p.row_bytes = K * w->bits / 8;
  p.cvt = (x_dtype == DIMQ_BF16 && w->cb_dtype != DIMQ_BF16) ? 1 : 0;
  p.nrb = static_cast<int>(N / 16); p.ks = plan.ks; p.passes = plan.passes; p.ranges = plan.ranges;
  p.nk = static_cast<int>(K / 128);
  p.partial = static_cast<float*>(workspace);
  p.chunk = plan.chunk; p.chunk_low = plan.chunk_low; p.fin_bytes = plan.fin_bytes;
  const bool f16 = x_dtype == DIMQ_F16 || p.cvt != 0;
  switch (w->bits) {
    case 2: return launch_rg_bits<2>(p, plan, f16, st);
    case 3: return launch_rg_bits<3>(p, plan, f16, st);
    default: return launch_rg_bits<4>(p, plan, f16, st);
  }
}

// Index stream of a Linear weight re-ordered for this kernel: every unit (16 rows x 128 k) contiguous, so
// that a warp's index load is one run of 512 bytes (4-bit) instead of sixteen 16-byte pieces in eight rows.
int launch_linear_prepack(const uint8_t* packed, int bits, int64_t N, int64_t K, uint8_t* out, cudaStream_t st) {
  if (bits != 2 && bits != 3 && bits != 4) return DIMQ_ERR_UNSUPPORTED;
  if (N < 16 || N % 16 != 0 || K < 128 || K % 128 != 0) return DIMQ_ERR_UNSUPPORTED;
  if (!aligned(packed, 4) || !aligned(out, 16)) return DIMQ_ERR_ALIGNMENT;
  const int64_t total_words = N * K * bits / 32;
  const int threads = 256;
  if ((total_words + threads - 1) / threads > 0x7FFFFFFFll) return DIMQ_ERR_TOO_LARGE;
  linear_prepack_kernel<<<static_cast<unsigned>((total_words + threads - 1) / threads), threads, 0, st>>>(
      reinterpret_cast<const uint32_t*>(packed), reinterpret_cast<uint32_t*>(out), bits, K * bits / 32, K / 128,
      total_words);
  return launch_status();
}

// Status word of this kernel (non-zero: the shared-memory window did not start where the fixed layout
// expects it and the launch did nothing); reading clears it.
int read_rg_status(uint32_t* status) {
  cudaError_t e = cudaMemcpyFromSymbol(status, g_rg_status, sizeof(uint32_t));
  if (e != cudaSuccess) return static_cast<int>(e);
  const uint32_t zero = 0;
  e = cudaMemcpyToSymbol(g_rg_status, &zero, sizeof(uint32_t));
  return e == cudaSuccess ? DIMQ_OK : static_cast<int>(e);
}

}  // namespace dimq
