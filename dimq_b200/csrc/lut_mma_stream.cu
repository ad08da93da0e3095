// Small-M weight-only LUT GEMM for 16-bit activations (M <= 32): the index-streaming regime.
//
// The packed indices are read from HBM exactly once: TMA box copies (16 rows x 128..512 k) land in a
// per-warp ring in shared memory, several boxes ahead of the arithmetic; lane 0 of the warp re-arms a
// slot as soon as the warp has copied its words out of it.  The work per weight is one table lookup
// for every TWO weights (four at 2 bits) and a share of a warp-level mma.sync, which stands in for the
// M fused multiply-adds per weight that a SIMT kernel cannot issue fast enough beyond M = 2.  The
// tensor pipe is nowhere near busy here: the kernel is bound by the index stream, the shared-memory
// lookups and instruction issue, so the warp-level MMA is the right tool and the tcgen05 path (which
// would need the weights staged as operands) is not.
//
// Work unit: 16 output rows x 128 k.  Lane (g = lane / 4, t = lane % 4) of a warp takes, for rows g
// and g + 8 of the block, the 32 consecutive indices k = 32 t .. 32 t + 31 of the chunk (16 B at
// 4 bits, 12 B at 3 bits, 8 B at 2 bits) out of the unit's ring slot.  Because a dot product does not
// care about the order of k, MMA step s (of 8) takes from every lane its indices 4 s .. 4 s + 3: the
// A fragment registers a0/a2 (row g) and a1/a3 (row g + 8) each hold two k-adjacent codewords, which
// is exactly one entry of a PAIR table indexed by the two packed indices (one byte of a 4-bit stream,
// six bits of a 3-bit stream; at 2 bits one byte gives a0 and a2 together).  The pair table is stored
// once per lane ([entry][lane]), so a lookup never has a bank conflict whatever the indices are, and
// it sits on a boundary of its own size, so a lookup address is (index bits masked in place) | base.
// The matching B fragments of two steps are x[m = g][32 t + 8 (s / 2) .. + 7]: one 16-byte read of the
// activations, staged in shared memory in [chunk][s / 2][t][8] order with a row stride of 2 K + 64
// bytes, which puts the eight lanes of a quarter-warp on distinct banks; MMA columns beyond M read a
// chunk of zeros.
//
// A CTA has 16 compute warps and 2 write-back warps.  It works on G row blocks at a time (G > 1 only
// when K has fewer than 16 chunks); every compute warp owns a fixed run of k chunks of one of them,
// so a unit costs a pointer increment.  The partial sums of a row block's warps go to per-warp
// buffers (double-buffered); after one __syncthreads per iteration the write-back warps add them,
// apply bias / epilogue / residual and store y while the compute warps are already on the next row
// blocks.  Every wait on a ring slot is bounded; a warp that gives up sets a flag and a status word.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "mma_small.cuh"

namespace dimq {
int encode_plain_tensor_map(void* out, int elem_bytes, int rank, const void* base, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box);

namespace {

using namespace small_m;

constexpr int kWarps = 16;
constexpr int kWriteWarps = 2;  // warps that only add the partial sums and write y, off the compute warps' path
constexpr int kThreads = (kWarps + kWriteWarps) * 32;
constexpr int kChunkK = 128;

// Absolute shared-memory addresses.  The lookup table sits on a boundary of its own size so that a
// lookup address is (index bits, masked in place) OR (table base | lane offset): no add.
//   [start, table)    codewords of the current group, mbarriers, the first activation rows
//   [table, +size)    pair table, one copy per lane
//   [table + size, )  the other activation rows, per-warp partial sums, per-warp index rings
template <int BITS>
struct Cfg {
  static constexpr int kWords = BITS;  // 32 indices per lane, row and unit
  static constexpr uint32_t kUnitBytes = 16 * kChunkK * BITS / 8;  // one ring slot: [16 rows][128 k]
  static constexpr int kEntryWords = PairTable<BITS>::kEntryWords;
  static constexpr uint32_t kTableBytes = PairTable<BITS>::kBytes;
  static constexpr uint32_t kTableAddr = PairTable<BITS>::kAddr;
  static constexpr uint32_t kXAddr = kTableAddr + kTableBytes;
};

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
  int wpr;       // warps per row block
  int cpw;       // consecutive k chunks per warp
  int chunks;    // K / 128
  int total_it;  // ceil(ceil(N / 16) / G)
  int ipc;       // iterations per CTA
  int xs;        // activation row stride in shared memory, elements
  int rows_low;  // activation rows 0 .. rows_low-1 live below the table (at x_low), the rest above it
  uint32_t x_low;  // shared address of row 0 when rows_low > 0
  uint32_t x_high; // shared address of row rows_low
  uint32_t zero;   // shared address of 256 zero bytes (the activations of MMA columns beyond M)
  uint32_t scale;  // shared address of 32 floats: per-row factor of the converting mode (else unused)
  int cvt;         // 1: x is bf16 in global memory and is converted to fp16 while it is staged
  int pf;          // ring slots per warp
  int bw;          // units (k chunks) per TMA box and ring slot: 1, 2 or 4
  uint32_t part;   // shared address of the partial sums: [2][warp][16 rows][MR]
  uint32_t ring;   // shared address of the rings: [warp][pf][unit]
  uint32_t bars;   // shared address of the slots' mbarriers: [warp][pf]
  uint32_t* status;  // device status word (set when the shared-memory window is not where it is expected)
};

static __device__ uint32_t g_ms_status;

// One lane of a converged warp: TMA copies are issued under this predicate from warp-uniform control
// flow (issued from a `lane == 0` branch the same instruction costs several times more issue time).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred px;\n\t"
      "elect.sync _|px, 0xFFFFFFFF;\n\t"
      "@px mov.s32 %0, 1;\n\t"
      "}\n"
      : "+r"(pred));
  return pred != 0;
}

constexpr uint32_t kPollLimit = 1u << 15;  // bounded wait: polls of up to 20 us each, then give up
constexpr uint32_t kPollHintNs = 20000u;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kPollHintNs)
      : "memory");
  return ok != 0;
}
// TMA box copy of a [16 rows][chunk bytes] tile of the packed index matrix into this CTA's shared memory
__device__ __forceinline__ void tma_load_unit(uint32_t dst, const CUtensorMap* map, uint32_t bar, int byte0, int row0) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(byte0), "r"(row0)
      : "memory");
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

template <int BITS, int NB, bool F16>
__global__ void __launch_bounds__(kThreads, 1)
linear_wq_mma_stream_kernel(const __grid_constant__ CUtensorMap wmap, const MsParams p) {
  using C = Cfg<BITS>;
  constexpr int W = C::kWords;
  constexpr int MR = 8 * NB;  // columns of the MMA tiles (activation rows, M rounded up)
  extern __shared__ __align__(16) unsigned char smem[];
  const uint32_t s0 = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  if (s0 > kLowStart) {  // the fixed layout below would not fit the window: report, do nothing
    if (threadIdx.x == 0) atomicOr(p.status, 0x80000901u);
    return;
  }
  unsigned char* const abs0 = smem - s0;  // generic address of shared address 0
  float* cb_s = reinterpret_cast<float*>(abs0 + kLowStart);                  // codewords of the current group
  float* part = reinterpret_cast<float*>(abs0 + p.part);                     // [2][warp][16 rows][MR]
  uint32_t* table = reinterpret_cast<uint32_t*>(abs0 + C::kTableAddr);
  // shared address of activation row m
  auto x_row_addr = [&](int m) -> uint32_t {
    return m < p.rows_low ? p.x_low + static_cast<uint32_t>(m) * p.xs * 2
                          : p.x_high + static_cast<uint32_t>(m - p.rows_low) * p.xs * 2;
  };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int it_begin = blockIdx.x * p.ipc;
  const int it_end = min(it_begin + p.ipc, p.total_it);
  const int my_iters = it_end - it_begin;
  if (my_iters <= 0) return;

  // the first group's codewords: the global load flies while the barriers are set up and the first
  // copies are issued
  const int64_t first_group = (static_cast<int64_t>(it_begin) * p.G * 16) / p.group_rows;
  float first_cb = 0.0f;
  if (tid < (1 << BITS) && tid < p.entries)
    first_cb = load_as_float(p.codebooks, p.cb_dtype, first_group * p.entries + tid);

  // ---- this warp's share: row block `slot` of every iteration, k chunks [c0, c0 + nch) ----
  const int slot = warp / p.wpr;
  const int c0 = (warp - slot * p.wpr) * p.cpw;
  const int nch = (warp < kWarps && slot < p.G) ? max(0, min(p.cpw, p.chunks - c0)) : 0;


  // ---- the warp's ring: p.pf slots of one unit each, one mbarrier per slot; lane 0 issues the copies ----
  constexpr int kChunkBytes = kChunkK * BITS / 8;  // per row
  const uint32_t ring_w = p.ring + warp * p.pf * p.bw * C::kUnitBytes;
  const uint32_t bars_w = p.bars + warp * p.pf * 8;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(abs0 + p.bars + kWarps * p.pf * 8);
  const int total = my_iters * nch;
  int ld_seq = 0, ld_j = 0, ld_slot = 0;
  int ld_row0 = (it_begin * p.G + slot) * 16;
  int pr_j = 0, pr_it = it_begin, pr_slot = 0;
  uint32_t pr_phase = 0;
  bool seq_live = true;  // false once a wait of this warp gave up

  // issue the copy of the next box of the sequence: p.bw consecutive chunks of the 16 rows (lane 0
  // only; the slot must be free)
  const uint32_t slot_bytes = p.bw * C::kUnitBytes;
  auto issue_unit = [&]() {   // whole warp: every lane keeps the cursor, one elected lane issues
    const uint32_t bar = bars_w + ld_slot * 8;
    if (elect_one()) {
      mbar_expect_tx(bar, slot_bytes);
      tma_load_unit(ring_w + ld_slot * slot_bytes, &wmap, bar, (c0 + ld_j) * kChunkBytes, ld_row0);
    }
    __syncwarp();
    ld_seq += p.bw;
    if (++ld_slot == p.pf) ld_slot = 0;
    ld_j += p.bw;
    if (ld_j == nch) {
      ld_j = 0;
      ld_row0 += p.G * 16;
    }
  };
  // The kernel that follows in the stream may start its own prologue now (programmatic dependent
  // launch): everything up to the activation staging below reads only weights and codebooks.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (nch > 0) {
    if (lane == 0) {
      for (int q = 0; q < p.pf; ++q) mbar_init(bars_w + q * 8, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // the first copies fly while the activations and the table are being set up
    for (int q = 0; q < p.pf && ld_seq < total; ++q) issue_unit();  // ld_seq counts units
  }
  if (tid == 0) *abort_flag = 0u;

  float* row_scale = reinterpret_cast<float*>(abs0 + p.scale);
  // ---- one-time staging of the activations (after the table, below): asynchronous copies, or, in the
  // converting mode, bf16 -> fp16 on the way (the codebook is fp16 / fp32, so the MMAs run in fp16) ----
  auto stage_activations = [&]() {
    // 16-byte group v = k / 8 of a row is [chunk | t (2 bits) | s / 2 (2 bits)]; it is stored at
    // [chunk | s / 2 | t], so that a pair of MMA steps finds the four lanes of a quad in adjacent slots
    const int vec_per_row = static_cast<int>(p.K >> 3);  // 8 elements = 16 bytes
    const uint4* xg = static_cast<const uint4*>(p.x);
    if (!p.cvt) {
      for (int m = 0; m < p.M; ++m) {
        const uint32_t row = x_row_addr(m);
        const uint4* src = xg + static_cast<int64_t>(m) * vec_per_row;
        for (int v = tid; v < vec_per_row; v += kThreads) {
          const int dv = (v & ~15) | ((v & 3) << 2) | ((v >> 2) & 3);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(row + dv * 16), "l"(src + v) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      return;
    }
    // Converting mode.  bf16 -> fp16 is exact for 6.1e-5 <= |x| <= 65504.  Pass 1 converts as is and
    // notes per row whether a finite value exceeds 2^15, whether any reaches 2^-10 and whether any is
    // non-zero.  A row that is too large, or non-zero but tiny throughout, is staged again scaled by a
    // power of two that brings its largest finite magnitude to [2^14, 2^15) (exact), and the write-back
    // multiplies its sums by the inverse: elements more than 2^29 below the row maximum lose bits, far
    // under the rounding of the fp32 accumulation.  All rows' vectors form one index space, four loads in
    // flight per thread.
    uint32_t* flags = reinterpret_cast<uint32_t*>(row_scale);   // per row: bit 0 too large, bit 1 some >= 2^-10, bit 2 non-zero
    if (tid < 32) flags[tid] = 0u;
    __syncthreads();
    const int total_vec = p.M * vec_per_row;
    auto convert_store = [&](int i, const uint4& q, float f, uint32_t& note) {
      const int m = i / vec_per_row, v = i - m * vec_per_row;
      const int dv = (v & ~15) | ((v & 3) << 2) | ((v >> 2) & 3);
      const uint32_t in[4] = {q.x, q.y, q.z, q.w};
      uint32_t out[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xy = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in[j]));
        xy.x *= f; xy.y *= f;
        const float a = fmaxf(fabsf(xy.x) < 3.0e38f ? fabsf(xy.x) : 0.0f, fabsf(xy.y) < 3.0e38f ? fabsf(xy.y) : 0.0f);
        note |= (a > 32768.0f ? 1u : 0u) | (a >= 0.0009765625f ? 2u : 0u) | (a > 0.0f ? 4u : 0u);
        const __half2 h = __float22half2_rn(xy);
        out[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(abs0 + x_row_addr(m) + dv * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    };
    for (int i0 = tid; i0 < total_vec; i0 += 4 * kThreads) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * kThreads < total_vec) q[u] = __ldg(xg + i0 + u * kThreads);   // rows are contiguous: [M][K]
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kThreads;
        if (i < total_vec) {
          uint32_t note = 0u;
          convert_store(i, q[u], 1.0f, note);
          const int m = i / vec_per_row;
          if ((flags[m] | note) != flags[m]) atomicOr(flags + m, note);
        }
      }
    }
    __syncthreads();
    bool redo = false;
    if (tid < 32 && tid < p.M) redo = (flags[tid] & 1u) != 0u || (flags[tid] & 6u) == 4u;
    if (__syncthreads_or(redo ? 1 : 0)) {
      // rare path: the rows that need it get their largest finite magnitude, then a power-of-two factor
      // scratch of this path: the start of the partial-sum buffers, not in use before the main loop
      uint32_t* row_max = reinterpret_cast<uint32_t*>(part);
      float* row_factor = part + 32;
      if (tid < 32) row_max[tid] = 0u;
      __syncthreads();
      for (int i = tid; i < total_vec; i += kThreads) {
        const int m = i / vec_per_row;
        if ((flags[m] & 1u) == 0u && (flags[m] & 6u) != 4u) continue;
        const uint4 q = __ldg(xg + i);
        const uint32_t in[4] = {q.x, q.y, q.z, q.w};
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xy = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in[j]));
          if (fabsf(xy.x) < 3.0e38f) a = fmaxf(a, fabsf(xy.x));
          if (fabsf(xy.y) < 3.0e38f) a = fmaxf(a, fabsf(xy.y));
        }
        if (a > 0.0f) atomicMax(row_max + m, __float_as_uint(a));   // non-negative floats order like their bits
      }
      __syncthreads();
      if (tid < 32) {
        float f = 1.0f;
        const float mx = __uint_as_float(row_max[tid]);
        if (mx > 0.0f) {
          int e;
          frexpf(mx, &e);               // mx = frac * 2^e, frac in [0.5, 1)
          f = ldexpf(1.0f, 15 - e);     // mx * f in [2^14, 2^15)
        }
        row_factor[tid] = f;
      }
      __syncthreads();
      for (int i = tid; i < total_vec; i += kThreads) {
        const int m = i / vec_per_row;
        if (row_factor[m] == 1.0f) continue;
        uint32_t note = 0u;
        convert_store(i, __ldg(xg + i), row_factor[m], note);
      }
      __syncthreads();
      if (tid < 32) row_scale[tid] = 1.0f / row_factor[tid];   // what the row's sums are multiplied by
    } else if (tid < 32) {
      row_scale[tid] = 1.0f;
    }
  };
  if (tid < 16) reinterpret_cast<uint4*>(abs0 + p.zero)[tid] = make_uint4(0u, 0u, 0u, 0u);

  // pair table of one codebook group, one copy per lane: word (entry * 32 + lane)
  auto build_table = [&](int64_t group, bool preloaded) {
    if (tid < (1 << BITS)) {
      if (preloaded) cb_s[tid] = first_cb;
      else cb_s[tid] = tid < p.entries ? load_as_float(p.codebooks, p.cb_dtype, group * p.entries + tid) : 0.0f;
    }
    __syncthreads();
    fill_pair_table<BITS, F16>(reinterpret_cast<uint4*>(table), cb_s, tid, kThreads);
  };
  auto group_of_iteration = [&](int it) -> int64_t {
    return (static_cast<int64_t>(it) * p.G * 16) / p.group_rows;
  };
  int64_t cur_group = first_group;
  build_table(cur_group, true);
  // the activations may be the output of the kernel before this one in the stream: wait for it
  asm volatile("griddepcontrol.wait;" ::: "memory");
  stage_activations();
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();

  // two accumulator sets (even / odd MMA steps) halve the dependent chain through the MMAs
  float acc[2][NB][4];
#pragma unroll
  for (int e = 0; e < 2; ++e)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[e][nb][j] = 0.0f;

  // The warp's partial sums of its row block go to its own buffer (no atomics: with all warps of a row
  // block adding into the same words at the same moment, shared-memory float adds serialise badly).
  auto flush = [&](int it) {
    float* s = part + (static_cast<size_t>(it & 1) * kWarps + warp) * (16 * MR);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int m = nb * 8 + 2 * t;
      *reinterpret_cast<float2*>(s + g * MR + m) =
          make_float2(acc[0][nb][0] + acc[1][nb][0], acc[0][nb][1] + acc[1][nb][1]);
      *reinterpret_cast<float2*>(s + (g + 8) * MR + m) =
          make_float2(acc[0][nb][2] + acc[1][nb][2], acc[0][nb][3] + acc[1][nb][3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[0][nb][j] = acc[1][nb][j] = 0.0f;
    }
  };

  // after the iteration's __syncthreads: sum the partials of each row block's warps, then bias,
  // epilogue, residual, store
  auto write_iteration = [&](int it) {
    const float* base = part + static_cast<size_t>(it & 1) * kWarps * (16 * MR);
    const int total_out = p.G * MR * 16;
    for (int idx = tid - kWarps * 32; idx < total_out; idx += kWriteWarps * 32) {
      const int r = idx & 15;
      const int m = (idx >> 4) % MR;
      const int sl = idx / (MR * 16);
      const float* src = base + static_cast<size_t>(sl) * p.wpr * (16 * MR) + r * MR + m;
      float v = 0.0f;
      for (int wi = 0; wi < p.wpr; ++wi) v += src[wi * (16 * MR)];
      if (p.cvt && m < p.M) v *= row_scale[m];
      const int64_t n = (static_cast<int64_t>(it) * p.G + sl) * 16 + r;
      if (m < p.M && n < p.N) {
        const float vb = v + (p.bias != nullptr ? load_as_float(p.bias, p.bias_dtype, n) : 0.0f);
        const int64_t o = static_cast<int64_t>(m) * p.N + n;
        const float res = p.residual != nullptr ? load_as_float(p.residual, p.y_dtype, o) : 0.0f;
        store_from_float(p.y, p.y_dtype, o, finish_value(vb, p.epilogue, p.residual != nullptr, res));
      }
    }
  };

  // Every warp of the CTA passes here once per iteration, in the same order.  The write-back warps read
  // buffer it & 1 after this barrier and reach the next one only when they are done, so the compute
  // warps cannot overwrite that buffer (iteration it + 2) before it has been read.
  auto end_iteration = [&](int it) {
    __syncthreads();
    if (warp >= kWarps) write_iteration(it);
    if (it + 1 < it_end) {
      const int64_t ng = group_of_iteration(it + 1);
      if (ng != cur_group) {  // uniform over the CTA: nobody reads the table between the barriers
        cur_group = ng;
        build_table(ng, false);
        __syncthreads();
      }
    }
  };

  if (nch == 0) {  // the write-back warps, and compute warps without chunks: only the barriers
    for (int it = it_begin; it < it_end; ++it) end_iteration(it);
    return;
  }

  // lookup address = (index bits masked in place) | tbl: the table base has those bits clear
  const uint32_t tbl = C::kTableAddr + lane * (4 * C::kEntryWords);
  // B fragments: column n = g of MMA tile nb is activation row nb * 8 + g; columns beyond M read a
  // chunk of zeros (and do not advance with the k chunk)
  uint32_t xrow[NB], xstep[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = nb * 8 + g;
    const bool live = m < p.M;
    xrow[nb] = live ? x_row_addr(m) + 16 * t + c0 * (kChunkK * 2) : p.zero + 16 * t;
    xstep[nb] = live ? kChunkK * 2 : 0;
  }

  // Unit `sub` of the current box: wait (bounded) for the box when it is its first unit, copy the lane's
  // indices out, and re-arm the slot after its last unit.  Returns false when there is no data (a wait
  // gave up here or elsewhere in the CTA).
  int sub = 0;
  bool box_ok = false;
  const uint32_t row_pitch = p.bw * kChunkBytes;  // bytes between rows inside a slot
  auto fetch_unit = [&](uint32_t (&buf)[2][W]) -> bool {
    if (sub == 0) {
      const uint32_t bar = bars_w + pr_slot * 8;
      box_ok = seq_live && mbar_test_wait(bar, pr_phase);  // usually the copy landed long ago
      if (!box_ok && seq_live) {
        for (uint32_t poll = 0; poll < kPollLimit; ++poll) {
          if (mbar_try_wait(bar, pr_phase)) { box_ok = true; break; }
          if ((poll & 63u) == 63u && *abort_flag != 0u) break;
        }
        if (!box_ok) {  // give up: no more copies are issued by this warp, the units left are skipped
          *abort_flag = 1u;
          atomicOr(p.status, 0x80000902u);
          seq_live = false;
        }
      }
      // the lanes poll the same barrier but may read the abort flag at different moments: agree
      box_ok = __all_sync(0xFFFFFFFFu, box_ok);
      if (!box_ok) seq_live = false;
    }
    const uint32_t src = ring_w + pr_slot * slot_bytes + g * row_pitch + sub * kChunkBytes + t * (4 * BITS);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t a = src + h * 8 * row_pitch;
      if constexpr (BITS == 4) {
        const uint4 q = lds_u128(a);
        buf[h][0] = q.x; buf[h][1] = q.y; buf[h][2] = q.z; buf[h][3] = q.w;
      } else if constexpr (BITS == 2) {
        const uint2 q = lds_u64(a);
        buf[h][0] = q.x; buf[h][1] = q.y;
      } else {
#pragma unroll
        for (int j = 0; j < W; ++j) buf[h][j] = lds_u32(a + 4 * j);
      }
    }
    if (++sub == p.bw) {
      sub = 0;
      __syncwarp();  // every lane has its words of the last unit: the slot may be overwritten
      if (box_ok && ld_seq < total) issue_unit();
      if (++pr_slot == p.pf) { pr_slot = 0; pr_phase ^= 1u; }
    }
    return box_ok;
  };

  // eight MMA steps over the 128 k of one unit
  auto process = [&](const uint32_t (&buf)[2][W]) {
    uint4 bfrag[NB];
    static_for<0, 8>([&](auto sc) {
      constexpr int s = decltype(sc)::value;
      uint32_t a0, a1, a2, a3;
      lookup_step<BITS, s>(buf[0], buf[1], tbl, a0, a1, a2, a3);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        if constexpr (s % 2 == 0) bfrag[nb] = lds_u128(xrow[nb] + pr_j * xstep[nb] + 32 * s);  // steps s, s + 1
        if constexpr (s % 2 == 0) mma_16816<F16>(acc[0][nb], a0, a1, a2, a3, bfrag[nb].x, bfrag[nb].y);
        else mma_16816<F16>(acc[1][nb], a0, a1, a2, a3, bfrag[nb].z, bfrag[nb].w);
      }
    });
  };

  for (int seq = 0; seq < total; ++seq) {
    uint32_t buf[2][W];
    if (fetch_unit(buf)) process(buf);
    if (++pr_j == nch) {
      pr_j = 0;
      flush(pr_it);
      end_iteration(pr_it);
      ++pr_it;
    }
  }
  // Only after a wait gave up: copies of this warp may still be in flight; give each a last bounded
  // chance to land before the CTA's shared memory is released.
  if (*abort_flag != 0u && lane == 0) {
    for (int q = 0; q < p.pf; ++q)
      for (uint32_t poll = 0; poll < 1024u; ++poll)
        if (mbar_try_wait(bars_w + q * 8, pr_phase) || mbar_try_wait(bars_w + q * 8, pr_phase ^ 1u)) break;
  }
}

struct Plan {
  int G, wpr, cpw, chunks, total_it, ipc, ctas, nb, rows_low, pf, bw;
  uint32_t x_low, x_high, ring, bars, part, zero, scale;
  size_t smem;
};

template <int BITS>
bool make_plan(const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K, Plan* out) {
  using C = Cfg<BITS>;
  Plan bp{};
  bp.nb = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  bp.chunks = static_cast<int>(K / kChunkK);
  if (bp.chunks >= kWarps) {  // one row block at a time, every warp a run of consecutive chunks
    bp.G = 1;
    bp.cpw = (bp.chunks + kWarps - 1) / kWarps;
    bp.wpr = (bp.chunks + bp.cpw - 1) / bp.cpw;
  } else {  // several row blocks at a time, one chunk per warp
    bp.cpw = 1;
    bp.wpr = bp.chunks;
    bp.G = kWarps / bp.chunks;
    // all row blocks of an iteration use one codebook
    while (bp.G > 1 && w->groups > 1 && w->group_rows % (16 * bp.G) != 0) --bp.G;
    // a small problem is better spread over more CTAs
    const int64_t row_blocks = (N + 15) / 16;
    while (bp.G > 1 && (row_blocks + bp.G - 1) / bp.G < kNumSMs) --bp.G;
    while (bp.G > 1 && w->groups > 1 && w->group_rows % (16 * bp.G) != 0) --bp.G;
  }
  const int64_t row_blocks = (N + 15) / 16;
  const int64_t total_it = (row_blocks + bp.G - 1) / bp.G;
  if (total_it > 0x3FFFFFF) return false;
  const int64_t ctas0 = total_it < kNumSMs ? total_it : kNumSMs;
  bp.ipc = static_cast<int>((total_it + ctas0 - 1) / ctas0);
  bp.total_it = static_cast<int>(total_it);
  bp.ctas = static_cast<int>((total_it + bp.ipc - 1) / bp.ipc);
  // fixed layout (absolute shared addresses): codewords, mbarriers and the first activation rows below
  // the table; the other activation rows, the partial sums and the rings above it
  constexpr int kMaxPf = 8;
  const size_t low = sizeof(float) * 16;  // codewords
  bp.bars = static_cast<uint32_t>(kLowStart + low);
  bp.zero = static_cast<uint32_t>((bp.bars + kWarps * kMaxPf * 8 + 16 + 127) & ~size_t(127));  // after the abort flag
  bp.scale = bp.zero + 256;                    // 32 per-row factors of the converting mode
  const size_t low_end = bp.scale + 128;
  if (low_end > C::kTableAddr) return false;
  // row stride 2 K + 64 bytes: the eight lanes of a quarter-warp (two rows x four 16-byte slots) cover
  // 128 consecutive bytes modulo the bank width
  const size_t row = (static_cast<size_t>(K) + 32) * 2;
  bp.x_low = static_cast<uint32_t>((low_end + 127) & ~size_t(127));
  const size_t rows = static_cast<size_t>(M);
  size_t rows_low = bp.x_low < C::kTableAddr ? (C::kTableAddr - bp.x_low) / row : 0;
  if (rows_low > rows) rows_low = rows;
  bp.rows_low = static_cast<int>(rows_low);
  // rows above the table continue the same bank pattern (64 bytes per row modulo 128)
  bp.x_high = C::kXAddr + static_cast<uint32_t>((rows_low % 2) * 64);
  const size_t x_end = bp.x_high + (rows - rows_low) * row;
  bp.part = static_cast<uint32_t>((x_end + 127) & ~size_t(127));
  const size_t part_bytes = sizeof(float) * 2 * kWarps * 16 * 8 * bp.nb;
  bp.ring = static_cast<uint32_t>((bp.part + part_bytes + 127) & ~size_t(127));
  // units per TMA box: several consecutive chunks when every warp owns the same whole number of them
  bp.bw = 1;
  if (bp.chunks % bp.cpw == 0) bp.bw = bp.cpw % 4 == 0 ? 4 : (bp.cpw % 2 == 0 ? 2 : 1);
  while (bp.bw > 1 && bp.ring + 2 * kWarps * bp.bw * C::kUnitBytes > kSmemWindow) bp.bw /= 2;
  const size_t slot_bytes = static_cast<size_t>(bp.bw) * C::kUnitBytes;
  if (bp.ring + kWarps * slot_bytes > kSmemWindow) return false;  // at least one slot per warp
  size_t pf = (kSmemWindow - bp.ring) / (kWarps * slot_bytes);
  bp.pf = static_cast<int>(pf > kMaxPf ? kMaxPf : pf);
  bp.smem = bp.ring + static_cast<size_t>(bp.pf) * kWarps * slot_bytes;  // counted from shared address 0
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
int launch_one(const CUtensorMap& wmap, MsParams& p, const Plan& plan, cudaStream_t st) {
  auto kern = linear_wq_mma_stream_kernel<BITS, NB, F16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemWindow);
  if (e != cudaSuccess) return static_cast<int>(e);
  void* status = nullptr;
  e = cudaGetSymbolAddress(&status, g_ms_status);
  if (e != cudaSuccess) return static_cast<int>(e);
  p.status = static_cast<uint32_t*>(status);
  // programmatic dependent launch: this kernel's prologue (barriers, first index copies, table) may
  // overlap the tail of the kernel before it in the stream; it waits (griddepcontrol.wait) before it
  // reads the activations or writes anything
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.ctas));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, wmap, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_status();
}

template <int BITS>
int launch_bits(const CUtensorMap& wmap, MsParams& p, const Plan& plan, bool f16, cudaStream_t st) {
  switch (plan.nb) {
    case 1: return f16 ? launch_one<BITS, 1, true>(wmap, p, plan, st) : launch_one<BITS, 1, false>(wmap, p, plan, st);
    case 2: return f16 ? launch_one<BITS, 2, true>(wmap, p, plan, st) : launch_one<BITS, 2, false>(wmap, p, plan, st);
    default: return f16 ? launch_one<BITS, 4, true>(wmap, p, plan, st) : launch_one<BITS, 4, false>(wmap, p, plan, st);
  }
}

}  // namespace

// 16-bit activations, M <= 32, K a multiple of 128, 2-, 3- or 4-bit indices.  fp16 activations run
// fp16 MMAs, bf16 activations with a bf16 codebook bf16 MMAs; bf16 activations with an fp16 / fp32
// codebook (what the reference's packed export stores) are converted to fp16 while they are staged.
bool mma_stream_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K) {
  if (x_dtype != DIMQ_F16 && x_dtype != DIMQ_BF16) return false;
  if (M < 1 || M > 32 || N < 1 || K < kChunkK || K % kChunkK != 0) return false;
  if (w->bits != 2 && w->bits != 3 && w->bits != 4) return false;
  if (w->groups > 1 && w->group_rows % 16 != 0) return false;
  if (!aligned(x, 8) || !aligned(w->packed, 16)) return false;
  if (N > 0x3FFFFFFF) return false;
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
  p.G = plan.G; p.wpr = plan.wpr; p.cpw = plan.cpw; p.chunks = plan.chunks; p.total_it = plan.total_it;
  p.ipc = plan.ipc; p.xs = static_cast<int>(K) + 32; p.rows_low = plan.rows_low; p.x_low = plan.x_low; p.x_high = plan.x_high;
  p.pf = plan.pf; p.bw = plan.bw; p.ring = plan.ring; p.bars = plan.bars; p.part = plan.part; p.zero = plan.zero;
  p.scale = plan.scale;
  p.cvt = (x_dtype == DIMQ_BF16 && w->cb_dtype != DIMQ_BF16) ? 1 : 0;
  // the packed index matrix as [N rows][K * bits / 8 bytes]; one box = one unit (16 rows x 128 k)
  CUtensorMap wmap;
  const uint64_t row_bytes = static_cast<uint64_t>(K) * w->bits / 8;
  const uint64_t dims[2] = {row_bytes, static_cast<uint64_t>(N)};
  const uint64_t strides[1] = {row_bytes};
  const uint32_t box[2] = {static_cast<uint32_t>(plan.bw * kChunkK * w->bits / 8), 16u};
  const int rc = encode_plain_tensor_map(&wmap, 1, 2, w->packed, dims, strides, box);
  if (rc != DIMQ_OK) return rc;
  const bool f16 = x_dtype == DIMQ_F16 || p.cvt != 0;
  switch (w->bits) {
    case 2: return launch_bits<2>(wmap, p, plan, f16, st);
    case 3: return launch_bits<3>(wmap, p, plan, f16, st);
    default: return launch_bits<4>(wmap, p, plan, f16, st);
  }
}

// Status word of this kernel (non-zero: the shared-memory window did not start where the fixed layout
// expects it and the launch did nothing); reading clears it.
int read_ms_status(uint32_t* status) {
  cudaError_t e = cudaMemcpyFromSymbol(status, g_ms_status, sizeof(uint32_t));
  if (e != cudaSuccess) return static_cast<int>(e);
  const uint32_t zero = 0;
  e = cudaMemcpyToSymbol(g_ms_status, &zero, sizeof(uint32_t));
  return e == cudaSuccess ? DIMQ_OK : static_cast<int>(e);
}

}  // namespace dimq
