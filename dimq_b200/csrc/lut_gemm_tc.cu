// Weight-only LUT GEMM on the 5th-generation tensor cores (tcgen05), for large M.
//
//   y[m][n] = sum_k x[m][k] * C[g(n)][idx(n, k)]
//
// The quantised weight is the *A* operand and lives in tensor memory: a tile is
// 128 weight rows (= 128 TMEM lanes) x 64 k per pipeline stage.  Dequantisation
// warps stream the packed indices of "their" row straight from global memory
// (one vector load per thread per stage), look pairs of indices up in a
// shared-memory table of packed 16-bit codeword pairs and write the result with
// tcgen05.st — the dequantised weight never touches shared memory.  The
// activations are the *B* operand: TMA (no multicast) stages [kTileX rows x 64 k]
// tiles with the 128-byte swizzle.  One thread issues tcgen05.mma (A from TMEM, B
// from shared memory), accumulating fp32 D[128 weight rows x kTileX activation
// rows] in TMEM, double-buffered so the epilogue of one tile overlaps the main
// loop of the next.  The accumulator is y-transposed: lane = output feature n,
// column = activation row m, so each epilogue warp store writes 32 consecutive n
// of one m (a 128-byte segment in fp32).
//
// Warp roles (576 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM
// allocator, warps 2-9 epilogue (two per TMEM lane quarter), warps 10-17
// dequantisation (two groups of four).  Persistent grid: one CTA per SM walks
// tiles blockIdx.x, blockIdx.x + gridDim.x, ...
//
// Building with -DDIMQ_B200_DIAG adds per-role cycle counters and role-skipping
// switches (set through dimq_diag_configure, an entry point that exists only in
// that build); the default build has neither.
#include <cstdlib>
#include <cstring>

#include "tc_common.cuh"

namespace dimq {
namespace {

using namespace tc;

constexpr int kTileW = 128;      // weight rows per tile (UMMA M)
constexpr int kTileX = 192;      // activation rows per tile (UMMA N)
constexpr int kBlockK = 64;      // k per stage: 128 bytes of 16-bit elements
constexpr int kXStages = 8;      // upper bound of shared-memory stages of the activation tile (p.x_stages are used)
constexpr int kWStages = 4;      // tensor-memory stages of the dequantised weight tile (2 in split mode)
constexpr int kAccStages = 2;    // accumulator buffers
constexpr int kTmemCols = 512;
constexpr int kAccCol = 0;                         // accumulators: columns [0, 2*kTileX)
constexpr int kWCol = kAccStages * kTileX;         // weight stages: 32 columns each
static_assert(kWCol + kWStages * (kBlockK / 2) <= kTmemCols, "TMEM layout");
constexpr int kXStageBytes = kTileX * kBlockK * 2;  // 24 KB
constexpr int kNumDequantGroups = 2;   // each group of 4 warps (one per TMEM lane quarter) takes every 2nd stage
constexpr int kNumDequantWarps = 4 * kNumDequantGroups;
constexpr int kRepWords = 2048;          // replicated lookup table of one dequantisation group (8 KB)
constexpr int kNumEpilogueWarps = 8;   // two per TMEM lane quarter, alternating 32-column chunks
constexpr int kThreads = (2 + kNumEpilogueWarps + kNumDequantWarps) * 32;
constexpr int kMaxTableBytes = 40 * 1024;

struct TcParams {
  const uint8_t* packed;      // [N][K] indices, `bits` wide, rows contiguous
  const void* codebooks;      // [groups][entries]
  int cb_dtype, entries;
  int64_t groups, group_rows;
  const void* bias;           // [N] or null
  int bias_dtype;
  const void* residual;       // [M][N] like y, or null
  void* y;
  int y_dtype;
  int64_t M, N, K;
  int epilogue;
  int w_fmt;                  // operand format of the dequantised weight: 0 fp16, 1 bf16.  In split
                              // mode (bf16 only) every codeword c is carried as hi = bf16(c) and
                              // lo = bf16(c - hi) and each k-step issues two MMAs, so the product is
                              // exact to ~2^-17 although the operands are bf16.
  uint32_t idesc;
  int m_tiles, n_tiles;
  int x_stages;               // activation stages that fit shared memory (3..kXStages)
  int tx;                     // activation rows per tile (UMMA N): 192 for the GEMM, 16..192 for conv
  uint32_t x_stage_bytes;     // tx * 128
  // implicit-GEMM convolution (conv != 0): activation rows are output pixels, a tile is a
  // tw x th x tb box of (ow, oh, batch); k runs over (kh, kw, ci) in blocks of 64 channels
  int conv;
  int tw, th, tb, tiles_w, tiles_h;
  int OW, OH, Bn;
  int stride, pad_h, pad_w, dil_h, dil_w, KW, c_blocks;
  // epilogue through shared memory and TMA stores (epi_tma != 0); chunk box of the conv output
  int epi_tma, epi_res;       // epi_res: the residual is fetched with TMA too
  int cbw, cbh;               // pixels of one 32-pixel chunk along w and h (conv)
  int rep;                    // 1: every 128-row tile lies in one codebook group -> replicated tables
  int ksplit;                 // K is cut into this many slices, one tile per (slice, n block, m block);
                              // > 1: partial sums are added into `ws` instead of being stored
  float* ws;                  // [M][N] fp32 workspace of the split-K mode (zeroed by the launcher)
#ifdef DIMQ_B200_DIAG
  int dbg;                    // 2 skip the TMEM stores of the dequantisation, 4 skip MMAs, 8 skip the activation copies, 16 skip the lookups
  unsigned long long* prof;   // per-CTA cycle counters, 32 words per CTA, or null
#endif
};

struct TmapSet {
  CUtensorMap m[4];   // GEMM: m[0]; conv: one map per (row, column) parity of a stride-2 input
  CUtensorMap y;      // output, boxes of 32 features x 32 rows / pixels (TMA-store epilogue)
  CUtensorMap r;      // residual, same geometry as y
};

struct SharedHeader {
  uint64_t x_full[kXStages], x_empty[kXStages];
  uint64_t w_full[kWStages], w_empty[kWStages];
  uint64_t d_full[kAccStages], d_empty[kAccStages];
  uint64_t r_full[kNumEpilogueWarps][2];   // residual tiles of the TMA epilogue, per warp, double-buffered
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};
constexpr int kHeaderBytes = 512;

#ifdef DIMQ_B200_DIAG
// cycles spent inside one bounded wait, accumulated per role when p.prof is set
#define DIMQ_TIMED(acc, expr)                                   \
  [&]() {                                                        \
    const long long t0_ = DIMQ_PROF_ON ? clock64() : 0;                \
    const bool ok_ = (expr);                                     \
    if (p.prof) acc += static_cast<unsigned long long>(clock64() - t0_); \
    return ok_;                                                  \
  }()
#define DIMQ_DBG(bit) ((p.dbg & (bit)) != 0)
#define DIMQ_PROF_ON (p.prof != nullptr)
#define DIMQ_PROF_STORE(i, v) do { if (p.prof) p.prof[blockIdx.x * 32 + (i)] = (v); } while (0)
#else
#define DIMQ_TIMED(acc, expr) (expr)
#define DIMQ_DBG(bit) false
#define DIMQ_PROF_ON false
#define DIMQ_PROF_STORE(i, v) do { } while (0)
#endif

template <int BITS>
__device__ __forceinline__ void load_unit(const uint8_t* p, uint32_t (&w)[BITS]) {
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

// field `i` of width FB bits out of the words of one unit (i is a constant after unrolling)
template <int NW, int FB>
__device__ __forceinline__ uint32_t get_field(const uint32_t (&w)[NW], int i) {
  const int bit = i * FB;
  const int word = bit >> 5, sh = bit & 31;
  uint32_t v = w[word] >> sh;
  if (sh + FB > 32) v |= w[word + 1] << (32 - sh);
  return v & ((1u << FB) - 1u);
}

__device__ __forceinline__ uint32_t to_operand16(float v, int w_fmt) {
  if (w_fmt == 0) return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(v)));
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}


// accumulator + bias -> activation / residual.  DIMQ_EPI_ADD_RELU adds the residual before the ReLU
// (a ResNet block); the other epilogues apply the activation first and add the residual after it.
template <typename T, bool RES>
__device__ __forceinline__ float finish(float v, int epilogue, const T* res) {
  if (epilogue == DIMQ_EPI_ADD_RELU) {
    if (RES) v += to_float<T>(*res);
    return fmaxf(v, 0.0f);
  }
  v = apply_epilogue(v, epilogue);
  if (RES) v += to_float<T>(*res);
  return v;
}

// Epilogue of one 32-column chunk: thread = output feature n, r[j] = accumulator of activation row
// (m_first + j).  yp / rp point at element [m_first][n]; a warp store covers 32 consecutive n.
template <typename T, bool RES>
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], T* __restrict__ yp, const T* __restrict__ rp,
                                            int64_t ld, int rows, float bias, int epilogue) {
  if (rows >= 32) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      yp[j * ld] = from_float<T>(finish<T, RES>(__uint_as_float(r[j]) + bias, epilogue, RES ? rp + j * ld : nullptr));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < rows) yp[j * ld] = from_float<T>(finish<T, RES>(__uint_as_float(r[j]) + bias, epilogue, RES ? rp + j * ld : nullptr));
    }
  }
}

template <typename T>
__device__ __forceinline__ void store_chunk_t(const uint32_t (&r)[32], void* y, const void* res, int64_t off,
                                              int64_t ld, int rows, float bias, int epilogue) {
  if (res != nullptr)
    store_chunk<T, true>(r, static_cast<T*>(y) + off, static_cast<const T*>(res) + off, ld, rows, bias, epilogue);
  else
    store_chunk<T, false>(r, static_cast<T*>(y) + off, nullptr, ld, rows, bias, epilogue);
}

// Convolution epilogue of one chunk: column (p0 + j) of the tile is output pixel
// (b0 + bb, oh0 + hh, ow0 + ww) with ww fastest; y and the residual are NHWC.
template <typename T>
__device__ __forceinline__ void store_chunk_conv(const uint32_t (&r)[32], const TcParams& p, int p0, int m_blk,
                                                 int64_t n, bool n_ok, float bias) {
  // lane j works out where pixel (p0 + j) of the tile lives (or that it is outside the image); the
  // offsets are then handed round with shuffles instead of being recomputed by every lane
  const int lane = threadIdx.x & 31;
  const int pj = p0 + lane;
  const int ww = pj % p.tw, hh = (pj / p.tw) % p.th, bb = pj / (p.tw * p.th);
  const int ow = (m_blk % p.tiles_w) * p.tw + ww;
  const int oh = ((m_blk / p.tiles_w) % p.tiles_h) * p.th + hh;
  const int ob = (m_blk / (p.tiles_w * p.tiles_h)) * p.tb + bb;
  long long mine = -1;
  if (pj < p.tx && ob < p.Bn && oh < p.OH && ow < p.OW)
    mine = ((static_cast<long long>(ob) * p.OH + oh) * p.OW + ow) * p.N;
  T* y = static_cast<T*>(p.y);
  const T* res = static_cast<const T*>(p.residual);
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const long long base = __shfl_sync(0xFFFFFFFFu, mine, j);
    if (base >= 0 && n_ok) {
      const long long off = base + n;
      const float v = __uint_as_float(r[j]) + bias;
      y[off] = from_float<T>(res != nullptr ? finish<T, true>(v, p.epilogue, res + off) : finish<T, false>(v, p.epilogue, nullptr));
    }
  }
}

// ---- epilogue through shared memory + TMA (p.epi_tma) -----------------------------------------
// Box coordinates of chunk c (32 rows / pixels) of tile t for the warp of TMEM lane quarter `quarter`.
__device__ __forceinline__ void epi_coords(const TcParams& p, int t, int c, int quarter, int& c0, int& c1, int& c2,
                                           int& c3) {
  const int m_blk = t % p.m_tiles, n_blk = t / p.m_tiles;
  c0 = n_blk * kTileW + quarter * 32;
  if (!p.conv) {
    c1 = m_blk * p.tx + c * 32;
    c2 = c3 = 0;
    return;
  }
  const int p0 = c * 32;                      // tw divides 32 or 32 divides tw * th: a chunk is a box
  const int hh0 = (p0 / p.tw) % p.th, bb0 = p0 / (p.tw * p.th);
  c1 = (m_blk % p.tiles_w) * p.tw;
  c2 = ((m_blk / p.tiles_w) % p.tiles_h) * p.th + hh0;
  c3 = (m_blk / (p.tiles_w * p.tiles_h)) * p.tb + bb0;
}

__device__ __forceinline__ void epi_issue_residual(const TmapSet& tmaps, const TcParams& p, SharedHeader* hdr,
                                                   unsigned char* dst, int ew, int buf, int t, int c, int quarter) {
  int c0, c1, c2, c3;
  epi_coords(p, t, c, quarter, c0, c1, c2, c3);
  const uint32_t bar = smem_u32(&hdr->r_full[ew][buf]);
  mbar_arrive_expect_tx(bar, 32u * 32u * 2u);
  if (p.conv) tma_load_4d(smem_u32(dst), &tmaps.r, bar, c0, c1, c2, c3);
  else tma_load_2d(smem_u32(dst), &tmaps.r, bar, c0, c1);
}

// thread = feature (lane), r[j] = row / pixel j of the chunk.  The epilogue kind and the residual are
// template parameters so that the 32 elements form straight-line code (a run-time switch inside the
// loop serialises them: measured ~100 cycles per element).
// GELU for 16-bit outputs: 0.5 v (1 + tanh(0.79788 (v + 0.044715 v^3))) with the hardware tanh.  It
// differs from the erf form by at most 4.8e-4 (relative L2 2e-4 on N(0,1) inputs), an eighth of the
// rounding error of the bf16 store that follows, and costs 6 instructions instead of 18; the erf
// form stays for fp32 outputs.
constexpr int kEpiGelu16 = 16;
__device__ __forceinline__ float gelu_tanh(float v) {
  const float u = v * fmaf(0.0356774081f, v * v, 0.7978845608f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float h = 0.5f * v;
  return fmaf(h, t, h);
}

template <int EPI, bool RES, typename RT>
__device__ __forceinline__ void finish_chunk(uint32_t (&r)[32], float bias, const RT* res) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float v = __uint_as_float(r[j]) + bias;
    if (EPI == DIMQ_EPI_ADD_RELU) {
      if (RES) v += to_float<RT>(res[j * 32]);
      v = fmaxf(v, 0.0f);
    } else {
      if (EPI == DIMQ_EPI_RELU) v = fmaxf(v, 0.0f);
      if (EPI == DIMQ_EPI_GELU) v = 0.5f * v * (1.0f + fast_erf(v * 0.70710678118654752440f));
      if (EPI == kEpiGelu16) v = gelu_tanh(v);
      if (RES) v += to_float<RT>(res[j * 32]);
    }
    r[j] = __float_as_uint(v);
  }
}

template <bool RES, typename RT>
__device__ __forceinline__ void finish_chunk_epi(uint32_t (&r)[32], float bias, const RT* res, int epilogue) {
  switch (epilogue) {
    case DIMQ_EPI_RELU: finish_chunk<DIMQ_EPI_RELU, RES, RT>(r, bias, res); break;
    case DIMQ_EPI_GELU: finish_chunk<DIMQ_EPI_GELU, RES, RT>(r, bias, res); break;
    case kEpiGelu16: finish_chunk<kEpiGelu16, RES, RT>(r, bias, res); break;
    case DIMQ_EPI_ADD_RELU: finish_chunk<DIMQ_EPI_ADD_RELU, RES, RT>(r, bias, res); break;
    default: finish_chunk<DIMQ_EPI_NONE, RES, RT>(r, bias, res); break;
  }
}

template <typename T>
__device__ __forceinline__ void write_chunk(const uint32_t (&r)[32], unsigned char* out, int lane) {
  T* o = reinterpret_cast<T*>(out) + lane;
#pragma unroll
  for (int j = 0; j < 32; ++j) o[j * 32] = from_float<T>(__uint_as_float(r[j]));
}

// [32 rows][32 features] staging tile of one chunk; `res` is the residual tile in the same layout.
__device__ __forceinline__ void stage_chunk(uint32_t (&r)[32], unsigned char* out, const unsigned char* res, int lane,
                                            float bias, int epilogue, int y_dtype) {
  if (epilogue == DIMQ_EPI_GELU && y_dtype != DIMQ_F32) epilogue = kEpiGelu16;
  if (res == nullptr) finish_chunk_epi<false, float>(r, bias, nullptr, epilogue);
  else if (y_dtype == DIMQ_BF16) finish_chunk_epi<true, __nv_bfloat16>(r, bias, reinterpret_cast<const __nv_bfloat16*>(res) + lane, epilogue);
  else finish_chunk_epi<true, __half>(r, bias, reinterpret_cast<const __half*>(res) + lane, epilogue);
  if (y_dtype == DIMQ_BF16) write_chunk<__nv_bfloat16>(r, out, lane);
  else if (y_dtype == DIMQ_F16) write_chunk<__half>(r, out, lane);
  else write_chunk<float>(r, out, lane);
}

__device__ __forceinline__ void cp_async(uint32_t dst, const void* src, int bytes) {
  if (bytes == 16)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
  else if (bytes == 8)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Prefetch ring of packed-index units: one slot per dequantisation thread and stage in flight.
constexpr int kIdxPrefetch = 3;
template <int BITS>
struct IdxSlot { static constexpr int kBytes = BITS == 8 ? 64 : 32; };  // 64 indices of one weight row

template <int BITS>
__device__ __forceinline__ void issue_unit(uint32_t dst, const uint8_t* src) {
  // 64 indices = 8 * BITS bytes
  if constexpr (BITS == 4) { cp_async(dst, src, 16); cp_async(dst + 16, src + 16, 16); }
  else if constexpr (BITS == 2) { cp_async(dst, src, 16); }
  else if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) cp_async(dst + 16 * i, src + 16 * i, 16);
  } else {
#pragma unroll
    for (int i = 0; i < BITS; ++i) cp_async(dst + 8 * i, src + 8 * i, 8);
  }
}

template <int BITS>
__device__ __forceinline__ void read_unit(const unsigned char* slot, uint32_t (&w)[2 * BITS]) {
  constexpr int kVec = (2 * BITS * 4 + 15) / 16;
  uint32_t v[kVec * 4];
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const uint4 q = *reinterpret_cast<const uint4*>(slot + 16 * i);
    v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
  }
#pragma unroll
  for (int i = 0; i < 2 * BITS; ++i) w[i] = v[i];
}

// 32-bit words of lookup table per codebook group.
//   PAIR : entry v (two adjacent indices, 2*BITS bits) -> {C[v & mask], C[v >> BITS]} as two 16-bit
//          operands in one word; in split mode two words {hi pair, lo pair}.
//   !PAIR: entry e -> one 16-bit operand (two per word); in split mode one word {hi | lo << 16}.
__host__ __device__ constexpr int table_words(int bits, bool pair, bool split) {
  return pair ? (1 << (2 * bits)) * (split ? 2 : 1) : (split ? (1 << bits) : (1 << bits) / 2);
}

__device__ __forceinline__ void split_bf16(float c, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 h = __float2bfloat16_rn(c);
  hi = __bfloat16_as_ushort(h);
  lo = __bfloat16_as_ushort(__float2bfloat16_rn(c - __bfloat162float(h)));
}

template <int BITS, bool PAIR, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
linear_wq_tc_kernel(const __grid_constant__ TmapSet tmaps, const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // [x stages (1024-aligned)] [header] [tables]
  // rounded up to 1024 bytes in the shared window; plain pointer arithmetic on the array keeps the
  // accesses below in the shared state space (no generic loads and stores)
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* x_stage = smem;
  const uint32_t n_xs = static_cast<uint32_t>(p.x_stages);
  SharedHeader* hdr = reinterpret_cast<SharedHeader*>(smem + n_xs * p.x_stage_bytes);
  unsigned char* epi_stage = reinterpret_cast<unsigned char*>(hdr) + kHeaderBytes;   // TMA epilogue staging, per warp
  const int out_esize = p.y_dtype == DIMQ_F32 ? 4 : 2;
  const uint32_t epi_out_bytes = 32u * 32u * out_esize;
  const uint32_t epi_warp_bytes = p.epi_tma ? epi_out_bytes * (p.epi_res ? 3u : 1u) : 0u;
  unsigned char* idx_ring = epi_stage + kNumEpilogueWarps * epi_warp_bytes;  // [kIdxPrefetch][dequant threads][slot]
  constexpr int kRingBytes = kIdxPrefetch * kNumDequantWarps * 32 * IdxSlot<BITS>::kBytes;
  uint32_t* rep_tables = reinterpret_cast<uint32_t*>(idx_ring + kRingBytes);  // [groups of warps][kRepWords]
  uint32_t* table = rep_tables + (p.rep ? kNumDequantGroups * kRepWords : 0);
  static_assert(sizeof(SharedHeader) <= kHeaderBytes, "header");

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  // tile t = (k slice * n_tiles + n block) * m_tiles + m block; one slice unless split-K is on
  const int num_tiles = p.m_tiles * p.n_tiles * p.ksplit;
  const int k_blocks = static_cast<int>(p.K / kBlockK) / p.ksplit;
  constexpr int kWStageCols = SPLIT ? kBlockK : kBlockK / 2;   // TMEM columns per weight stage
  constexpr uint32_t kWStagesUsed = SPLIT ? kWStages / 2 : kWStages;

  // ---- one-time setup ---------------------------------------------------------
  if (tid == 0) {
    for (int s = 0; s < kXStages; ++s) { mbar_init(smem_u32(&hdr->x_full[s]), 1); mbar_init(smem_u32(&hdr->x_empty[s]), 1); }
    for (int s = 0; s < kWStages; ++s) { mbar_init(smem_u32(&hdr->w_full[s]), 4); mbar_init(smem_u32(&hdr->w_empty[s]), 1); }
    for (int s = 0; s < kAccStages; ++s) { mbar_init(smem_u32(&hdr->d_full[s]), 1); mbar_init(smem_u32(&hdr->d_empty[s]), kNumEpilogueWarps); }
    for (int e = 0; e < kNumEpilogueWarps; ++e) { mbar_init(smem_u32(&hdr->r_full[e][0]), 1); mbar_init(smem_u32(&hdr->r_full[e][1]), 1); }
    hdr->abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tmaps.m[0]);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&hdr->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  {
    constexpr uint32_t mask = (1u << BITS) - 1u;
    constexpr int n_entries = PAIR ? (1 << (2 * BITS)) : (1 << BITS);
    const int total = static_cast<int>(p.groups) * n_entries;
    auto cw = [&](int g, int e) -> float {
      return e < p.entries ? load_as_float(p.codebooks, p.cb_dtype, static_cast<int64_t>(g) * p.entries + e) : 0.0f;
    };
    for (int i = tid; i < total; i += kThreads) {
      const int g = i / n_entries, v = i % n_entries;
      if (PAIR) {
        const float c0 = cw(g, v & mask), c1 = cw(g, v >> BITS);
        if (SPLIT) {
          uint32_t h0, l0, h1, l1;
          split_bf16(c0, h0, l0);
          split_bf16(c1, h1, l1);
          table[2 * i] = h0 | (h1 << 16);
          table[2 * i + 1] = l0 | (l1 << 16);
        } else {
          table[i] = to_operand16(c0, p.w_fmt) | (to_operand16(c1, p.w_fmt) << 16);
        }
      } else {
        const float c = cw(g, v);
        if (SPLIT) {
          uint32_t h, l;
          split_bf16(c, h, l);
          table[i] = h | (l << 16);
        } else {
          reinterpret_cast<uint16_t*>(table)[i] = static_cast<uint16_t>(to_operand16(c, p.w_fmt));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  if (warp == 0) {
    // ===================== TMA producer =====================
    // The whole warp walks the loop; one elected lane issues the copies (see elect_one).
    {
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      unsigned long long w_xe = 0;
      const long long t_begin = clock64();
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = t % p.m_tiles;
        const int k0 = ((t / p.m_tiles) / p.n_tiles) * k_blocks;  // first k block of this tile's slice
        int ow0 = 0, oh0 = 0, b0 = 0, tap = 0, cb = 0;
        if (p.conv) {
          ow0 = (m_blk % p.tiles_w) * p.tw;
          oh0 = ((m_blk / p.tiles_w) % p.tiles_h) * p.th;
          b0 = (m_blk / (p.tiles_w * p.tiles_h)) * p.tb;
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!__all_sync(0xFFFFFFFFu, DIMQ_TIMED(w_xe, mbar_wait(smem_u32(&hdr->x_empty[stage]), phase ^ 1u, abort_flag, 0x100u | stage)))) { ok = false; break; }
          const uint32_t full = smem_u32(&hdr->x_full[stage]);
          const uint32_t dst = smem_u32(x_stage + stage * p.x_stage_bytes);
          if (DIMQ_DBG(8)) {
            if (elect_one()) mbar_arrive(full);
          } else if (!p.conv) {
            if (elect_one()) {
              mbar_arrive_expect_tx(full, p.x_stage_bytes);
              tma_load_2d(dst, &tmaps.m[0], full, (k0 + kb) * kBlockK, m_blk * p.tx);
            }
          } else {
            // tap (kh, kw), channels [64 cb, 64 cb + 64): input pixel = s * out + tap offset.  With
            // stride 2 the input is addressed through one tensor map per (row, column) parity, so the
            // box stays dense; taps that fall outside the image read the zero fill.
            const int kh = tap / p.KW, kw = tap - kh * p.KW;
            const int dy = kh * p.dil_h - p.pad_h, dx = kw * p.dil_w - p.pad_w;
            int map = 0, hy = oh0 + dy, wx = ow0 + dx;
            if (p.stride == 2) {
              const int py = dy & 1, px = dx & 1;          // parity (two's complement: also right for negatives)
              map = py * 2 + px;
              hy = oh0 + ((dy - py) >> 1);
              wx = ow0 + ((dx - px) >> 1);
            }
            if (elect_one()) {
              mbar_arrive_expect_tx(full, p.x_stage_bytes);
              tma_load_4d(dst, &tmaps.m[map], full, cb * kBlockK, wx, hy, b0);
            }
            if (++cb == p.c_blocks) { cb = 0; ++tap; }
          }
          __syncwarp();
          ++issued;
          if (++stage == n_xs) { stage = 0; phase ^= 1u; }
        }
      }
      if (lane == 0) {
        DIMQ_PROF_STORE(0, w_xe);
        DIMQ_PROF_STORE(1, clock64() - t_begin);
      }
      if (!ok && lane == 0) {
        // Gave up: wait (bounded) for the copies still in flight so that no TMA write
        // lands in shared memory after this CTA has exited.
        const uint32_t n_back = issued < n_xs ? issued : n_xs;
        uint32_t s = stage, ph = phase;
        for (uint32_t i = 0; i < n_back; ++i) {
          if (s == 0) { s = n_xs - 1; ph ^= 1u; } else { --s; }
          for (uint32_t it = 0; it < kSpinLimit; ++it)
            if (mbar_try_wait(smem_u32(&hdr->x_full[s]), ph)) break;
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    // The whole warp walks the loop and polls the barriers; one elected lane issues the MMAs and
    // the commits (see elect_one).
    {
      uint32_t xs = 0, xph = 0, ws = 0, wph = 0, as = 0, aph = 0;
      bool ok = true;
      unsigned long long w_de = 0, w_xf = 0, w_wf = 0, t_cm = 0, t_fe = 0, t_mm = 0;
      const long long t_begin = clock64();
      const uint64_t desc0 = make_smem_desc_sw128(smem_u32(x_stage));
      const uint32_t a0 = tmem_base + kWCol;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!__all_sync(0xFFFFFFFFu, DIMQ_TIMED(w_de, mbar_wait(smem_u32(&hdr->d_empty[as]), aph ^ 1u, abort_flag, 0x200u | as)))) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + kAccCol + as * kTileX;
        // k blocks are issued two at a time: the four barrier polls of a pair overlap
        auto issue_block = [&](int kb, uint32_t xs_, uint32_t ws_) {
          const uint64_t b_desc = desc0 + static_cast<uint64_t>(xs_ * (p.x_stage_bytes >> 4));
          const uint32_t a_tmem = a0 + ws_ * kWStageCols;
          if (!DIMQ_DBG(4)) {
            // advance 16 k: 32 bytes inside the swizzled row (encoded >> 4), 8 TMEM columns
            if (kb == 0) mma_f16_ts(d_tmem, a_tmem, b_desc, p.idesc, 0u);
            else mma_f16_ts_acc(d_tmem, a_tmem, b_desc, p.idesc);
            if (SPLIT) mma_f16_ts_acc(d_tmem, a_tmem + kBlockK / 2, b_desc, p.idesc);
#pragma unroll
            for (int j = 1; j < kBlockK / 16; ++j) {
              mma_f16_ts_acc(d_tmem, a_tmem + j * 8, b_desc + static_cast<uint64_t>(j * 2), p.idesc);
              if (SPLIT) mma_f16_ts_acc(d_tmem, a_tmem + kBlockK / 2 + j * 8, b_desc + static_cast<uint64_t>(j * 2), p.idesc);
            }
          }
          // one commit per k block: the producer (activation slot) and the dequantisation group
          // that will reuse this weight slot both wait on it
          mma_commit(smem_u32(&hdr->x_empty[xs_]));
        };
        for (int kb = 0; kb < k_blocks;) {
          const bool two = kb + 1 < k_blocks;
          uint32_t xs1 = xs + 1, xph1 = xph, ws1 = ws + 1, wph1 = wph;
          if (xs1 == n_xs) { xs1 = 0; xph1 ^= 1u; }
          if (ws1 == kWStagesUsed) { ws1 = 0; wph1 ^= 1u; }
          const long long tq0 = DIMQ_PROF_ON ? clock64() : 0;
          const bool got = two ? mbar_wait4(smem_u32(&hdr->x_full[xs]), xph, smem_u32(&hdr->w_full[ws]), wph,
                                            smem_u32(&hdr->x_full[xs1]), xph1, smem_u32(&hdr->w_full[ws1]), wph1,
                                            abort_flag, 0x300u | xs)
                               : mbar_wait2(smem_u32(&hdr->x_full[xs]), xph, smem_u32(&hdr->w_full[ws]), wph,
                                            abort_flag, 0x300u | xs);
          if (!__all_sync(0xFFFFFFFFu, got)) { ok = false; break; }
          tc_fence_after();
          const long long tq1 = DIMQ_PROF_ON ? clock64() : 0;
          if (elect_one()) {
            issue_block(kb, xs, ws);
            if (two) issue_block(kb + 1, xs1, ws1);
          }
          __syncwarp();
          if (DIMQ_PROF_ON) { w_xf += tq1 - tq0; t_mm += clock64() - tq1; }
          const int nb = two ? 2 : 1;
          for (int i = 0; i < nb; ++i) {
            if (++xs == n_xs) { xs = 0; xph ^= 1u; }
            if (++ws == kWStagesUsed) { ws = 0; wph ^= 1u; }
          }
          kb += nb;
        }
        if (!ok) break;
        if (elect_one()) mma_commit(smem_u32(&hdr->d_full[as]));
        __syncwarp();
        if (++as == kAccStages) { as = 0; aph ^= 1u; }
      }
      if (lane == 0) {
        DIMQ_PROF_STORE(2, w_de); DIMQ_PROF_STORE(3, w_xf); DIMQ_PROF_STORE(4, w_wf);
        DIMQ_PROF_STORE(5, clock64() - t_begin);
        DIMQ_PROF_STORE(11, t_cm); DIMQ_PROF_STORE(12, t_fe); DIMQ_PROF_STORE(13, t_mm);
      }
    }
  } else if (warp < 2 + kNumEpilogueWarps) {
    // ===================== epilogue =====================
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32)
    const int sub = (warp - 2) >> 2;  // which of the two warps of this quarter: chunks sub, sub + 2, ...
    const int ew = warp - 2;          // epilogue warp index, 0..7
    unsigned char* my_out = epi_stage + ew * epi_warp_bytes;
    unsigned char* my_res = my_out + epi_out_bytes;
    uint32_t res_ph[2] = {0u, 0u};
    int res_buf = 0;
    if (p.epi_tma && p.epi_res) {
      // residual tile of this warp's first chunk
      const int t0 = blockIdx.x;
      if (t0 < num_tiles && sub < (p.tx + 31) / 32 && (t0 / p.m_tiles) * kTileW + quarter * 32 < p.N) {
        if (elect_one()) epi_issue_residual(tmaps, p, hdr, my_res, ew, 0, t0, sub, quarter);
      }
      __syncwarp();
    }
    uint32_t as = 0, aph = 0;
    bool ok = true;
    unsigned long long w_df = 0, t_ewait = 0, t_estage = 0;
    const long long t_begin = clock64();
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m_blk = t % p.m_tiles, n_blk = (t / p.m_tiles) % p.n_tiles;
      const int64_t n = static_cast<int64_t>(n_blk) * kTileW + quarter * 32 + lane;
      const int64_t m0 = static_cast<int64_t>(m_blk) * p.tx;
      const bool n_ok = n < p.N;
      const float bias = (p.bias != nullptr && n_ok) ? load_as_float(p.bias, p.bias_dtype, n) : 0.0f;
      // tcgen05.ld is warp-collective: the whole warp proceeds or the whole warp gives up
      if (!__all_sync(0xFFFFFFFFu, DIMQ_TIMED(w_df, mbar_wait(smem_u32(&hdr->d_full[as]), aph, abort_flag, 0x500u | as)))) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kAccCol + as * kTileX;
      const int n_chunks = (p.tx + 31) / 32;
      if (sub >= n_chunks) {   // fewer chunks than warps: nothing to read, release at once
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&hdr->d_empty[as]));
      }
      if (p.epi_tma) {
        const int n_box = n_blk * kTileW + quarter * 32;   // first feature of this warp's boxes
        const bool warp_has_n = n_box < p.N;
        for (int c = sub; c < n_chunks; c += 2) {
          uint32_t r[32];
          __syncwarp();
          tmem_ld32(d_tmem + c * 32, r);
          tmem_ld_wait();
          if (c + 2 >= n_chunks) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&hdr->d_empty[as]));
          }
          if (!warp_has_n) continue;
          // the next chunk of this warp (same tile, or the first one of its next tile)
          int t_next = t, c_next = c + 2;
          if (c_next >= n_chunks) { t_next = t + gridDim.x; c_next = sub; }
          const bool has_next = t_next < num_tiles && c_next < n_chunks &&
                                (t_next / p.m_tiles) * kTileW + quarter * 32 < p.N;
          if (p.epi_res) {
            if (has_next) {
              if (elect_one()) epi_issue_residual(tmaps, p, hdr, my_res + (res_buf ^ 1) * epi_out_bytes, ew, res_buf ^ 1, t_next, c_next, quarter);
            }
            uint32_t got = 0;
            if (lane == 0) got = mbar_wait(smem_u32(&hdr->r_full[ew][res_buf]), res_ph[res_buf], abort_flag, 0x700u | ew) ? 1u : 0u;
            if (!__shfl_sync(0xFFFFFFFFu, got, 0)) { ok = false; break; }
            res_ph[res_buf] ^= 1u;
          }
          // the previous store of this warp must have finished reading the staging tile
          const long long te0 = DIMQ_PROF_ON ? clock64() : 0;
          if (elect_one()) tma_store_wait_read();
          __syncwarp();
          const long long te1 = DIMQ_PROF_ON ? clock64() : 0;
          const unsigned char* res_tile = my_res + res_buf * epi_out_bytes;
          stage_chunk(r, my_out, p.epi_res ? res_tile : nullptr, lane, bias, p.epilogue, p.y_dtype);
          fence_proxy_async_smem();
          __syncwarp();
          if (DIMQ_PROF_ON) { const long long te2 = clock64(); t_ewait += te1 - te0; t_estage += te2 - te1; }
          {
            int c0, c1, c2, c3;
            epi_coords(p, t, c, quarter, c0, c1, c2, c3);
            if (elect_one()) {
              if (p.conv) tma_store_4d(&tmaps.y, smem_u32(my_out), c0, c1, c2, c3);
              else tma_store_2d(&tmaps.y, smem_u32(my_out), c0, c1);
              tma_store_commit();
            }
          }
          if (p.epi_res) res_buf ^= 1;
        }
        if (!ok) break;
      } else
      for (int c = sub; c < n_chunks; c += 2) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(d_tmem + c * 32, r);
        tmem_ld_wait();
        if (c + 2 >= n_chunks) {
          // every column of this buffer is in registers: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&hdr->d_empty[as]));
        }
        if (!p.conv) {
          const int64_t m_first = m0 + c * 32;
          const int64_t rows64 = p.M - m_first;
          const int rows = rows64 >= 32 ? 32 : static_cast<int>(rows64);
          if (n_ok && rows > 0 && p.ksplit > 1) {
            // split-K: this tile holds the sum over one K slice only
            float* wsp = p.ws + m_first * p.N + n;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < rows) atomicAdd(wsp + j * p.N, __uint_as_float(r[j]));
          } else if (n_ok && rows > 0) {
            const int64_t off = m_first * p.N + n;
            if (p.y_dtype == DIMQ_BF16) store_chunk_t<__nv_bfloat16>(r, p.y, p.residual, off, p.N, rows, bias, p.epilogue);
            else if (p.y_dtype == DIMQ_F16) store_chunk_t<__half>(r, p.y, p.residual, off, p.N, rows, bias, p.epilogue);
            else store_chunk_t<float>(r, p.y, p.residual, off, p.N, rows, bias, p.epilogue);
          }
        } else {
          if (p.y_dtype == DIMQ_BF16) store_chunk_conv<__nv_bfloat16>(r, p, c * 32, m_blk, n, n_ok, bias);
          else if (p.y_dtype == DIMQ_F16) store_chunk_conv<__half>(r, p, c * 32, m_blk, n, n_ok, bias);
          else store_chunk_conv<float>(r, p, c * 32, m_blk, n, n_ok, bias);
        }
      }
      if (++as == kAccStages) { as = 0; aph ^= 1u; }
    }
    __syncwarp();
    if (p.epi_tma) {
      if (elect_one()) tma_store_wait_all();
    }
    if (warp == 2 && lane == 0) {
      DIMQ_PROF_STORE(14, t_ewait); DIMQ_PROF_STORE(15, t_estage); DIMQ_PROF_STORE(6, w_df);
      DIMQ_PROF_STORE(7, clock64() - t_begin);
    }
  } else {
    // ===================== dequantisation =====================
    // 8 warps in 2 groups of 4 (one warp per TMEM lane quarter).  Group g dequantises stages
    // g, g + 2, g + 4, ... completely (64 k of 128 weight rows: thread = weight row), so a warp has
    // two stage periods for one stage's latency chain.
    // A group may run at most one mbarrier phase ahead of the MMA warp, which holds when the number
    // of active groups does not exceed the number of weight stages (2 in split mode): the third
    // group idles there.
    constexpr int kGroups = SPLIT ? 2 : kNumDequantGroups;
    static_assert(kGroups <= (SPLIT ? kWStages / 2 : kWStages), "dequant groups vs weight stages");
    const int dw = warp - (2 + kNumEpilogueWarps);  // 0..7
    const int grp = dw >> 2;
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may write
    const int row_in_tile = quarter * 32 + lane;
    const int64_t row_bytes = p.K * BITS / 8;
    constexpr int per_group = table_words(BITS, PAIR, SPLIT);
    constexpr int kWpe = SPLIT ? 2 : 1;                       // words per pair-table entry
    constexpr int kPairEntries = 1 << (2 * BITS);
    constexpr int kRepRaw = kRepWords / (kPairEntries * kWpe);
    constexpr int kRep = kRepRaw < 1 ? 1 : (kRepRaw > 32 / kWpe ? 32 / kWpe : kRepRaw);  // copies per entry
    const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const int total_iters = my_tiles * k_blocks;
    const int n_own = (grp < kGroups && total_iters > grp) ? (total_iters - grp + kGroups - 1) / kGroups : 0;
    const int n_rows = static_cast<int>(p.N);
    const int group_rows = static_cast<int>(p.group_rows);
    const bool rep = PAIR && p.rep != 0;
    uint32_t* my_rep = rep_tables + grp * kRepWords;
    const int gt = (dw & 3) * 32 + lane;            // thread index inside the group, 0..127
    auto row_of = [&](int t) -> int {
      int row = ((t / p.m_tiles) % p.n_tiles) * kTileW + row_in_tile;
      return row >= n_rows ? n_rows - 1 : row;
    };
    auto advance = [&](int& t, int& kb, int steps) {
      kb += steps;
      while (kb >= k_blocks) { kb -= k_blocks; t += gridDim.x; }
    };
    const int dq_tid = tid - (2 + kNumEpilogueWarps) * 32;
    constexpr int kSlot = IdxSlot<BITS>::kBytes;
    constexpr int kRingStride = kNumDequantWarps * 32 * kSlot;
    const uint32_t ring_u32 = smem_u32(idx_ring + dq_tid * kSlot);  // slot s at + s * kRingStride
    const unsigned char* my_ring = idx_ring + dq_tid * kSlot;
    // prefetch cursor: the packed indices of an own stage are fetched kIdxPrefetch - 1 own stages ahead
    int pf_tile = blockIdx.x, pf_kb = 0, pf_slot = 0, pf_j = 0, pf_row_tile = -1;
    advance(pf_tile, pf_kb, grp);
    const uint8_t* pf_row = p.packed;
    auto prefetch_next = [&]() {
      if (pf_j < n_own) {
        if (pf_tile != pf_row_tile) {
          pf_row = p.packed + static_cast<int64_t>(row_of(pf_tile)) * row_bytes +
                   static_cast<int64_t>((pf_tile / p.m_tiles) / p.n_tiles) * k_blocks * (8 * BITS);
          pf_row_tile = pf_tile;
        }
        issue_unit<BITS>(ring_u32 + pf_slot * kRingStride, pf_row + pf_kb * (8 * BITS));
        ++pf_j;
        advance(pf_tile, pf_kb, kGroups);
      }
      cp_async_commit();
      if (++pf_slot == kIdxPrefetch) pf_slot = 0;
    };
#pragma unroll
    for (int s0 = 0; s0 < kIdxPrefetch - 1; ++s0) prefetch_next();
    int slot = 0;
    unsigned long long w_we = 0, w_cp = 0, t_look = 0, t_st = 0, t_arr = 0;
    const long long t_begin = clock64();
    // activation slot and parity of k block (it - kWStagesUsed) for this group's first waiting stage
    uint32_t rel_slot, rel_par;
    {
      // first own stage that has to wait: the smallest it = grp + j * kGroups with it >= kWStagesUsed
      int it0 = grp;
      while (it0 < static_cast<int>(kWStagesUsed)) it0 += kGroups;
      const uint32_t rel = static_cast<uint32_t>(it0) - kWStagesUsed;
      rel_slot = rel % n_xs;
      rel_par = (rel / n_xs) & 1u;
    }
    int t = blockIdx.x, kb = 0, cur_tile = -1, cur_group = -1;
    advance(t, kb, grp);
    const uint32_t* tbl = table;
#pragma unroll 1
    for (int j = 0; j < n_own; ++j) {
      const int it = grp + j * kGroups;
      const uint32_t ws = static_cast<uint32_t>(it) % kWStagesUsed;
      if (t != cur_tile) {
        cur_tile = t;
        const int g = row_of(t) / group_rows;
        if (rep) {
          // all 128 rows of the tile share codebook group g: (re)build this warp group's replicated
          // table, entry e copied kRep times so that lane l reads copy (l mod kRep) in its own bank
          const int g0 = (((t / p.m_tiles) % p.n_tiles) * kTileW) / group_rows;
          if (g0 != cur_group) {
            bar_sync(1 + grp, 128);
            const uint32_t* src = table + g0 * per_group;
            for (int i = gt; i < kPairEntries * kRep; i += 128) {
              const int e = i / kRep;
              if (SPLIT) { my_rep[2 * i] = src[2 * e]; my_rep[2 * i + 1] = src[2 * e + 1]; }
              else my_rep[i] = src[e];
            }
            bar_sync(1 + grp, 128);
            cur_group = g0;
          }
          tbl = my_rep + (lane & (kRep - 1)) * kWpe;
        } else {
          tbl = table + g * per_group;
        }
      }
      prefetch_next();
      { const long long t0_ = DIMQ_PROF_ON ? clock64() : 0; cp_async_wait<kIdxPrefetch - 1>(); if (DIMQ_PROF_ON) w_cp += clock64() - t0_; }
      const long long tl0 = DIMQ_PROF_ON ? clock64() : 0;
      uint32_t cur[2 * BITS];
      read_unit<BITS>(my_ring + slot * kRingStride, cur);
      if (++slot == kIdxPrefetch) slot = 0;
      uint32_t out[32];
      uint32_t out_lo[SPLIT ? 32 : 1];
      if (DIMQ_DBG(16)) {   // diagnostics: no lookups
#pragma unroll
        for (int q = 0; q < 32; ++q) { out[q] = cur[q % (2 * BITS)]; if (SPLIT) out_lo[SPLIT ? q : 0] = 0u; }
      } else
      if (PAIR) {
        const int stride = rep ? kRep * kWpe : kWpe;  // words between consecutive entries
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          const uint32_t v = get_field<2 * BITS, 2 * BITS>(cur, q);
          if (SPLIT) {
            const uint2 e = *reinterpret_cast<const uint2*>(tbl + v * stride);
            out[q] = e.x;
            out_lo[SPLIT ? q : 0] = e.y;
          } else {
            out[q] = tbl[v * stride];
          }
        }
      } else if (SPLIT) {
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          const uint32_t a = tbl[get_field<2 * BITS, BITS>(cur, 2 * q)];
          const uint32_t b = tbl[get_field<2 * BITS, BITS>(cur, 2 * q + 1)];
          out[q] = (a & 0xFFFFu) | (b << 16);
          out_lo[SPLIT ? q : 0] = (a >> 16) | (b & 0xFFFF0000u);
        }
      } else {
        const uint16_t* tbl16 = reinterpret_cast<const uint16_t*>(tbl);
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          const uint32_t lo = tbl16[get_field<2 * BITS, BITS>(cur, 2 * q)];
          const uint32_t hi = tbl16[get_field<2 * BITS, BITS>(cur, 2 * q + 1)];
          out[q] = lo | (hi << 16);
        }
      }
      if (DIMQ_PROF_ON) t_look += clock64() - tl0;
      // tcgen05.st is warp-collective: the whole warp proceeds or the whole warp gives up
      // weight slot ws was last read by k block (it - kWStagesUsed): wait for its commit, which was
      // signalled on the activation slot of that k block
      if (it >= static_cast<int>(kWStagesUsed)) {
        if (!__all_sync(0xFFFFFFFFu, DIMQ_TIMED(w_we, mbar_wait(smem_u32(&hdr->x_empty[rel_slot]), rel_par, abort_flag, 0x600u | ws)))) break;
        rel_slot += kGroups;
        if (rel_slot >= n_xs) { rel_slot -= n_xs; rel_par ^= 1u; }
      }
      tc_fence_after();
      const long long ts0 = DIMQ_PROF_ON ? clock64() : 0;
      const uint32_t w_tmem = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kWCol + ws * kWStageCols;
      if (!DIMQ_DBG(2)) {
        tmem_st32(w_tmem, out);
        if (SPLIT) {
          uint32_t lo32[32];
#pragma unroll
          for (int q = 0; q < 32; ++q) lo32[q] = out_lo[SPLIT ? q : 0];
          tmem_st32(w_tmem + kBlockK / 2, lo32);
        }
      }
      // one arrival per warp: per-thread arrivals on one mbarrier serialise in shared memory
      tmem_st_wait();
      const long long ts1 = DIMQ_PROF_ON ? clock64() : 0;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&hdr->w_full[ws]));
      if (DIMQ_PROF_ON) { t_st += ts1 - ts0; t_arr += clock64() - ts1; }
      advance(t, kb, kGroups);
    }
    if (dq_tid == 0) {
      DIMQ_PROF_STORE(8, w_we); DIMQ_PROF_STORE(9, w_cp); DIMQ_PROF_STORE(10, clock64() - t_begin);
      DIMQ_PROF_STORE(16, t_look); DIMQ_PROF_STORE(17, t_st); DIMQ_PROF_STORE(18, t_arr);
    }
  }

  // ---- teardown -----------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

template <int BITS, bool PAIR, bool SPLIT>
int launch_tc(const TmapSet& tmap, const TcParams& p, size_t smem, int grid, cudaStream_t st) {
  auto kern = linear_wq_tc_kernel<BITS, PAIR, SPLIT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  kern<<<grid, kThreads, smem, st>>>(tmap, p);
  return launch_status();
}

size_t table_bytes(int bits, int64_t groups, bool pair, bool split) {
  return static_cast<size_t>(groups) * table_words(bits, pair, split) * 4;
}

}  // namespace

// Tiled tensor map over plain bytes (elem_bytes 1) or 16-bit elements (2), no swizzle, zero fill;
// `out` points at a CUtensorMap.  For kernels outside this file that stage tiles with TMA.
int encode_plain_tensor_map(void* out, int elem_bytes, int rank, const void* base, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn encode = get_encode_tiled();
  if (encode == nullptr || rank < 1 || rank > 5) return DIMQ_ERR_DRIVER;
  cuuint64_t d[5], st[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
  const CUresult r = encode(static_cast<CUtensorMap*>(out),
                            elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, rank,
                            const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DIMQ_OK : DIMQ_ERR_DRIVER;
}

bool tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K) {
  if (x_dtype != DIMQ_BF16 && x_dtype != DIMQ_F16) return false;
  if (M < 1 || N < 1 || K < kBlockK || K % kBlockK != 0) return false;
  if (!aligned(x, 16) || !aligned(w->packed, 16)) return false;
  if (M > 0x7FFFFFFF / 2 || N > 0x7FFFFFFF / 2) return false;
  if (table_bytes(w->bits, w->groups, false, true) > (size_t)kMaxTableBytes) return false;
  const int64_t tiles = ((M + kTileX - 1) / kTileX) * ((N + kTileW - 1) / kTileW);
  return tiles < 0x7FFFFFFF;
}

#ifdef DIMQ_B200_DIAG
// Diagnostics build only: role-skipping switches, replicated-table switch and the buffer of per-CTA
// cycle counters (32 words per CTA; ignored unless it holds at least 148 * 32 words).
static int g_diag_dbg = 0, g_diag_rep = 0;
static unsigned long long* g_diag_prof = nullptr;
static int64_t g_diag_prof_words = 0;
void diag_configure(int dbg, int rep, unsigned long long* prof, int64_t prof_words) {
  g_diag_dbg = dbg;
  g_diag_rep = rep;
  g_diag_prof = prof;
  g_diag_prof_words = prof != nullptr ? prof_words : 0;
}
#endif

namespace {

bool epi_tma_enabled() {
  // read once per process: DIMQ_B200_TC_EPI=0 selects the direct-store epilogue
  static const bool enabled = [] {
    const char* env = getenv("DIMQ_B200_TC_EPI");
    return env == nullptr || atoi(env) != 0;
  }();
  return enabled;
}

CUtensorMapDataType tmap_dtype(int dtype) {
  return dtype == DIMQ_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : (dtype == DIMQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
}

// Tensor map over an output-like tensor (y or the residual): rank 2 [rows][N] for the GEMM, rank 4
// [B][OH][OW][N] for the convolution; boxes of 32 features x 32 rows / pixels, no swizzle.
bool encode_out_map(EncodeTiledFn encode, CUtensorMap* m, const void* base, int dtype, int rank,
                    const cuuint64_t* dims, const cuuint32_t* box) {
  const cuuint64_t es = dtype == DIMQ_F32 ? 4 : 2;
  cuuint64_t strides[3];
  cuuint64_t acc = dims[0] * es;
  for (int i = 0; i < rank - 1; ++i) { strides[i] = acc; acc *= dims[i + 1]; }
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode(m, tmap_dtype(dtype), rank, const_cast<void*>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Whether y (and the residual) can go through the TMA epilogue.
bool epi_tma_possible(const void* y, int y_dtype, const void* residual, int64_t N) {
  if (!epi_tma_enabled()) return false;
  const int64_t es = y_dtype == DIMQ_F32 ? 4 : 2;
  if (!aligned(y, 16) || (N * es) % 16 != 0) return false;
  if (residual != nullptr && (y_dtype == DIMQ_F32 || !aligned(residual, 16))) return false;
  return true;
}

// Fills the fields shared by the GEMM and the convolution, sizes shared memory and launches.
int finish_launch(const TmapSet& tmaps, TcParams& p, const dimq_wq_weight* w, const uint8_t* packed, int x_dtype,
                  const void* bias, int bias_dtype, const void* residual, void* y, int y_dtype, int epilogue,
                  int precision, cudaStream_t st) {
  p.packed = packed;
  p.codebooks = w->codebooks;
  p.cb_dtype = w->cb_dtype;
  p.entries = w->entries;
  p.groups = w->groups;
  p.group_rows = w->group_rows;
  p.bias = bias;
  p.bias_dtype = bias_dtype;
  p.residual = residual;
  p.y = y;
  p.y_dtype = y_dtype;
  p.epilogue = epilogue;
  // Both MMA operands must have the same 16-bit format (a bf16 x fp16 mix is rejected by the
  // hardware as an illegal instruction).  fp16 activations: fp16 codewords.  bf16 activations:
  // bf16 codewords, exact when the codebook is stored in bf16, otherwise the hi + lo split.
  const int w_fmt = x_dtype == DIMQ_BF16 ? 1 : 0;
  const bool split = w_fmt == 1 && precision != 1 && w->cb_dtype != DIMQ_BF16;
  p.w_fmt = w_fmt;
  p.idesc = tc::make_idesc_f16(w_fmt, w_fmt, kTileW, p.tx);
  p.x_stage_bytes = static_cast<uint32_t>(p.tx) * kBlockK * 2;
#ifdef DIMQ_B200_DIAG
  p.dbg = g_diag_dbg;
  p.prof = g_diag_prof_words >= static_cast<int64_t>(kNumSMs) * 32 ? g_diag_prof : nullptr;
#endif
  p.n_tiles = static_cast<int>((p.N + kTileW - 1) / kTileW);
  if (p.ksplit < 1) p.ksplit = 1;
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles * p.ksplit;
  if (tiles >= 0x7FFFFFFF) return DIMQ_ERR_TOO_LARGE;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);

  const bool pair = w->bits != 8 && table_bytes(w->bits, w->groups, true, split) <= (size_t)kMaxTableBytes;
  p.rep = 0;
#ifdef DIMQ_B200_DIAG
  p.rep = (g_diag_rep != 0 && (w->groups == 1 || w->group_rows % kTileW == 0)) ? 1 : 0;
#endif
  const size_t epi_bytes = p.epi_tma ? static_cast<size_t>(kNumEpilogueWarps) * 32 * 32 * (y_dtype == DIMQ_F32 ? 4 : 2) * (p.epi_res ? 3 : 1) : 0;
  const size_t fixed = 1024 + kHeaderBytes + epi_bytes + static_cast<size_t>(kIdxPrefetch) * kNumDequantWarps * 32 * (w->bits == 8 ? 64 : 32) +
                       (p.rep ? static_cast<size_t>(kNumDequantGroups) * kRepWords * 4 : 0) +
                       table_bytes(w->bits, w->groups, pair, split);
  const size_t kSmemMax = 227 * 1024;
  int x_stages = static_cast<int>((kSmemMax - fixed) / p.x_stage_bytes);
  if (x_stages > kXStages) x_stages = kXStages;
  if (x_stages < 3) return DIMQ_ERR_UNSUPPORTED;
  p.x_stages = x_stages;
  const size_t smem = fixed + static_cast<size_t>(x_stages) * p.x_stage_bytes;
#define DIMQ_TC_CASE(B)                                                                             \
  case B:                                                                                           \
    if (B != 8 && pair) return split ? launch_tc<B, B != 8, true>(tmaps, p, smem, grid, st)         \
                                     : launch_tc<B, B != 8, false>(tmaps, p, smem, grid, st);       \
    return split ? launch_tc<B, false, true>(tmaps, p, smem, grid, st)                              \
                 : launch_tc<B, false, false>(tmaps, p, smem, grid, st);
  switch (w->bits) {
#ifdef DIMQ_B200_DIAG_BITS   // diagnostics build: instantiate one index width only (shorter compile)
    DIMQ_TC_CASE(DIMQ_B200_DIAG_BITS)
#else
    DIMQ_TC_CASE(2)
    DIMQ_TC_CASE(3)
    DIMQ_TC_CASE(4)
    DIMQ_TC_CASE(8)
#endif
    default: return DIMQ_ERR_BAD_BITS;
  }
#undef DIMQ_TC_CASE
}

}  // namespace

// Split-K factor for a GEMM whose tiles would leave most SMs idle while each CTA walks a long K:
// a power of two that divides the k blocks, leaves at least four k blocks per slice and does not
// create more tiles than SMs.  1 = do not split.
int tc_split_k(int64_t M, int64_t N, int64_t K) {
  int tx = kTileX;
  {
    double best = -1.0;
    for (int c = 32; c <= kTileX; c += 32) {
      const double covered = static_cast<double>((M + c - 1) / c) * c;
      const double score = static_cast<double>(M) / covered * c / (c > 96 ? c : 96);
      if (score >= best) { best = score; tx = c; }
    }
  }
  const int64_t tiles = ((M + tx - 1) / tx) * ((N + kTileW - 1) / kTileW);
  const int64_t kb = K / kBlockK;
  int s = 1;
  while (s < 16 && tiles * (s * 2) <= kNumSMs && kb % (s * 2) == 0 && kb / (s * 2) >= 4) s *= 2;
  // a two-way split pays for the zeroing and the finishing kernel only when K is long
  return (s >= 4 || (s == 2 && kb >= 32)) ? s : 1;
}

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const float* __restrict__ ws, const void* __restrict__ bias, int bias_dtype,
                     const T* __restrict__ residual, T* __restrict__ y, int64_t total, int64_t N, int epilogue) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total) return;
  const float v = ws[i] + (bias != nullptr ? load_as_float(bias, bias_dtype, i % N) : 0.0f);
  const float res = residual != nullptr ? to_float<T>(residual[i]) : 0.0f;
  y[i] = from_float<T>(finish_value(v, epilogue, residual != nullptr, res));
}

}  // namespace

int launch_linear_wq_tc(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                        const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                        int precision, cudaStream_t st, void* workspace = nullptr, int64_t workspace_bytes = 0) {
  if (!tc_supported(x, x_dtype, w, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  EncodeTiledFn encode = get_encode_tiled();
  if (encode == nullptr) return DIMQ_ERR_DRIVER;
  TmapSet tmaps;
  memset(&tmaps, 0, sizeof(tmaps));
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  // activation rows per tile: 192 unless M is small or just above a multiple of a smaller tile, where a
  // narrower tile wastes fewer MMA columns (same throughput model as the convolution's tile choice)
  int tx_best = kTileX;
  double tx_score = -1.0;
  for (int tx = 32; tx <= kTileX; tx += 32) {
    const double covered = static_cast<double>((M + tx - 1) / tx) * tx;
    const double score = static_cast<double>(M) / covered * tx / (tx > 96 ? tx : 96);
    if (score >= tx_score) { tx_score = score; tx_best = tx; }
  }
  const cuuint32_t box[2] = {kBlockK, static_cast<cuuint32_t>(tx_best)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(&tmaps.m[0], x_dtype == DIMQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                            2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return DIMQ_ERR_DRIVER;
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = N;
  p.K = K;
  p.tx = tx_best;
  p.m_tiles = static_cast<int>((M + tx_best - 1) / tx_best);
  const int ksplit = workspace != nullptr ? tc_split_k(M, N, K) : 1;
  if (ksplit > 1) {
    // partial sums of the K slices meet in the caller's fp32 workspace; a second small kernel applies
    // bias / epilogue / residual and writes y
    if (workspace_bytes < M * N * 4) return DIMQ_ERR_SCRATCH_TOO_SMALL;
    if (!aligned(workspace, 16)) return DIMQ_ERR_ALIGNMENT;
    cudaError_t e = cudaMemsetAsync(workspace, 0, static_cast<size_t>(M) * N * 4, st);
    if (e != cudaSuccess) return static_cast<int>(e);
    p.ksplit = ksplit;
    p.ws = static_cast<float*>(workspace);
    int rc = finish_launch(tmaps, p, w, w->packed, x_dtype, nullptr, 0, nullptr, y, y_dtype, DIMQ_EPI_NONE, precision, st);
    if (rc != DIMQ_OK) return rc;
    const int64_t total = M * N;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    if (y_dtype == DIMQ_F32)
      splitk_finish_kernel<float><<<blocks, 256, 0, st>>>(p.ws, bias, bias_dtype, static_cast<const float*>(residual),
                                                          static_cast<float*>(y), total, N, epilogue);
    else if (y_dtype == DIMQ_F16)
      splitk_finish_kernel<__half><<<blocks, 256, 0, st>>>(p.ws, bias, bias_dtype, static_cast<const __half*>(residual),
                                                           static_cast<__half*>(y), total, N, epilogue);
    else
      splitk_finish_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(p.ws, bias, bias_dtype,
                                                                  static_cast<const __nv_bfloat16*>(residual),
                                                                  static_cast<__nv_bfloat16*>(y), total, N, epilogue);
    return launch_status();
  }
  if (epi_tma_possible(y, y_dtype, residual, N)) {
    const cuuint64_t odims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
    const cuuint32_t obox[2] = {32, 32};
    bool ok_maps = encode_out_map(encode, &tmaps.y, y, y_dtype, 2, odims, obox);
    if (ok_maps && residual != nullptr) ok_maps = encode_out_map(encode, &tmaps.r, residual, y_dtype, 2, odims, obox);
    if (ok_maps) { p.epi_tma = 1; p.epi_res = residual != nullptr ? 1 : 0; }
  }
  return finish_launch(tmaps, p, w, w->packed, x_dtype, bias, bias_dtype, residual, y, y_dtype, epilogue, precision, st);
}

// ---- implicit-GEMM convolution ----------------------------------------------------------------

bool conv_tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, int y_dtype) {
  if (w->packed_khwc == nullptr) return false;
  if (x_dtype != DIMQ_BF16 && x_dtype != DIMQ_F16) return false;
  if (y_dtype != x_dtype && y_dtype != DIMQ_F32) return false;
  if (g->groups != 1 || g->in_channels % kBlockK != 0) return false;
  if (g->stride_h != g->stride_w || (g->stride_h != 1 && g->stride_h != 2)) return false;
  // stride 2 reads the input through one tensor map per (row, column) parity; a one-pixel-wide or
  // one-pixel-high input has an empty parity plane, which no tensor map can describe
  if (g->stride_h == 2 && (g->in_w < 2 || g->in_h < 2)) return false;
  // channels_last storage of both tensors
  const int64_t C = g->in_channels, W = g->in_w, H = g->in_h;
  if (g->x_stride[1] != 1 || g->x_stride[3] != C || g->x_stride[2] != W * C || g->x_stride[0] != H * W * C) return false;
  const int64_t OC = g->out_channels, OW = g->out_w, OH = g->out_h;
  if (g->y_stride[1] != 1 || g->y_stride[3] != OC || g->y_stride[2] != OW * OC || g->y_stride[0] != OH * OW * OC) return false;
  if (!aligned(x, 16) || !aligned(w->packed_khwc, 16)) return false;
  if (table_bytes(w->bits, w->groups, false, true) > (size_t)kMaxTableBytes) return false;
  return g->batch >= 1 && OW >= 1 && OH >= 1;
}

int launch_conv2d_wq_tc(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                        const void* residual, void* y, int y_dtype, const dimq_conv_geom* g, int epilogue,
                        cudaStream_t st) {
  if (!conv_tc_supported(x, x_dtype, w, g, y_dtype)) return DIMQ_ERR_UNSUPPORTED;
  EncodeTiledFn encode = get_encode_tiled();
  if (encode == nullptr) return DIMQ_ERR_DRIVER;
  const int OW = g->out_w, OH = g->out_h, B = g->batch;
  // Tile = tw x th x tb output pixels (tx = tw*th*tb, a multiple of 16 up to 192).  Prefer the shape
  // that wastes the fewest MMA columns on positions outside the image, then the largest tile.
  int best_tx = 0, best_tw = 0, best_th = 0, best_tb = 0;
  double best_score = -1.0;
  // the TMA epilogue stores 32-pixel chunks as boxes: that needs tw and th to be powers of two
  // (tw <= 32) and tx a multiple of 32
  int pow_tx = 0, pow_tw = 0, pow_th = 0, pow_tb = 0;
  double pow_score = -1.0;
  for (int tx = kTileX; tx >= 16; tx -= 16) {
    for (int tw = 1; tw <= tx && tw <= 256; ++tw) {
      if (tx % tw != 0 || tw > OW + 15) continue;
      const int rest = tx / tw;
      for (int th = 1; th <= rest && th <= 256; ++th) {
        if (rest % th != 0 || th > OH + 15) continue;
        const int tb = rest / th;
        if (tb > 256) continue;
        const double covered = static_cast<double>((OW + tw - 1) / tw) * tw * ((OH + th - 1) / th) * th *
                               ((B + tb - 1) / tb) * tb;
        const double useful = static_cast<double>(OW) * OH * B / covered;
        // throughput model: a stage costs max(MMA time ~ tx, a fixed issue overhead ~ 96 columns)
        const double score = useful * tx / (tx > 96 ? tx : 96) + 1e-4 * tw;
        if (score > best_score) { best_score = score; best_tx = tx; best_tw = tw; best_th = th; best_tb = tb; }
        const bool pow2 = (tw & (tw - 1)) == 0 && (th & (th - 1)) == 0 && tw <= 32 && tx % 32 == 0;
        if (pow2 && score > pow_score) { pow_score = score; pow_tx = tx; pow_tw = tw; pow_th = th; pow_tb = tb; }
      }
    }
  }
  bool use_tma_epi = pow_tx != 0 && pow_score >= 0.8 * best_score && epi_tma_possible(y, y_dtype, residual, g->out_channels);
  if (use_tma_epi) { best_tx = pow_tx; best_tw = pow_tw; best_th = pow_th; best_tb = pow_tb; }
  if (best_tx == 0) return DIMQ_ERR_UNSUPPORTED;

  TcParams p;
  memset(&p, 0, sizeof(p));
  p.conv = 1;
  p.tx = best_tx;
  p.tw = best_tw;
  p.th = best_th;
  p.tb = best_tb;
  p.tiles_w = (OW + best_tw - 1) / best_tw;
  p.tiles_h = (OH + best_th - 1) / best_th;
  const int tiles_b = (B + best_tb - 1) / best_tb;
  p.m_tiles = p.tiles_w * p.tiles_h * tiles_b;
  p.OW = OW;
  p.OH = OH;
  p.Bn = B;
  p.stride = g->stride_h;
  p.pad_h = g->pad_h;
  p.pad_w = g->pad_w;
  p.dil_h = g->dilation_h;
  p.dil_w = g->dilation_w;
  p.KW = g->kernel_w;
  p.c_blocks = g->in_channels / kBlockK;
  p.M = static_cast<int64_t>(B) * OH * OW;
  p.N = g->out_channels;
  p.K = static_cast<int64_t>(g->kernel_h) * g->kernel_w * g->in_channels;

  TmapSet tmaps;
  memset(&tmaps, 0, sizeof(tmaps));
  const int s = g->stride_h;
  const int64_t C = g->in_channels, W = g->in_w, H = g->in_h;
  const CUtensorMapDataType dt = x_dtype == DIMQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  for (int py = 0; py < s; ++py) {
    for (int px = 0; px < s; ++px) {
      const int64_t Wp = (W - px + s - 1) / s, Hp = (H - py + s - 1) / s;
      CUtensorMap* m = &tmaps.m[py * s + px];
      if (Wp <= 0 || Hp <= 0) return DIMQ_ERR_UNSUPPORTED;   // excluded by conv_tc_supported
      const cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(Wp), static_cast<cuuint64_t>(Hp),
                                  static_cast<cuuint64_t>(B)};
      const cuuint64_t strides[3] = {static_cast<cuuint64_t>(s * C * 2), static_cast<cuuint64_t>(s * W * C * 2),
                                     static_cast<cuuint64_t>(H * W * C * 2)};
      const cuuint32_t box[4] = {kBlockK, static_cast<cuuint32_t>(best_tw), static_cast<cuuint32_t>(best_th),
                                 static_cast<cuuint32_t>(best_tb)};
      const cuuint32_t estr[4] = {1, 1, 1, 1};
      void* base = const_cast<char*>(static_cast<const char*>(x)) + (py * W + px) * C * 2;
      const CUresult r = encode(m, dt, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return DIMQ_ERR_DRIVER;
    }
  }
  if (use_tma_epi) {
    p.cbw = best_tw;                                         // tw <= 32
    p.cbh = best_th < 32 / best_tw ? best_th : 32 / best_tw;
    const int cbb = 32 / (p.cbw * p.cbh);
    const cuuint64_t odims[4] = {static_cast<cuuint64_t>(g->out_channels), static_cast<cuuint64_t>(OW),
                                 static_cast<cuuint64_t>(OH), static_cast<cuuint64_t>(B)};
    const cuuint32_t obox[4] = {32, static_cast<cuuint32_t>(p.cbw), static_cast<cuuint32_t>(p.cbh),
                                static_cast<cuuint32_t>(cbb)};
    bool ok_maps = encode_out_map(encode, &tmaps.y, y, y_dtype, 4, odims, obox);
    if (ok_maps && residual != nullptr) ok_maps = encode_out_map(encode, &tmaps.r, residual, y_dtype, 4, odims, obox);
    if (ok_maps) { p.epi_tma = 1; p.epi_res = residual != nullptr ? 1 : 0; }
  }
  return finish_launch(tmaps, p, w, w->packed_khwc, x_dtype, bias, bias_dtype, residual, y, y_dtype, epilogue, 0, st);
}

int read_device_status(uint32_t* status) { return tc::read_and_clear_device_status(status); }

namespace {

// One warp waits, with a poll limit the caller chooses, on an mbarrier that nothing ever arrives at,
// and reports what the bounded wait did: result[0] = 1 if the wait returned "gave up", result[1] = the
// CTA abort flag afterwards.  The status word is left set for dimq_last_device_status.
__global__ void __launch_bounds__(32, 1) bounded_wait_selftest_kernel(uint32_t polls, uint32_t* result) {
  __shared__ uint64_t bar;
  __shared__ volatile uint32_t abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    abort_flag = 0u;
    tc::fence_barrier_init();
  }
  __syncwarp();
  const bool got = tc::mbar_wait(tc::smem_u32(&bar), 0u, &abort_flag, 0x7E57u, polls);
  const bool all_gave_up = __all_sync(0xFFFFFFFFu, !got);
  __syncwarp();
  if (threadIdx.x == 0) {
    result[0] = all_gave_up ? 1u : 0u;
    result[1] = abort_flag;
  }
}

}  // namespace

int launch_bounded_wait_selftest(uint32_t polls, uint32_t* result, cudaStream_t st) {
  bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(polls, result);
  return launch_status();
}

}  // namespace dimq
