// Weight-only LUT GEMM / implicit-GEMM convolution for LARGE M in two steps.
//
//   1. lut_expand_kernel: every packed index is looked up ONCE and the codeword is written, in the
//      activations' 16-bit format, to a caller-owned scratch matrix W16[N][K] (a few MB: it stays in
//      the 126 MB L2).
//   2. lut_dense_tc_kernel: y = x * W16^T on the 5th-generation tensor cores.  Both operands are staged
//      by TMA (128-byte swizzle, no multicast) and read by tcgen05.mma from shared memory; fp32
//      accumulators live in tensor memory, double-buffered so that the epilogue of a tile overlaps the
//      main loop of the next.
//
// Why not look up inside the GEMM pipeline (lut_gemm_tc.cu does): there every CTA tile repeats the
// lookups of its 128 weight rows, i.e. the N*K lookups are done M/192 times - 131 times for the
// ViT-B/16 batch (M = 25 216) - and the lookup rate, not the tensor pipe, bounds the kernel (measured:
// 1 560 cycles per 64-k block against 384 cycles of MMA).  Here the lookups cost N*K once (~1 % of the
// GEMM's time) and the main loop is a plain two-operand TMA -> MMA pipeline.
//
// Tile: 128 activation rows (UMMA M, one TMEM lane each) x up to 256 weight rows (UMMA N = 256 is the
// shape whose four MMAs per 64-k block fill the tensor pipe: 512 cycles per block; narrower shapes pay
// about 240 cycles of wait / elect / commit per block beside 48-64 cycles per MMA).  For a GEMM whose tile
// counts favour it, two CTAs of a cluster share a 256 x 256 tile (cta_group::2, see the helpers below).
// Warp roles (448 threads): warp 0 and warps 10-13 fetch the tiles.  A warp gets through one copy instruction
// in ~330 cycles whatever its size (a 4-D box: ~555), so the producers take the k blocks of the CTA's sequence
// in turn, the owner of a block issuing both of its copies (never more producers than ring stages).  Warp 1 MMA
// issuer + TMEM owner, warps 2-9 epilogue (two per TMEM lane quarter, alternating 32-column chunks).
// Persistent grid, one CTA per SM.
// The accumulator is y-oriented (lane = output row m, column = output feature n): an epilogue thread
// holds 32 consecutive features of one row, adds bias / activation / residual, writes them as 16-byte
// vectors into a swizzled staging tile and one TMA store per 32 x 32 chunk writes y.
#include <cstring>

#include "tc_common.cuh"

namespace dimq {
namespace {

using namespace tc;

constexpr int kBM = 128;         // activation rows (output pixels) per tile
constexpr int kBK = 64;          // k per pipeline stage: 128 bytes of 16-bit elements
constexpr int kMaxStages = 8;
constexpr int kPairBlockCycles = 630, kSingleBlockCycles = 750;   // per 64-k block of a 256-wide tile (measured: a pair is ~15 % faster per block)
constexpr int kAccStages = 2;
constexpr int kAccCols = 256;    // TMEM columns per accumulator buffer
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 8;
constexpr int kProducers = 5;                         // warp 0 and the four warps after the epilogue warps
constexpr int kThreads = (1 + kProducers + kEpiWarps) * 32;
constexpr uint32_t kABytes = kBM * kBK * 2;   // 16 KB
constexpr int kHeaderBytes = 1024;
constexpr int kBiasBytes = kEpiWarps * 128;
constexpr size_t kSmemMax = 227 * 1024;

struct DenseParams {
  const void* bias;
  int bias_dtype;
  const void* residual;     // same element type and layout as y, or null
  int y_dtype;
  int64_t M, N;             // output rows (GEMM) / pixels (conv), output features
  int k_blocks;             // 64-k blocks of one pass over the reduction
  int passes;               // 2 when the scratch carries hi and lo terms of every codeword side by side
  int bn;                   // weight rows per tile: 64, 128 or 256
  int m_tiles, n_tiles;
  int stages;
  uint32_t b_bytes;         // bn * 128
  uint32_t idesc;
  int epilogue;
  // implicit-GEMM convolution: rows are output pixels, a tile is a tw x th x tb box of (ow, oh, batch)
  int conv;
  int tw, th, tb, tiles_w, tiles_h;
  int OW, OH, Bn;
  int stride, pad_h, pad_w, dil_h, dil_w, KW, c_blocks;
  int kps;                  // 64-k blocks per ring stage (1 or 2): narrow tiles amortise the per-stage wait / commit over 8 MMAs
  int b_res;                // convolution: the whole expanded weight (one tile wide) stays in shared memory
  int pair;                 // 1: CTA pairs (cta_group::2), GEMM only; m_tiles then counts 256-row pairs of blocks
#ifdef DIMQ_B200_DIAG
  int diag;
  unsigned long long* prof;   // 32 cycle counters per CTA, or null
#endif
};

#ifdef DIMQ_B200_DIAG
// diagnostics build: 1 = the producer skips the weight-tile copies, 2 = skips the activation-tile copies
// (timing experiments: results are wrong)
static int g_dense_diag = 0;
static unsigned long long* g_stem_prof = nullptr;
#endif

struct DenseMaps {
  CUtensorMap a[4];   // activations; conv: one map per (row, column) parity of a stride-2 input
  CUtensorMap b;      // expanded weights [N][passes * K]
  CUtensorMap y;      // output, boxes of 32 features x 32 rows / pixels
};

#ifdef DIMQ_B200_DIAG
#define STEM_CLK(v) const long long v = clock64()
#define STEM_ACC(slot, since) do { if (p.prof != nullptr && lane == 0) acc_[slot] += static_cast<unsigned long long>(clock64() - (since)); } while (0)
#define STEM_ACC_DECL unsigned long long acc_[8] = {0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull}
#define STEM_FLUSH(first, n) do { if (p.prof != nullptr && lane == 0) for (int q_ = 0; q_ < (n); ++q_) p.prof[blockIdx.x * 32 + (first) + q_] = acc_[q_]; } while (0)
#else
#define STEM_CLK(v)
#define STEM_ACC(slot, since)
#define STEM_ACC_DECL
#define STEM_FLUSH(first, n)
#endif

struct DenseHeader {
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t d_full[kAccStages], d_empty[kAccStages];
  uint64_t b_res_full;              // convolution with a resident weight: all its tiles have landed
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};
static_assert(sizeof(DenseHeader) <= kHeaderBytes, "header");

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float gelu_tanh16(float v) {
  const float u = v * fmaf(0.0356774081f, v * v, 0.7978845608f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float h = 0.5f * v;
  return fmaf(h, t, h);
}

constexpr int kEpiGelu16 = 16;   // GELU for 16-bit outputs: tanh form on the hardware tanh (see lut_gemm_tc.cu)

// 32 accumulators of one output row (+ bias) -> activation / residual, in place.
template <int EPI, bool RES>
__device__ __forceinline__ void finish_row(float (&v)[32], const float* __restrict__ bias_s, const float (&res)[32]) {
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    const float4 b = *reinterpret_cast<const float4*>(bias_s + 4 * j4);   // same address for all lanes: broadcast
    v[4 * j4] += b.x; v[4 * j4 + 1] += b.y; v[4 * j4 + 2] += b.z; v[4 * j4 + 3] += b.w;
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float x = v[j];
    if (EPI == DIMQ_EPI_ADD_RELU) {
      if (RES) x += res[j];
      x = fmaxf(x, 0.0f);
    } else {
      if (EPI == DIMQ_EPI_RELU) x = fmaxf(x, 0.0f);
      if (EPI == DIMQ_EPI_GELU) x = 0.5f * x * (1.0f + fast_erf(x * 0.70710678118654752440f));
      if (EPI == kEpiGelu16) x = gelu_tanh16(x);
      if (RES) x += res[j];
    }
    v[j] = x;
  }
}

// The same with the activation chosen at run time (warp-uniform).  Plain compares in order of
// frequency, not a switch: the jump table of a switch cost the epilogue 240 cycles per call.  For
// 16-bit outputs a ReLU that comes last is left to the conversion (cvt.rn.relu): returns true then.
template <int ES, bool RES>
__device__ __forceinline__ bool finish_row_epi(float (&v)[32], const float* bias_s, const float (&res)[32], int epilogue) {
  const bool relu_last = epilogue == DIMQ_EPI_ADD_RELU || (epilogue == DIMQ_EPI_RELU && !RES);
  if (epilogue == DIMQ_EPI_NONE || (ES == 2 && relu_last)) {
    finish_row<DIMQ_EPI_NONE, RES>(v, bias_s, res);
    return ES == 2 && relu_last;
  }
  if (epilogue == DIMQ_EPI_RELU) finish_row<DIMQ_EPI_RELU, RES>(v, bias_s, res);
  else if (epilogue == DIMQ_EPI_ADD_RELU) finish_row<DIMQ_EPI_ADD_RELU, RES>(v, bias_s, res);
  else if (ES == 2) finish_row<kEpiGelu16, RES>(v, bias_s, res);
  else finish_row<DIMQ_EPI_GELU, RES>(v, bias_s, res);
  return false;
}

// two floats -> one packed pair of 16-bit numbers (lo in the low half), optionally clamped at zero
template <bool BF16, bool RELU>
__device__ __forceinline__ uint32_t cvt_pair16(float lo, float hi) {
  uint32_t d;
  if (BF16) {
    if (RELU) asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  } else {
    if (RELU) asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  }
  return d;
}

// 32 values of one row as 16-bit numbers into a [32 rows][64 bytes] staging tile with the 64-byte swizzle
// (16-byte piece j of row r sits at piece j ^ ((r >> 1) & 3) = j ^ sw).
template <bool BF16, bool RELU>
__device__ __forceinline__ void stage_row16(const float (&v)[32], unsigned char* row_ptr, int sw) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = cvt_pair16<BF16, RELU>(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
    *reinterpret_cast<uint4*>(row_ptr + ((j ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__device__ __forceinline__ void stage_row16_any(const float (&v)[32], unsigned char* row_ptr, int sw, int y_dtype, bool relu) {
  if (y_dtype == DIMQ_BF16) {
    if (relu) stage_row16<true, true>(v, row_ptr, sw);
    else stage_row16<true, false>(v, row_ptr, sw);
  } else {
    if (relu) stage_row16<false, true>(v, row_ptr, sw);
    else stage_row16<false, false>(v, row_ptr, sw);
  }
}

// 32 residual values of one row: `p` points at the first of them (16-byte aligned), `valid` of them exist
// (a multiple of 8 for 16-bit elements, of 4 for fp32: the row pitch is a multiple of 16 bytes).
template <int ES>
__device__ __forceinline__ void load_residual(const void* p, int y_dtype, int valid, float (&res)[32]) {
  if (ES == 2) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 q = make_uint4(0u, 0u, 0u, 0u);
      if (8 * c + 8 <= valid) q = __ldg(reinterpret_cast<const uint4*>(p) + c);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (y_dtype == DIMQ_BF16) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
          res[8 * c + 2 * i] = f.x; res[8 * c + 2 * i + 1] = f.y;
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
          res[8 * c + 2 * i] = f.x; res[8 * c + 2 * i + 1] = f.y;
        }
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
      if (4 * c + 4 <= valid) q = __ldg(reinterpret_cast<const float4*>(p) + c);
      res[4 * c] = q.x; res[4 * c + 1] = q.y; res[4 * c + 2] = q.z; res[4 * c + 3] = q.w;
    }
  }
}

// CTA-pair helpers (cta_group::2): the two CTAs of a cluster work on one 256 x 256 tile.  Each loads its own
// 128 activation rows and its own half (128 rows) of the weight tile, and counts the bytes on the LEADER's
// (cluster rank 0) stage barrier; the leader issues M = 256 MMAs that read both CTAs' shared memory and write
// both CTAs' tensor memory; its commits arrive on the barriers of both CTAs (multicast).  Per CTA a 64-k block
// then needs 32 KB from L2 instead of 48 KB.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {   // the same shared address in CTA `rank` of the cluster
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void remote_arrive(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// TMA tile copy into this CTA's shared memory whose bytes are counted on a barrier of the cluster (no multicast)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {   // one arrival on `bar` in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

// ES = bytes per output element (2: bf16 / fp16, 4: fp32); PAIR: CTA pairs (GEMM only, bn = 256)
template <int ES, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
lut_dense_tc_kernel(const __grid_constant__ DenseMaps maps, const DenseParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // [stages: A 16 KB | B bn*128 B (all 1024-aligned)] [header] [bias slices] [staging tiles]
  // rounded up to 1024 bytes in the shared window; plain pointer arithmetic on the array keeps the
  // accesses below in the shared state space (no generic loads and stores)
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // b_res: [stages: A 16 KB] [the weight: k blocks x bn*128 B] [header] ...
  const uint32_t sub_bytes = p.b_res ? kABytes : kABytes + p.b_bytes;   // one 64-k block of a stage: A tile, then B tile
  const uint32_t stage_bytes = static_cast<uint32_t>(p.kps) * sub_bytes;
  const uint32_t n_st = static_cast<uint32_t>(p.stages);
  unsigned char* b_resident = smem + n_st * stage_bytes;
  DenseHeader* hdr = reinterpret_cast<DenseHeader*>(
      b_resident + (p.b_res ? static_cast<uint32_t>(p.k_blocks * p.passes) * p.b_bytes : 0u));
  float* bias_area = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(hdr) + kHeaderBytes);
  unsigned char* staging = reinterpret_cast<unsigned char*>(bias_area) + kBiasBytes;   // 1024-aligned
  constexpr uint32_t kStagingBytes = 32u * 32u * ES;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int num_tiles = p.m_tiles * p.n_tiles;   // PAIR: m_tiles counts 256-row pairs of blocks
  const int total_kb = p.k_blocks * p.passes;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int tile0 = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int tile_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

  if (tid == 0) {
    for (int s = 0; s < kMaxStages; ++s) { mbar_init(smem_u32(&hdr->full[s]), 1); mbar_init(smem_u32(&hdr->empty[s]), 1); }   // full: one arrival per producer warp
    for (int s = 0; s < kAccStages; ++s) { mbar_init(smem_u32(&hdr->d_full[s]), 1); mbar_init(smem_u32(&hdr->d_empty[s]), PAIR ? 2 * kEpiWarps : kEpiWarps); }
    mbar_init(smem_u32(&hdr->b_res_full), 1);
    hdr->abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&maps.a[0]);
    prefetch_tensormap(&maps.b);
    prefetch_tensormap(&maps.y);
  }
  if (warp == 1) {
    if constexpr (PAIR) {   // one warp of each CTA of the pair: the same columns in both tensor memories
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hdr->tmem_base)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      tmem_alloc(smem_u32(&hdr->tmem_base), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if constexpr (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  const uint32_t tmem_base = hdr->tmem_base;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  if (warp == 0 || warp >= 2 + kEpiWarps) {
    // ===================== TMA producers (whole warp loops, one elected lane issues) =====================
    // The producer warps take the k blocks of the CTA's sequence in turn; the owner of a block arms its stage
    // and issues both copies, back to back.  A warp gets through one copy instruction in ~330 cycles whatever
    // its size (measured alone: 64, 128 or 256 rows per copy, 1-D or 2-D, 334-363 cycles per copy and warp;
    // a 4-D box 554; N warps issue N times as many), so one warp issuing two copies per block held a GEMM
    // block at ~750 cycles and a convolution block, tap arithmetic included, at ~850.
    const uint32_t my_turn = warp == 0 ? 0u : static_cast<uint32_t>(warp - (1 + kEpiWarps));   // 0 .. kProducers - 1
    // No more producers than stages: a warp's successive blocks must be at most one ring revolution apart, or its
    // parity wait on a stage's `empty` barrier could be satisfied by the completion before the one it needs (five
    // producers over a four-stage ring overwrote live stages and ended in "unspecified launch failure").
    uint32_t n_turns = n_st < static_cast<uint32_t>(kProducers) ? n_st : static_cast<uint32_t>(kProducers), turn = 0;
#ifdef DIMQ_B200_DIAG
    if (p.diag & 32768) n_turns = 1;   // timing experiments: warp 0 issues every block's copies
#endif
    // programmatic dependent launch: the expansion kernel before this one in the stream must have finished
    // before the first weight tile is read (the activations were complete before that kernel started)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t stage = 0, phase = 0, issued = 0;
    bool ok = true;
    if (p.b_res && my_turn == 1) {
      // resident weight: every k block's tile once, one barrier for all of them; no per-stage weight copies
      if (elect_one()) {
        const uint32_t bar = smem_u32(&hdr->b_res_full);
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(total_kb) * p.b_bytes);
        for (int kb = 0; kb < total_kb; ++kb)
          tma_load_2d(smem_u32(b_resident + static_cast<uint32_t>(kb) * p.b_bytes), &maps.b, bar, kb * kBK, 0);
      }
      __syncwarp();
    }
    STEM_ACC_DECL;
    STEM_CLK(t_all);
    for (int t = tile0; t < num_tiles && ok; t += tile_step) {
      const int n_blk = t % p.n_tiles, m_blk = PAIR ? 2 * (t / p.n_tiles) + static_cast<int>(rank) : t / p.n_tiles;
      int ow0 = 0, oh0 = 0, b0 = 0;
      if (p.conv) {
        ow0 = (m_blk % p.tiles_w) * p.tw;
        oh0 = ((m_blk / p.tiles_w) % p.tiles_h) * p.th;
        b0 = (m_blk / (p.tiles_w * p.tiles_h)) * p.tb;
      }
      int g = 0, sub = 0;      // k block of the tile (over all passes), position inside the current stage
      bool mine = false;
      uint32_t full = 0, dst = 0;
      for (int pass = 0; pass < p.passes && ok; ++pass) {
        // convolution: k block kb = (tap (kh, kw), channel block cb); the tap's input offset is kept by carrying
        int kh = 0, kw = 0, cb = 0;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++g) {
          if (sub == 0) {   // a new stage: its owner waits for it and arms it with the bytes of all its blocks
            mine = turn == my_turn;
            if (++turn == n_turns) turn = 0;
            if (mine) {
              STEM_CLK(t_w);
              if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->empty[stage]), phase ^ 1u, abort_flag, 0x1100u | stage))) { ok = false; break; }
              STEM_ACC(1, t_w);
              full = smem_u32(&hdr->full[stage]);
              dst = smem_u32(smem + stage * stage_bytes);
              const int left = total_kb - g;
              const uint32_t bytes = static_cast<uint32_t>(left < p.kps ? left : p.kps) * sub_bytes;
              if (elect_one()) {
                if constexpr (PAIR) { if (rank == 0) mbar_arrive_expect_tx(full, 2 * bytes); }   // both CTAs' copies
                else mbar_arrive_expect_tx(full, bytes);
              }
              __syncwarp();
            }
          }
          if (mine) {
            STEM_CLK(t_is);
            const uint32_t dst_a = dst + static_cast<uint32_t>(sub) * sub_bytes;
            const int kcol_b = g * kBK;
            if (!p.conv) {
              if constexpr (PAIR) {
                if (elect_one()) {
                  const uint32_t lead_full = map_to_cta(full, 0);
                  tma_load_2d_pair(dst_a, &maps.a[0], lead_full, kb * kBK, m_blk * kBM);
                  tma_load_2d_pair(dst_a + kABytes, &maps.b, lead_full, kcol_b, n_blk * p.bn + static_cast<int>(rank) * (p.bn / 2));
                }
              } else if (elect_one()) {
                tma_load_2d(dst_a, &maps.a[0], full, kb * kBK, m_blk * kBM);
                tma_load_2d(dst_a + kABytes, &maps.b, full, kcol_b, n_blk * p.bn);
              }
            } else {
              // input pixel = stride * out + tap offset.  With stride 2 the input is addressed through one
              // tensor map per (row, column) parity, so the box stays dense; taps that fall outside the image
              // read the zero fill.
              const int dy = kh * p.dil_h - p.pad_h, dx = kw * p.dil_w - p.pad_w;
              int map = 0, hy = oh0 + dy, wx = ow0 + dx;
              if (p.stride == 2) {
                const int py = dy & 1, px = dx & 1;
                map = py * 2 + px;
                hy = oh0 + ((dy - py) >> 1);
                wx = ow0 + ((dx - px) >> 1);
              }
              if (elect_one()) {
                tma_load_4d(dst_a, &maps.a[map], full, cb * kBK, wx, hy, b0);
                if (!p.b_res) tma_load_2d(dst_a + kABytes, &maps.b, full, kcol_b, n_blk * p.bn);
              }
            }
            __syncwarp();
            STEM_ACC(2, t_is);
          }
          if (++sub == p.kps || g + 1 == total_kb) {   // the stage is complete (a tile's last stage may hold one block)
            sub = 0;
            ++issued;
            if (++stage == n_st) { stage = 0; phase ^= 1u; }
          }
          if (++cb == p.c_blocks) {
            cb = 0;
            if (++kw == p.KW) { kw = 0; ++kh; }
          }
        }
      }
    }
    STEM_ACC(0, t_all);
    if (warp == 0) STEM_FLUSH(0, 3);
    if (!ok && lane == 0) {
      // gave up: wait (bounded) for the copies still in flight so that none lands after the CTA has exited
      const uint32_t n_back = issued < n_st ? issued : n_st;
      uint32_t s = stage, ph = phase;
      for (uint32_t i = 0; i < n_back; ++i) {
        if (s == 0) { s = n_st - 1; ph ^= 1u; } else { --s; }
        for (uint32_t it = 0; it < kSpinLimit; ++it)
          if (mbar_try_wait(smem_u32(&hdr->full[s]), ph)) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer (whole warp loops, one elected lane issues) =====================
    // PAIR: only the leader CTA issues; its MMAs and commits act on both CTAs
    uint32_t stage = 0, phase = 0, as = 0, aph = 0;
    bool ok = !PAIR || rank == 0;
    const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem));
    const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(p.b_res ? b_resident : smem + kABytes));
    const uint32_t a_lo0 = static_cast<uint32_t>(a_desc0), a_hi = static_cast<uint32_t>(a_desc0 >> 32);
    const uint32_t b_lo0 = static_cast<uint32_t>(b_desc0), b_hi = static_cast<uint32_t>(b_desc0 >> 32);
    if (p.b_res && ok && !__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->b_res_full), 0u, abort_flag, 0x1A00u))) ok = false;
    STEM_ACC_DECL;
    STEM_CLK(t_all);
    for (int t = tile0; t < num_tiles && ok; t += tile_step) {
      STEM_CLK(t_w1);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->d_empty[as]), aph ^ 1u, abort_flag, 0x1200u | as))) { ok = false; break; }
      STEM_ACC(1, t_w1);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + as * kAccCols;
      for (int g = 0; g < total_kb; g += p.kps) {
        const int nblk = total_kb - g < p.kps ? total_kb - g : p.kps;   // 64-k blocks in this stage
        STEM_CLK(t_w2);
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->full[stage]), phase, abort_flag, 0x1300u | stage))) { ok = false; break; }
        STEM_ACC(2, t_w2);
        STEM_CLK(t_is);
        tc_fence_after();
        // descriptor low words (start address >> 4, 14 bits: shared addresses stay below 256 KB, so adding offsets
        // never carries out of the field); the high words never change
        const uint32_t a_lo = a_lo0 + ((stage * stage_bytes) >> 4);
        const uint32_t b_lo = p.b_res ? b_lo0 + static_cast<uint32_t>(g) * (p.b_bytes >> 4) : b_lo0 + ((stage * stage_bytes) >> 4);
        const uint32_t b_step = p.b_res ? p.b_bytes >> 4 : sub_bytes >> 4;
        if (elect_one()) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {      // kps <= 2
            if (i < nblk) {
              const uint32_t al = a_lo + static_cast<uint32_t>(i) * (sub_bytes >> 4), bl = b_lo + static_cast<uint32_t>(i) * b_step;
#pragma unroll
              for (int j = 0; j < kBK / 16; ++j) {  // 16 k = 32 bytes inside the swizzled row (encoded >> 4)
                const uint64_t a_desc = (static_cast<uint64_t>(a_hi) << 32) | (al + 2u * j);
                const uint64_t b_desc = (static_cast<uint64_t>(b_hi) << 32) | (bl + 2u * j);
                if constexpr (PAIR) mma_f16_ss_pair(d_tmem, a_desc, b_desc, p.idesc, (g | i | j) ? 1u : 0u);
                else mma_f16_ss(d_tmem, a_desc, b_desc, p.idesc, (g | i | j) ? 1u : 0u);
              }
            }
          }
          // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if constexpr (PAIR) mma_commit_pair(smem_u32(&hdr->empty[stage]));
          else mma_commit(smem_u32(&hdr->empty[stage]));
        }
        __syncwarp();
        STEM_ACC(3, t_is);
        if (++stage == n_st) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (elect_one()) {
        if constexpr (PAIR) mma_commit_pair(smem_u32(&hdr->d_full[as]));
        else mma_commit(smem_u32(&hdr->d_full[as]));
      }
      __syncwarp();
      if (++as == kAccStages) { as = 0; aph ^= 1u; }
    }
    STEM_ACC(0, t_all);
    STEM_FLUSH(4, 4);
  } else if (warp < 2 + kEpiWarps) {   // the last warp has no work in a GEMM: it must not fall into this branch
    // ===================== epilogue =====================
    const int quarter = warp & 3;          // TMEM lanes [32 quarter, 32 quarter + 32) = rows of the tile
    const int sub = (warp - 2) >> 2;       // which of the two warps of this quarter: chunks sub, sub + 2, ...
    const int ew = warp - 2;
    float* my_bias = bias_area + ew * 32;
    unsigned char* my_out = staging + ew * kStagingBytes;
    const int n_chunks = p.bn / 32;
    uint32_t as = 0, aph = 0;
    bool ok = true;
    STEM_ACC_DECL;
    STEM_CLK(t_all);
    for (int t = tile0; t < num_tiles && ok; t += tile_step) {
      const int n_blk = t % p.n_tiles, m_blk = PAIR ? 2 * (t / p.n_tiles) + static_cast<int>(rank) : t / p.n_tiles;
      // where this thread's output row lives (for the residual); the store itself goes through TMA
      int64_t row_off = -1;    // element offset of [row][0] in y, or -1 when the row is outside the tensor
      int c1 = 0, c2 = 0, c3 = 0;   // TMA store coordinates of this warp's 32 rows
      if (!p.conv) {
        const int64_t row = static_cast<int64_t>(m_blk) * kBM + quarter * 32 + lane;
        if (row < p.M) row_off = row * p.N;
        c1 = m_blk * kBM + quarter * 32;
      } else {
        const int pj = quarter * 32 + lane;
        const int ww = pj % p.tw, hh = (pj / p.tw) % p.th, bb = pj / (p.tw * p.th);
        const int ow = (m_blk % p.tiles_w) * p.tw + ww;
        const int oh = ((m_blk / p.tiles_w) % p.tiles_h) * p.th + hh;
        const int ob = (m_blk / (p.tiles_w * p.tiles_h)) * p.tb + bb;
        if (ob < p.Bn && oh < p.OH && ow < p.OW)
          row_off = ((static_cast<int64_t>(ob) * p.OH + oh) * p.OW + ow) * p.N;
        const int p0 = quarter * 32;         // all tile dimensions are powers of two: 32 pixels form a box
        c1 = (m_blk % p.tiles_w) * p.tw + p0 % p.tw;
        c2 = ((m_blk / p.tiles_w) % p.tiles_h) * p.th + (p0 / p.tw) % p.th;
        c3 = (m_blk / (p.tiles_w * p.tiles_h)) * p.tb + p0 / (p.tw * p.th);
      }
      // bias slices of this warp's chunks (at most four), one feature per lane, fetched before the wait for
      // the accumulator so that the global-memory latency is off the critical path
      float bj[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t nb = static_cast<int64_t>(n_blk) * p.bn + (sub + 2 * i) * 32 + lane;
        bj[i] = (p.bias != nullptr && sub + 2 * i < n_chunks && nb < p.N) ? load_as_float(p.bias, p.bias_dtype, nb) : 0.0f;
      }
      // tcgen05.ld is warp-collective: the whole warp proceeds or the whole warp gives up
      STEM_CLK(t_w1);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->d_full[as]), aph, abort_flag, 0x1500u | as))) { ok = false; break; }
      STEM_ACC(1, t_w1);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * kAccCols;
      if (sub >= n_chunks) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) remote_arrive(map_to_cta(smem_u32(&hdr->d_empty[as]), 0));
          else mbar_arrive(smem_u32(&hdr->d_empty[as]));
        }
      }
      for (int c = sub; c < n_chunks; c += 2) {
        const int64_t n_first = static_cast<int64_t>(n_blk) * p.bn + c * 32;
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(d_tmem + c * 32, r);
        {
          const int i = (c - sub) >> 1;
          my_bias[lane] = i == 0 ? bj[0] : i == 1 ? bj[1] : i == 2 ? bj[2] : bj[3];
        }
        tmem_ld_wait();
        if (c + 2 >= n_chunks) {
          // every column this warp reads of the buffer is in registers: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) remote_arrive(map_to_cta(smem_u32(&hdr->d_empty[as]), 0));   // the leader's MMA warp waits for both CTAs
            else mbar_arrive(smem_u32(&hdr->d_empty[as]));
          }
        }
        __syncwarp();
        if (n_first >= p.N) continue;        // chunk beyond the last feature (warp-uniform)
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        float res[32];
        const int64_t left = p.N - n_first;
        const int valid = left >= 32 ? 32 : static_cast<int>(left);
        bool relu_cvt;
        if (p.residual != nullptr) {
          if (row_off >= 0)
            load_residual<ES>(static_cast<const char*>(p.residual) + (row_off + n_first) * ES, p.y_dtype, valid, res);
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) res[j] = 0.0f;
          }
          relu_cvt = finish_row_epi<ES, true>(v, my_bias, res, p.epilogue);
        } else {
          relu_cvt = finish_row_epi<ES, false>(v, my_bias, res, p.epilogue);
        }
        // the previous store of this warp must have finished reading the staging tile
        if (elect_one()) tma_store_wait_read();
        __syncwarp();
        if (ES == 2) {
          // [32 rows][64 bytes], 64-byte swizzle: 16-byte piece j of row r sits at piece j ^ ((r >> 1) & 3)
          stage_row16_any(v, my_out + lane * 64, (lane >> 1) & 3, p.y_dtype, relu_cvt);
        } else {
          // [32 rows][128 bytes], 128-byte swizzle: piece j of row r sits at piece j ^ (r & 7)
          unsigned char* row_ptr = my_out + lane * 128;
          const int sw = lane & 7;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(row_ptr + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
#ifdef DIMQ_B200_DIAG
        if (!(p.diag & 16))
#endif
        if (elect_one()) {
          if (p.conv) tma_store_4d(&maps.y, smem_u32(my_out), static_cast<int>(n_first), c1, c2, c3);
          else tma_store_2d(&maps.y, smem_u32(my_out), static_cast<int>(n_first), c1);
          tma_store_commit();
        }
      }
      if (++as == kAccStages) { as = 0; aph ^= 1u; }
    }
    STEM_ACC(0, t_all);
    if (ew == 0) STEM_FLUSH(8, 2);
    __syncwarp();
    if (elect_one()) tma_store_wait_all();
    __syncwarp();
  }

  // ---- teardown -----------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // neither CTA leaves, or frees tensor memory, while the peer may still use it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else
      tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- step 1: expand the index stream to 16-bit codewords ---------------------------------------
// One thread = 32 consecutive indices of one row (4 * BITS bytes, 4-byte aligned because K % 64 == 0).
// out[row][k] (row pitch passes * K) = codeword in `fmt` (0 fp16, 1 bf16); with passes == 2 the bf16
// remainder c - bf16(c) goes to out[row][K + k], so that hi + lo carries the codeword to ~2^-17.
template <int BITS>
__global__ void __launch_bounds__(256)
lut_expand_kernel(const uint8_t* __restrict__ packed, const void* __restrict__ codebooks, int cb_dtype, int entries,
                  int64_t group_rows, int64_t rows, int64_t K, int fmt, int passes, uint16_t* __restrict__ out) {
  // the GEMM that follows in the stream is launched as a programmatic dependent: its prologue may start now,
  // and it waits (griddepcontrol.wait) before it reads what this kernel writes
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t units_per_row = K / 32;
  const int64_t total = rows * units_per_row;
  const int64_t u = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  // Up to 16-entry codebooks: the codewords of the groups this block's rows belong to are converted once
  // into a shared-memory table (hi | lo << 16), so an index costs one shared-memory read instead of a global
  // read and two conversions.  A block covers at most 256 * 32 / 64 = 128 rows, i.e. at most 129 groups.
  constexpr bool kTable = BITS <= 4;
  __shared__ uint32_t tbl[kTable ? 129 * 16 : 1];
  int64_t g_first = 0;
  if (kTable) {
    const int64_t u_first = static_cast<int64_t>(blockIdx.x) * 256;
    const int64_t u_last = u_first + 255 < total - 1 ? u_first + 255 : total - 1;
    g_first = (u_first / units_per_row) / group_rows;
    const int n_groups = static_cast<int>((u_last / units_per_row) / group_rows - g_first) + 1;
    for (int i = threadIdx.x; i < n_groups * 16; i += 256) {
      const int e = i & 15;
      const float c = e < entries ? load_as_float(codebooks, cb_dtype, (g_first + (i >> 4)) * entries + e) : 0.0f;
      uint32_t v;
      if (fmt == 0) {
        v = __half_as_ushort(__float2half_rn(c));
      } else {
        const __nv_bfloat16 h = __float2bfloat16_rn(c);
        v = __bfloat16_as_ushort(h) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(c - __bfloat162float(h)))) << 16);
      }
      tbl[i] = v;
    }
    __syncthreads();
  }
  if (u >= total) return;
  const int64_t row = u / units_per_row;
  const int64_t k0 = (u - row * units_per_row) * 32;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(packed + (row * K + k0) * BITS / 8);
  uint32_t w[BITS];
#pragma unroll
  for (int i = 0; i < BITS; ++i) w[i] = __ldg(src + i);
  const int64_t cb0 = (row / group_rows) * entries;
  const uint32_t* my_tbl = tbl + (kTable ? static_cast<int>(row / group_rows - g_first) * 16 : 0);
  uint16_t hi[32], lo[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int bit = i * BITS, word = bit >> 5, sh = bit & 31;
    uint32_t idx = w[word] >> sh;
    if (sh + BITS > 32) idx |= w[word + 1 < BITS ? word + 1 : word] << (32 - sh);
    idx &= (1u << BITS) - 1u;
    if (kTable) {
      const uint32_t v = my_tbl[idx];      // entries past the codebook's count hold zero
      hi[i] = static_cast<uint16_t>(v);
      lo[i] = static_cast<uint16_t>(v >> 16);
    } else {
      const float c = idx < static_cast<uint32_t>(entries) ? load_as_float(codebooks, cb_dtype, cb0 + idx) : 0.0f;
      if (fmt == 0) {
        hi[i] = __half_as_ushort(__float2half_rn(c));
        lo[i] = 0;
      } else {
        const __nv_bfloat16 h = __float2bfloat16_rn(c);
        hi[i] = __bfloat16_as_ushort(h);
        lo[i] = __bfloat16_as_ushort(__float2bfloat16_rn(c - __bfloat162float(h)));
      }
    }
  }
  uint16_t* dst = out + row * (K * passes) + k0;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 q;
    q.x = hi[8 * v] | (static_cast<uint32_t>(hi[8 * v + 1]) << 16);
    q.y = hi[8 * v + 2] | (static_cast<uint32_t>(hi[8 * v + 3]) << 16);
    q.z = hi[8 * v + 4] | (static_cast<uint32_t>(hi[8 * v + 5]) << 16);
    q.w = hi[8 * v + 6] | (static_cast<uint32_t>(hi[8 * v + 7]) << 16);
    reinterpret_cast<uint4*>(dst)[v] = q;
  }
  if (passes == 2) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint4 q;
      q.x = lo[8 * v] | (static_cast<uint32_t>(lo[8 * v + 1]) << 16);
      q.y = lo[8 * v + 2] | (static_cast<uint32_t>(lo[8 * v + 3]) << 16);
      q.z = lo[8 * v + 4] | (static_cast<uint32_t>(lo[8 * v + 5]) << 16);
      q.w = lo[8 * v + 6] | (static_cast<uint32_t>(lo[8 * v + 7]) << 16);
      reinterpret_cast<uint4*>(dst + K)[v] = q;
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(sym);
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

CUtensorMapDataType map_dtype(int dtype) {
  return dtype == DIMQ_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : (dtype == DIMQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
}

// Weight rows per tile: the candidate that needs the fewest cycles for the whole problem under a
// simple model - waves of tiles over the SMs times the measured cycles of a 64-k block (four MMAs and
// a commit: ~590 at N = 256, ~450 at N = 128, ~430 at N = 64: below N = 256 the per-instruction floor
// of about 106 cycles shows).
int choose_bn(int64_t m_tiles, int64_t N) {
  const int cand[3] = {256, 128, 64};
  const double cycles[3] = {590.0, 450.0, 430.0};
  int best = 256;
  double best_cost = -1.0;
  for (int i = 0; i < 3; ++i) {
    const int64_t tiles = m_tiles * ((N + cand[i] - 1) / cand[i]);
    const double cost = static_cast<double>((tiles + kNumSMs - 1) / kNumSMs) * cycles[i];
    if (best_cost < 0.0 || cost < best_cost) { best_cost = cost; best = cand[i]; }
  }
  return best;
}

int expand(const dimq_wq_weight* w, const uint8_t* packed, int64_t rows, int64_t K, int fmt, int passes, void* scratch,
           cudaStream_t st) {
  const int64_t units = rows * (K / 32);
  const unsigned blocks = static_cast<unsigned>((units + 255) / 256);
  uint16_t* out = static_cast<uint16_t*>(scratch);
#define DIMQ_EXPAND_CASE(B)                                                                                     \
  case B:                                                                                                       \
    lut_expand_kernel<B><<<blocks, 256, 0, st>>>(packed, w->codebooks, w->cb_dtype, w->entries, w->group_rows,  \
                                                 rows, K, fmt, passes, out);                                    \
    break;
  switch (w->bits) {
    DIMQ_EXPAND_CASE(2)
    DIMQ_EXPAND_CASE(3)
    DIMQ_EXPAND_CASE(4)
    DIMQ_EXPAND_CASE(8)
    default: return DIMQ_ERR_BAD_BITS;
  }
#undef DIMQ_EXPAND_CASE
  return launch_status();
}

// Shared tail of the GEMM and the convolution launchers: weight map, shared-memory budget, launch.
// Launch as a programmatic dependent of the kernel before it in the stream (the weight expansion): the
// prologue (barriers, TMEM, tensor-map prefetch, the first activation copies) overlaps that kernel's tail
// and the launch latency; the kernel itself waits before it reads the expanded weight.
template <typename Kern, typename Maps, typename Params>
cudaError_t launch_dependent(Kern kern, int grid, int threads, size_t smem, cudaStream_t st, const Maps& maps, const Params& p,
                             int cluster = 1) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster > 1) {   // CTA pairs: consecutive CTAs of the grid form a cluster
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
#ifdef DIMQ_B200_DIAG
  if ((g_dense_diag & 1024) && cluster == 1) cfg.numAttrs = 0;   // timing experiment: plain stream order
#endif
  return cudaLaunchKernelEx(&cfg, kern, maps, p);
}

int launch_dense(DenseMaps& maps, DenseParams& p, const void* scratch, int64_t K, int x_dtype, const void* bias,
                 int bias_dtype, const void* residual, int y_dtype, int epilogue, cudaStream_t st) {
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return DIMQ_ERR_DRIVER;
  p.bias = bias;
  p.bias_dtype = bias_dtype;
  p.residual = residual;
  p.y_dtype = y_dtype;
  p.epilogue = epilogue;
  p.k_blocks = static_cast<int>(K / kBK);
  const bool pair = p.pair != 0;   // CTA pairs: each CTA stages half of the 256 weight rows of a tile
  p.b_bytes = static_cast<uint32_t>(pair ? p.bn / 2 : p.bn) * kBK * 2;
#ifdef DIMQ_B200_DIAG
  p.diag = g_dense_diag;
  p.prof = g_stem_prof;
#endif
  const int fmt = x_dtype == DIMQ_BF16 ? 1 : 0;
  p.idesc = tc::make_idesc_f16(fmt, fmt, pair ? 2 * kBM : kBM, p.bn);
  const cuuint64_t bdims[2] = {static_cast<cuuint64_t>(K * p.passes), static_cast<cuuint64_t>(p.N)};
  const cuuint64_t bstr[1] = {static_cast<cuuint64_t>(K * p.passes) * 2};
  const cuuint32_t bbox[2] = {kBK, static_cast<cuuint32_t>(pair ? p.bn / 2 : p.bn)};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(&maps.b, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
             const_cast<void*>(scratch), bdims, bstr, bbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return DIMQ_ERR_DRIVER;
  const int es = y_dtype == DIMQ_F32 ? 4 : 2;
  const size_t fixed = 1024 + kHeaderBytes + kBiasBytes + static_cast<size_t>(kEpiWarps) * 32 * 32 * es;
  // Narrow tiles (bn <= 128) put two 64-k blocks into a ring stage: the MMA warp's wait / elect / commit of a
  // stage costs ~240 cycles beside 48-64 per MMA, so eight MMAs per stage nearly halve its time per block.
  // A convolution whose expanded weight is one tile wide and fits beside the activation stages keeps it in
  // shared memory: no per-stage weight copies.
  p.kps = (!pair && p.bn <= 128) ? 2 : 1;
#ifdef DIMQ_B200_DIAG
  if (g_dense_diag & 65536) p.kps = 1;   // timing experiments: one block per stage
#endif
  size_t stage_bytes = 0, resident = 0;
  int stages = 0;
  for (;;) {
    p.b_res = 0;
    resident = 0;
    size_t sub = kABytes + p.b_bytes;
    if (p.conv && !pair && p.n_tiles == 1) {
      const size_t need = static_cast<size_t>(p.k_blocks) * p.passes * p.b_bytes;
      if (fixed + need + 3 * static_cast<size_t>(p.kps) * kABytes <= kSmemMax && need < (1u << 20)) {
        p.b_res = 1;
        resident = need;
        sub = kABytes;
      }
    }
#ifdef DIMQ_B200_DIAG
    if ((g_dense_diag & 16384) && p.b_res) { p.b_res = 0; resident = 0; sub = kABytes + p.b_bytes; }
#endif
    stage_bytes = static_cast<size_t>(p.kps) * sub;
    stages = static_cast<int>((kSmemMax - fixed - resident) / stage_bytes);
    if (stages >= 3 || p.kps == 1) break;
    p.kps = 1;   // two blocks per stage do not leave three stages: one block per stage
  }
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 3) return DIMQ_ERR_UNSUPPORTED;
  p.stages = stages;
  const size_t smem = fixed + resident + stages * stage_bytes;
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
  if (tiles >= 0x7FFFFFFF) return DIMQ_ERR_TOO_LARGE;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  cudaError_t e;
  if (pair) {
    const int clusters = static_cast<int>(tiles < kNumSMs / 2 ? tiles : kNumSMs / 2);
    if (es == 2) {
      e = cudaFuncSetAttribute(lut_dense_tc_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      e = launch_dependent(lut_dense_tc_kernel<2, true>, 2 * clusters, kThreads, smem, st, maps, p, 2);
    } else {
      e = cudaFuncSetAttribute(lut_dense_tc_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      e = launch_dependent(lut_dense_tc_kernel<4, true>, 2 * clusters, kThreads, smem, st, maps, p, 2);
    }
  } else if (es == 2) {
    e = cudaFuncSetAttribute(lut_dense_tc_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    e = launch_dependent(lut_dense_tc_kernel<2, false>, grid, kThreads, smem, st, maps, p);
  } else {
    e = cudaFuncSetAttribute(lut_dense_tc_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    e = launch_dependent(lut_dense_tc_kernel<4, false>, grid, kThreads, smem, st, maps, p);
  }
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_status();
}

bool out_map(EncodeTiledFn encode, CUtensorMap* m, const void* base, int dtype, int rank, const cuuint64_t* dims,
             const cuuint32_t* box) {
  const cuuint64_t es = dtype == DIMQ_F32 ? 4 : 2;
  cuuint64_t strides[3];
  cuuint64_t acc = dims[0] * es;
  for (int i = 0; i < rank - 1; ++i) { strides[i] = acc; acc *= dims[i + 1]; }
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode(m, map_dtype(dtype), rank, const_cast<void*>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, es == 4 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// hi + lo split of the codewords: bf16 activations with a codebook that is not stored in bf16
int passes_for(int x_dtype, const dimq_wq_weight* w) { return (x_dtype == DIMQ_BF16 && w->cb_dtype != DIMQ_BF16) ? 2 : 1; }

}  // namespace

int read_dense_status(uint32_t* status) { return tc::read_and_clear_device_status(status); }
#ifdef DIMQ_B200_DIAG
void dense_diag_configure(int mode) { g_dense_diag = mode; }
void stem_diag_prof(unsigned long long* prof) { g_stem_prof = prof; }   // 16 words per SM, or null
#endif

// ---- GEMM ----------------------------------------------------------------------------------------

// Smallest M for which expanding the weight first pays (below it the in-pipeline kernel or its split-K
// form runs: the expansion and the second launch cost a few microseconds).
constexpr int64_t kDenseMinRows = 1024;

bool dense_pays(int64_t rows) { return rows >= kDenseMinRows; }

bool dense_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const void* y, int y_dtype,
                     const void* residual, int64_t M, int64_t N, int64_t K) {
  if (x_dtype != DIMQ_BF16 && x_dtype != DIMQ_F16) return false;
  if (y_dtype != x_dtype && y_dtype != DIMQ_F32) return false;
  if (M < 1 || N < 1 || K < kBK || K % kBK != 0) return false;
  if (M > 0x7FFFFFFF / 2 || N > 0x7FFFFFFF / 2) return false;
  const int64_t es = y_dtype == DIMQ_F32 ? 4 : 2;
  if (!aligned(x, 16) || !aligned(w->packed, 4) || !aligned(y, 16) || (N * es) % 16 != 0) return false;
  if (residual != nullptr && !aligned(residual, 16)) return false;
  return w->bits == 2 || w->bits == 3 || w->bits == 4 || w->bits == 8;
}

int64_t dense_workspace_bytes(int x_dtype, const dimq_wq_weight* w, int64_t N, int64_t K) {
  return N * K * 2 * passes_for(x_dtype, w);
}

// CTA pairs pay when the single-CTA tiling is the 128 x 256 one and the pair tiling's waves (74 clusters) at its
// per-block cost come out ahead of the single-CTA waves (148 CTAs) at theirs.
bool pair_pays(int m_blocks, int64_t N, int64_t k_total, int bn) {
#ifdef DIMQ_B200_DIAG
  if (g_dense_diag & 2048) return bn == 256;    // timing experiments: always / never
  if (g_dense_diag & 4096) return false;
#endif
  if (bn != 256) return false;
  const int64_t n_tiles = (N + 255) / 256;
  const int64_t single = static_cast<int64_t>(m_blocks) * n_tiles, pairs = static_cast<int64_t>((m_blocks + 1) / 2) * n_tiles;
  const int64_t waves_single = (single + kNumSMs - 1) / kNumSMs, waves_pair = (pairs + kNumSMs / 2 - 1) / (kNumSMs / 2);
  (void)k_total;
  return waves_pair * kPairBlockCycles < waves_single * kSingleBlockCycles;
}

int launch_linear_wq_dense(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                           const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                           void* workspace, int64_t workspace_bytes, cudaStream_t st) {
  if (!dense_supported(x, x_dtype, w, y, y_dtype, residual, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < dense_workspace_bytes(x_dtype, w, N, K)) return DIMQ_ERR_SCRATCH_TOO_SMALL;
  if (!aligned(workspace, 16)) return DIMQ_ERR_ALIGNMENT;
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return DIMQ_ERR_DRIVER;
  DenseParams p;
  memset(&p, 0, sizeof(p));
  DenseMaps maps;
  memset(&maps, 0, sizeof(maps));
  p.M = M;
  p.N = N;
  p.passes = passes_for(x_dtype, w);
  p.m_tiles = static_cast<int>((M + kBM - 1) / kBM);
  p.bn = choose_bn(p.m_tiles, N);
  p.n_tiles = static_cast<int>((N + p.bn - 1) / p.bn);
  if (pair_pays(p.m_tiles, N, K * p.passes, p.bn)) {
    p.pair = 1;
    p.bn = 256;
    p.m_tiles = (p.m_tiles + 1) / 2;
    p.n_tiles = static_cast<int>((N + 255) / 256);
  }
  const CUtensorMapDataType dt = x_dtype == DIMQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint64_t adims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
  const cuuint64_t astr[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t abox[2] = {kBK, kBM};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(&maps.a[0], dt, 2, const_cast<void*>(x), adims, astr, abox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return DIMQ_ERR_DRIVER;
  const cuuint64_t odims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
  const cuuint32_t obox[2] = {32, 32};
  if (!out_map(encode, &maps.y, y, y_dtype, 2, odims, obox)) return DIMQ_ERR_DRIVER;
  int rc = expand(w, w->packed, N, K, x_dtype == DIMQ_BF16 ? 1 : 0, p.passes, workspace, st);
  if (rc != DIMQ_OK) return rc;
  rc = launch_dense(maps, p, workspace, K, x_dtype, bias, bias_dtype, residual, y_dtype, epilogue, st);
  if (rc > 0 && p.pair) {
    // the cluster launch was refused (a positive status is the cudaError_t of the launch: e.g. a partition of the
    // GPU that cannot co-schedule CTA pairs): the same problem on single CTAs, over the weight already expanded
    (void)cudaGetLastError();
    p.pair = 0;
    p.m_tiles = static_cast<int>((M + kBM - 1) / kBM);
    p.bn = choose_bn(p.m_tiles, N);
    p.n_tiles = static_cast<int>((N + p.bn - 1) / p.bn);
    rc = launch_dense(maps, p, workspace, K, x_dtype, bias, bias_dtype, residual, y_dtype, epilogue, st);
  }
  return rc;
}

// ---- stem convolution: 3 input channels, stride 2 ----------------------------------------------------
//
// The first convolution of an image model (ResNet: 7x7, stride 2, pad 3, 3 -> 64) has too few input
// channels for 64-channel k blocks.  Here the patch matrix exists only in shared memory: the input window
// of a 16 x 8 output tile (NHWC, 6 bytes per pixel) is copied into shared memory, builder warps cut it into
// the 128 patch rows of the A operand (K-major, 128-byte swizzle) and the MMA warp multiplies them with the
// expanded weight, which stays resident in shared memory for the whole kernel.
//   k = kh * 24 + lead + kw * 3 + c   (lead = pad_w & 1, lead + KW * 3 <= 24, kh < KH <= 8; the rest of the
//   192 columns is zero)
// so the 24 slots of one kernel row of a patch are 24 consecutive input elements, and the lead slot makes
// that run start on a 4-byte boundary of the window whatever the padding.
// Warp roles (448 threads): warps 0-7 build A tiles (double-buffered), warp 8 issues the MMAs, warps 9-12 are
// the epilogue (bias / activation / residual, swizzled staging, one TMA store per 32 pixels x 32 channels),
// warp 13 fetches the input windows (one TMA box per tile, zero fill outside the image).
namespace {

constexpr int kStemTW = 16, kStemTH = 8;        // output tile: 16 x 8 pixels of one image = 128 rows
constexpr int kStemKRow = 24;                   // padded elements per kernel row (8 pixels x 3 channels)
constexpr int kStemK = 192;                     // padded reduction length: 3 k blocks of 64
constexpr int kStemBuilders = 8;
constexpr int kStemThreads = (kStemBuilders + 1 + 4 + 1) * 32;   // builders, MMA, epilogue, window producer
constexpr int kStemWinRows = 2 * (kStemTH - 1) + 8;          // input rows a tile can touch (KH <= 8): 22
// elements per window row: the 114 a tile's patches span, up to 7 more in front (the TMA box starts on a
// 16-byte boundary) - 144 makes the row pitch 72 words, which keeps the two half-warps of a patch read on
// different banks
constexpr int kStemWinPitch = 144;
constexpr uint32_t kStemABytes = kBM * kStemK * 2;           // 48 KB per A buffer
constexpr uint32_t kStemWinBytes = kStemWinRows * kStemWinPitch * 2;   // 6336: what one TMA box delivers
constexpr uint32_t kStemWinStride = (kStemWinBytes + 127u) & ~127u;      // a TMA box must land on a 128-byte boundary
constexpr int kStemWinBufs = 6;   // window ring (2..6 slots, as shared memory allows): the copies run several tiles ahead of the patch cutting (TMA latency)

struct StemParams {
  const void* x;            // NHWC 16-bit input, 3 channels
  const void* bias;
  int bias_dtype;
  const void* residual;
  int y_dtype;
  int64_t N;                // output channels (multiple of 16, <= 128)
  int H, W, OH, OW, Bn;
  int KH, KW, pad_h, pad_w;
  int tiles_w, tiles_h, m_tiles;
  int passes;
  int win_bufs;             // slots of the window ring in use
  int lead;                 // pad_w & 1: patch rows start one element early so that they are word-aligned in the window
#ifdef DIMQ_B200_DIAG
  int diag;                 // timing experiments (results are wrong): 4 = no patch cutting, 8 = no MMAs, 16 = no output stores, 32 = no window copies
  unsigned long long* prof; // 16 cycle counters per CTA, or null
#endif
  uint32_t b_bytes;         // N * 384 * passes
  uint32_t idesc;
  int epilogue;
};

struct StemMaps {
  CUtensorMap x;      // input as [B][H][W * 3] elements, boxes of one tile's window
  CUtensorMap b;      // expanded weight [N][192 * passes]
  CUtensorMap y;      // output NHWC, boxes of 32 channels x 16 x 2 pixels
};

struct StemHeader {
  uint64_t a_full[2], a_empty[2], d_full[2], d_empty[2], b_full, win_full[kStemWinBufs], win_empty[kStemWinBufs];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};


// Tile t = (image b, tile row, tile column); a CTA walks t = blockIdx.x, + gridDim.x, ... and keeps the three
// indices by carrying instead of dividing.
struct TileWalk {
  int tw, th, b, d_w, d_h, d_b, tiles_w, tiles_h;
  __device__ __forceinline__ void start(int t, int step, int tiles_w_, int tiles_h_) {
    tiles_w = tiles_w_; tiles_h = tiles_h_;
    tw = t % tiles_w; th = (t / tiles_w) % tiles_h; b = t / (tiles_w * tiles_h);
    d_w = step % tiles_w; d_h = (step / tiles_w) % tiles_h; d_b = step / (tiles_w * tiles_h);
  }
  __device__ __forceinline__ void next() {
    tw += d_w;
    th += d_h;
    if (tw >= tiles_w) { tw -= tiles_w; ++th; }
    b += d_b;
    if (th >= tiles_h) { th -= tiles_h; ++b; }
  }
};

template <int ES>
__global__ void __launch_bounds__(kStemThreads, 1)
lut_stem_conv_kernel(const __grid_constant__ StemMaps maps, const StemParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // [A0 | A1 (48 KB each)] [B: passes x 3 k blocks of N x 128 B] [header] [bias, one copy per epilogue warp] [staging] [windows]
  // rounded up to 1024 bytes in the shared window; plain pointer arithmetic on the array keeps the
  // accesses below in the shared state space (no generic loads and stores)
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* b_tile = smem + 2 * kStemABytes;
  StemHeader* hdr = reinterpret_cast<StemHeader*>(b_tile + p.b_bytes);
  float* bias_area = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(hdr) + kHeaderBytes);
  unsigned char* staging = reinterpret_cast<unsigned char*>(bias_area) + 2048;   // 1024-aligned
  constexpr uint32_t kStagingBytes = 32u * 32u * ES;
  unsigned char* windows = staging + 4 * kStagingBytes;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t kb_bytes = static_cast<uint32_t>(p.N) * 128u;   // one k block of the weight

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&hdr->a_full[s]), kStemBuilders);
      mbar_init(smem_u32(&hdr->a_empty[s]), 1);
      mbar_init(smem_u32(&hdr->d_full[s]), 1);
      mbar_init(smem_u32(&hdr->d_empty[s]), 4);
    }
    for (int s = 0; s < kStemWinBufs; ++s) {
      mbar_init(smem_u32(&hdr->win_full[s]), 1);
      mbar_init(smem_u32(&hdr->win_empty[s]), kStemBuilders);
    }
    mbar_init(smem_u32(&hdr->b_full), 1);
    hdr->abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&maps.x);
    prefetch_tensormap(&maps.b);
    prefetch_tensormap(&maps.y);
  }
  if (warp == kStemBuilders) {
    tmem_alloc(smem_u32(&hdr->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  // columns 168..191 of every patch row (k beyond KH * 24) never change: zero the two A buffers once
  for (uint32_t i = tid; i < 2 * kStemABytes / 16; i += kStemThreads) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  TileWalk walk;
  walk.start(blockIdx.x, gridDim.x, p.tiles_w, p.tiles_h);

  if (warp == kStemBuilders + 5) {
    // ===================== window producer =====================
    // One TMA box per tile: input rows 2 oh0 - pad_h .. + 21, elements from the 16-byte boundary at or
    // before pixel 2 ow0 - pad_w; rows and elements outside the image arrive as zeros.
    uint32_t buf = 0, phase = 0;
    bool ok = true;
    STEM_ACC_DECL;
    STEM_CLK(t_all);
    for (int t = blockIdx.x; t < p.m_tiles && ok; t += gridDim.x) {
      const int b = walk.b, oh0 = walk.th * kStemTH, ow0 = walk.tw * kStemTW;
      walk.next();
      STEM_CLK(t_w);
#ifdef DIMQ_B200_DIAG
      if (p.diag & 64) {
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_relaxed(smem_u32(&hdr->win_empty[buf]), phase ^ 1u, abort_flag, 0x2600u | buf))) { ok = false; break; }
      } else
#endif
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->win_empty[buf]), phase ^ 1u, abort_flag, 0x2600u | buf))) { ok = false; break; }
      STEM_ACC(1, t_w);
      const int e0 = (2 * ow0 - p.pad_w) * 3;
      const int x_al = e0 & ~7;                      // round down to 8 elements (also right for negatives)
#ifdef DIMQ_B200_DIAG
      if (p.diag & 32) {
        if (elect_one()) mbar_arrive(smem_u32(&hdr->win_full[buf]));
      } else
#endif
      if (elect_one()) {
        const uint32_t full = smem_u32(&hdr->win_full[buf]);
        mbar_arrive_expect_tx(full, kStemWinBytes);
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(smem_u32(windows + buf * kStemWinStride)), "l"(reinterpret_cast<uint64_t>(&maps.x)), "r"(full), "r"(x_al),
              "r"(2 * oh0 - p.pad_h), "r"(b)
            : "memory");
      }
      __syncwarp();
      if (++buf == static_cast<uint32_t>(p.win_bufs)) { buf = 0; phase ^= 1u; }
    }
    STEM_ACC(0, t_all);
    STEM_FLUSH(14, 2);
    if (!ok && lane == 0) {   // gave up: let the copy still in flight land before the CTA exits
      for (int s2 = 0; s2 < p.win_bufs; ++s2)
        for (uint32_t it = 0; it < kSpinLimit; ++it)
          if (mbar_try_wait(smem_u32(&hdr->win_full[s2]), 0u) || mbar_try_wait(smem_u32(&hdr->win_full[s2]), 1u)) break;
    }
    __syncwarp();
  } else if (warp < kStemBuilders) {
    // ===================== patch builders =====================
    uint32_t buf = 0, phase = 0, wbuf = 0, wphase = 0;   // A buffer / window ring positions
    bool ok = true;
    // Thread -> (patch row, kernel rows of one parity).  The 24 slots of kernel row kh are the window
    // elements from one before pixel 2 ow - pad_w (pad_w odd) or from that pixel (pad_w even): a word-aligned
    // run of 12 words, so a piece is four plain 32-bit loads.  Slots outside the KW * 3 values belong to
    // neighbouring pixels: their weights are zero, but a non-finite value there must not reach the product,
    // so they are cleared with masks computed once.
    const int row = tid & (kBM - 1), half = tid >> 7;
    const int oh_l = row >> 4, ow_l = row & 15;
    uint32_t mask[12];
#pragma unroll
    for (int m = 0; m < 12; ++m) {
      const int s0 = 2 * m - p.lead, s1 = 2 * m + 1 - p.lead;
      mask[m] = ((s0 >= 0 && s0 < p.KW * 3) ? 0x0000FFFFu : 0u) | ((s1 >= 0 && s1 < p.KW * 3) ? 0xFFFF0000u : 0u);
    }
    STEM_ACC_DECL;
    STEM_CLK(t_all);
    for (int t = blockIdx.x; t < p.m_tiles && ok; t += gridDim.x) {
      const int ow0 = walk.tw * kStemTW;
      walk.next();
      STEM_CLK(t_w1);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->win_full[wbuf]), wphase, abort_flag, 0x2700u | wbuf))) { ok = false; break; }
      STEM_ACC(1, t_w1);
      STEM_CLK(t_w2);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->a_empty[buf]), phase ^ 1u, abort_flag, 0x2100u | buf))) { ok = false; break; }
      STEM_ACC(2, t_w2);
      STEM_CLK(t_cut);
      const int e0 = (2 * ow0 - p.pad_w) * 3;
      const int off = e0 - (e0 & ~7);                  // distance of the first pixel from the box start; off - lead is even
      unsigned char* a_tile = smem + buf * kStemABytes + row * 128;
      const uint32_t* win32 = reinterpret_cast<const uint32_t*>(windows + wbuf * kStemWinStride) +
                              2 * oh_l * (kStemWinPitch / 2) + ((off - p.lead) >> 1) + 3 * ow_l;
#ifdef DIMQ_B200_DIAG
      if (!(p.diag & 4))
#endif
      for (int kh = half; kh < p.KH; kh += 2) {
        const uint32_t* src = win32 + kh * (kStemWinPitch / 2);
        uint32_t w12[12];
#pragma unroll
        for (int m = 0; m < 12; ++m) w12[m] = src[m] & mask[m];
#pragma unroll
        for (int part = 0; part < 3; ++part) {
          const int chunk = kh * 3 + part;
          *reinterpret_cast<uint4*>(a_tile + (chunk >> 3) * (kBM * 128) + (((chunk & 7) ^ (row & 7)) << 4)) =
              make_uint4(w12[4 * part], w12[4 * part + 1], w12[4 * part + 2], w12[4 * part + 3]);
        }
      }
      STEM_ACC(3, t_cut);
      STEM_CLK(t_fence);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&hdr->a_full[buf]));
        mbar_arrive(smem_u32(&hdr->win_empty[wbuf]));
      }
      STEM_ACC(4, t_fence);
      if (++buf == 2) { buf = 0; phase ^= 1u; }
      if (++wbuf == static_cast<uint32_t>(p.win_bufs)) { wbuf = 0; wphase ^= 1u; }
    }
    STEM_ACC(0, t_all);
    if (warp == 0) STEM_FLUSH(0, 4);
#ifdef DIMQ_B200_DIAG
    if (warp == 0 && p.prof != nullptr && lane == 0) p.prof[blockIdx.x * 32 + 16] = acc_[4];
#endif
  } else if (warp == kStemBuilders) {
    // ===================== MMA issuer =====================
    bool ok = true;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the expanded weight is written by the kernel before this one
    if (elect_one()) {
      mbar_arrive_expect_tx(smem_u32(&hdr->b_full), p.b_bytes);
      for (int kb = 0; kb < 3 * p.passes; ++kb)
        tma_load_2d(smem_u32(b_tile + kb * kb_bytes), &maps.b, smem_u32(&hdr->b_full), kb * kBK, 0);
    }
    __syncwarp();
    ok = __all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->b_full), 0u, abort_flag, 0x2200u));
    uint32_t buf = 0, phase = 0, as = 0, aph = 0;
    const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem));
    const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(b_tile));
    STEM_ACC_DECL;
    STEM_CLK(t_all);
    for (int t = blockIdx.x; t < p.m_tiles && ok; t += gridDim.x) {
      STEM_CLK(t_w1);
#ifdef DIMQ_B200_DIAG
      if (p.diag & 64) {
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_relaxed(smem_u32(&hdr->d_empty[as]), aph ^ 1u, abort_flag, 0x2300u | as))) { ok = false; break; }
      } else
#endif
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->d_empty[as]), aph ^ 1u, abort_flag, 0x2300u | as))) { ok = false; break; }
      STEM_ACC(1, t_w1);
      STEM_CLK(t_w2);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->a_full[buf]), phase, abort_flag, 0x2400u | buf))) { ok = false; break; }
      STEM_ACC(2, t_w2);
      tc_fence_after();
      if (elect_one()) {
        const uint32_t d_tmem = tmem_base + as * kAccCols;
#ifdef DIMQ_B200_DIAG
        if (!(p.diag & 8))
#endif
        for (int kb = 0; kb < 3 * p.passes; ++kb) {
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((buf * kStemABytes + (kb % 3) * (kBM * 128)) >> 4);
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((kb * kb_bytes) >> 4);
#pragma unroll
          for (int j = 0; j < kBK / 16; ++j)
            mma_f16_ss(d_tmem, a_desc + static_cast<uint64_t>(2 * j), b_desc + static_cast<uint64_t>(2 * j), p.idesc,
                       (kb | j) ? 1u : 0u);
        }
        mma_commit(smem_u32(&hdr->a_empty[buf]));
        mma_commit(smem_u32(&hdr->d_full[as]));
      }
      __syncwarp();
      if (++buf == 2) { buf = 0; phase ^= 1u; }
      if (++as == kAccStages) { as = 0; aph ^= 1u; }
    }
    STEM_ACC(0, t_all);
    STEM_FLUSH(4, 3);
  } else {
    // ===================== epilogue =====================
    const int quarter = warp & 3;          // TMEM lanes [32 quarter, +32): tile rows 2 quarter, 2 quarter + 1
    const int ew = warp - (kStemBuilders + 1);
    float* my_bias = bias_area + ew * 128;   // all N <= 128 bias values, read from global memory once
    unsigned char* my_out = staging + ew * kStagingBytes;
    const int n_chunks = static_cast<int>((p.N + 31) / 32);
    for (int j = lane; j < 128; j += 32) my_bias[j] = (p.bias != nullptr && j < p.N) ? load_as_float(p.bias, p.bias_dtype, j) : 0.0f;
    __syncwarp();
    uint32_t as = 0, aph = 0;
    bool ok = true;
    STEM_ACC_DECL;
    STEM_CLK(t_all);
    for (int t = blockIdx.x; t < p.m_tiles && ok; t += gridDim.x) {
      const int b = walk.b, oh0 = walk.th * kStemTH, ow0 = walk.tw * kStemTW;
      walk.next();
      const int pj = quarter * 32 + lane;
      const int oh = oh0 + (pj >> 4), ow = ow0 + (pj & 15);
      int64_t row_off = -1;
      if (p.residual != nullptr && oh < p.OH && ow < p.OW) row_off = ((static_cast<int64_t>(b) * p.OH + oh) * p.OW + ow) * p.N;
      STEM_CLK(t_w1);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->d_full[as]), aph, abort_flag, 0x2500u | as))) { ok = false; break; }
      STEM_ACC(1, t_w1);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * kAccCols;
      for (int c = 0; c < n_chunks; ++c) {
        const int64_t n_first = static_cast<int64_t>(c) * 32;
        uint32_t r[32];
        __syncwarp();
        STEM_CLK(t_ld);
        tmem_ld32(d_tmem + c * 32, r);
        tmem_ld_wait();
        STEM_ACC(7, t_ld);
        if (c + 1 == n_chunks) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&hdr->d_empty[as]));
        }
        float v[32], res[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        const int64_t left = p.N - n_first;
        const int valid = left >= 32 ? 32 : static_cast<int>(left);
        bool relu_cvt = false;
#ifdef DIMQ_B200_DIAG
        if (!(p.diag & 128))
#endif
        if (p.residual != nullptr) {
          if (row_off >= 0)
            load_residual<ES>(static_cast<const char*>(p.residual) + (row_off + n_first) * ES, p.y_dtype, valid, res);
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) res[j] = 0.0f;
          }
          relu_cvt = finish_row_epi<ES, true>(v, my_bias + c * 32, res, p.epilogue);
        } else {
          relu_cvt = finish_row_epi<ES, false>(v, my_bias + c * 32, res, p.epilogue);
        }
        STEM_ACC(2, t_ld);
        STEM_CLK(t_rd);
        if (elect_one()) tma_store_wait_read();
        __syncwarp();
        STEM_ACC(3, t_rd);
        STEM_CLK(t_sts);
        if (ES == 2) {
          stage_row16_any(v, my_out + lane * 64, (lane >> 1) & 3, p.y_dtype, relu_cvt);
        } else {
          unsigned char* row_ptr = my_out + lane * 128;
          const int sw = lane & 7;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(row_ptr + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        STEM_ACC(4, t_sts);
        STEM_CLK(t_fence);
        fence_proxy_async_smem();
        __syncwarp();
        STEM_ACC(5, t_fence);
        STEM_CLK(t_issue);
#ifdef DIMQ_B200_DIAG
        if (!(p.diag & 16))
#endif
        if (elect_one()) {
          tma_store_4d(&maps.y, smem_u32(my_out), static_cast<int>(n_first), ow0, oh0 + 2 * quarter, b);
          tma_store_commit();
        }
        __syncwarp();
        STEM_ACC(6, t_issue);
      }
      if (++as == kAccStages) { as = 0; aph ^= 1u; }
    }
    STEM_ACC(0, t_all);
    if (ew == 0) STEM_FLUSH(7, 7);
#ifdef DIMQ_B200_DIAG
    if (ew == 0 && p.prof != nullptr && lane == 0) p.prof[blockIdx.x * 32 + 17] = acc_[7];
#endif
    __syncwarp();
    if (elect_one()) tma_store_wait_all();
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kStemBuilders) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Expanded stem weight [N][192 * passes]: column kh * 24 + lead + kw * 3 + c of row n is the codeword of
// idx[n][c][kh][kw] (the reference's "conv_kcrs" stream), zero elsewhere; lo terms in the second pass.
__global__ void __launch_bounds__(256)
stem_expand_kernel(const uint8_t* __restrict__ packed, int bits, int64_t nbytes, const void* __restrict__ codebooks,
                   int cb_dtype, int entries, int64_t group_rows, int64_t N, int KH, int KW, int lead, int fmt,
                   int passes, uint16_t* __restrict__ out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // see lut_expand_kernel
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= N * kStemK) return;
  const int64_t n = i / kStemK;
  const int k = static_cast<int>(i - n * kStemK);
  const int kh = k / kStemKRow, j = k - kh * kStemKRow - lead;
  const int kw = j / 3, c = j - kw * 3;
  float v = 0.0f;
  if (kh < KH && j >= 0 && kw < KW) {
    const uint32_t idx = get_index(packed, ((n * 3 + c) * KH + kh) * KW + kw, bits, nbytes);
    if (idx < static_cast<uint32_t>(entries)) v = load_as_float(codebooks, cb_dtype, (n / group_rows) * entries + idx);
  }
  uint16_t hi, lo = 0;
  if (fmt == 0) {
    hi = __half_as_ushort(__float2half_rn(v));
  } else {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi = __bfloat16_as_ushort(h);
    lo = __bfloat16_as_ushort(__float2bfloat16_rn(v - __bfloat162float(h)));
  }
  out[n * (kStemK * passes) + k] = hi;
  if (passes == 2) out[n * (kStemK * passes) + kStemK + k] = lo;
}

}  // namespace

bool stem_conv_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, const void* y,
                         int y_dtype, const void* residual) {
  if (x_dtype != DIMQ_BF16 && x_dtype != DIMQ_F16) return false;
  if (y_dtype != x_dtype && y_dtype != DIMQ_F32) return false;
  if (g->groups != 1 || g->in_channels != 3) return false;
  if (g->stride_h != 2 || g->stride_w != 2 || g->dilation_h != 1 || g->dilation_w != 1) return false;
  if (g->kernel_h > 8 || g->kernel_w * 3 + (g->pad_w & 1) > kStemKRow) return false;   // one lead slot when pad_w is odd
  if (g->pad_h < 0 || g->pad_w < 0 || g->pad_h > 8 || g->pad_w > 8) return false;
  if (g->out_channels % 16 != 0 || g->out_channels > 128) return false;
  const int64_t W = g->in_w, H = g->in_h;
  if (g->x_stride[1] != 1 || g->x_stride[3] != 3 || g->x_stride[2] != W * 3 || g->x_stride[0] != H * W * 3) return false;
  const int64_t OC = g->out_channels, OW = g->out_w, OH = g->out_h;
  if (g->y_stride[1] != 1 || g->y_stride[3] != OC || g->y_stride[2] != OW * OC || g->y_stride[0] != OH * OW * OC) return false;
  const int64_t es = y_dtype == DIMQ_F32 ? 4 : 2;
  // the window is a TMA box over [B][H][W * 3]: 16-byte aligned base and row pitch
  if (!aligned(x, 16) || (W * 6) % 16 != 0 || !aligned(y, 16) || (OC * es) % 16 != 0) return false;
  if (residual != nullptr && !aligned(residual, 16)) return false;
  if (w->bits != 2 && w->bits != 3 && w->bits != 4 && w->bits != 8) return false;
  return g->batch >= 1 && OW >= 1 && OH >= 1;
}

int64_t stem_conv_workspace_bytes(int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g) {
  return static_cast<int64_t>(g->out_channels) * kStemK * 2 * passes_for(x_dtype, w);
}

int launch_stem_conv(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                     const void* residual, void* y, int y_dtype, const dimq_conv_geom* g, int epilogue, void* workspace,
                     int64_t workspace_bytes, cudaStream_t st) {
  if (!stem_conv_supported(x, x_dtype, w, g, y, y_dtype, residual)) return DIMQ_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < stem_conv_workspace_bytes(x_dtype, w, g)) return DIMQ_ERR_SCRATCH_TOO_SMALL;
  if (!aligned(workspace, 16)) return DIMQ_ERR_ALIGNMENT;
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return DIMQ_ERR_DRIVER;
  StemParams p;
  memset(&p, 0, sizeof(p));
  StemMaps maps;
  memset(&maps, 0, sizeof(maps));
  const int fmt = x_dtype == DIMQ_BF16 ? 1 : 0;
  p.x = x;
  p.bias = bias;
  p.bias_dtype = bias_dtype;
  p.residual = residual;
  p.y_dtype = y_dtype;
  p.N = g->out_channels;
  p.H = g->in_h; p.W = g->in_w; p.OH = g->out_h; p.OW = g->out_w; p.Bn = g->batch;
  p.KH = g->kernel_h; p.KW = g->kernel_w; p.pad_h = g->pad_h; p.pad_w = g->pad_w;
  p.lead = g->pad_w & 1;
  p.tiles_w = (p.OW + kStemTW - 1) / kStemTW;
  p.tiles_h = (p.OH + kStemTH - 1) / kStemTH;
  const int64_t m_tiles = static_cast<int64_t>(p.tiles_w) * p.tiles_h * p.Bn;
  if (m_tiles >= 0x7FFFFFFF) return DIMQ_ERR_TOO_LARGE;
  p.m_tiles = static_cast<int>(m_tiles);
  p.passes = passes_for(x_dtype, w);
  p.b_bytes = static_cast<uint32_t>(p.N) * kStemK * 2 * p.passes;
  p.idesc = tc::make_idesc_f16(fmt, fmt, kBM, static_cast<int>(p.N));
  p.epilogue = epilogue;
  const int64_t ktot = static_cast<int64_t>(kStemK) * p.passes;
  const cuuint64_t bdims[2] = {static_cast<cuuint64_t>(ktot), static_cast<cuuint64_t>(p.N)};
  const cuuint64_t bstr[1] = {static_cast<cuuint64_t>(ktot) * 2};
  const cuuint32_t bbox[2] = {kBK, static_cast<cuuint32_t>(p.N)};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(&maps.b, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, workspace, bdims,
             bstr, bbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return DIMQ_ERR_DRIVER;
  const cuuint64_t xdims[3] = {static_cast<cuuint64_t>(p.W) * 3, static_cast<cuuint64_t>(p.H), static_cast<cuuint64_t>(p.Bn)};
  const cuuint64_t xstr[2] = {static_cast<cuuint64_t>(p.W) * 6, static_cast<cuuint64_t>(p.H) * p.W * 6};
  const cuuint32_t xbox[3] = {kStemWinPitch, kStemWinRows, 1};
  const cuuint32_t xes[3] = {1, 1, 1};
  if (encode(&maps.x, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
             const_cast<void*>(x), xdims, xstr, xbox, xes, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return DIMQ_ERR_DRIVER;
  const cuuint64_t odims[4] = {static_cast<cuuint64_t>(p.N), static_cast<cuuint64_t>(p.OW), static_cast<cuuint64_t>(p.OH),
                               static_cast<cuuint64_t>(p.Bn)};
  const cuuint32_t obox[4] = {32, kStemTW, 2, 1};
  if (!out_map(encode, &maps.y, y, y_dtype, 4, odims, obox)) return DIMQ_ERR_DRIVER;
  const int64_t n_w = p.N * 3 * p.KH * p.KW;
  const int64_t total = p.N * kStemK;
  stem_expand_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(
      w->packed, w->bits, (n_w * w->bits + 7) / 8, w->codebooks, w->cb_dtype, w->entries, w->group_rows, p.N, p.KH, p.KW,
      p.lead, fmt, p.passes, static_cast<uint16_t*>(workspace));
  int rc = launch_status();
  if (rc != DIMQ_OK) return rc;
  const int es = y_dtype == DIMQ_F32 ? 4 : 2;
#ifdef DIMQ_B200_DIAG
  p.diag = g_dense_diag;
  p.prof = g_stem_prof;
#endif
  const size_t smem_fixed = 1024 + 2 * kStemABytes + p.b_bytes + kHeaderBytes + 2048 + 4 * 32 * 32 * es;
  if (smem_fixed + 2 * kStemWinStride > kSmemMax) return DIMQ_ERR_UNSUPPORTED;
  p.win_bufs = static_cast<int>((kSmemMax - smem_fixed) / kStemWinStride);
  if (p.win_bufs > kStemWinBufs) p.win_bufs = kStemWinBufs;
  const size_t smem = smem_fixed + p.win_bufs * kStemWinStride;
  const int grid = p.m_tiles < kNumSMs ? p.m_tiles : kNumSMs;
  cudaError_t e;
  if (es == 2) {
    e = cudaFuncSetAttribute(lut_stem_conv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    e = launch_dependent(lut_stem_conv_kernel<2>, grid, kStemThreads, smem, st, maps, p);
  } else {
    e = cudaFuncSetAttribute(lut_stem_conv_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    e = launch_dependent(lut_stem_conv_kernel<4>, grid, kStemThreads, smem, st, maps, p);
  }
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_status();
}

// ---- implicit-GEMM convolution ------------------------------------------------------------------------

bool conv_dense_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, const void* y,
                          int y_dtype, const void* residual) {
  if (w->packed_khwc == nullptr) return false;
  if (x_dtype != DIMQ_BF16 && x_dtype != DIMQ_F16) return false;
  if (y_dtype != x_dtype && y_dtype != DIMQ_F32) return false;
  if (g->groups != 1 || g->in_channels % kBK != 0) return false;
  if (g->stride_h != g->stride_w || (g->stride_h != 1 && g->stride_h != 2)) return false;
  if (g->stride_h == 2 && (g->in_w < 2 || g->in_h < 2)) return false;   // a parity plane would be empty
  const int64_t C = g->in_channels, W = g->in_w, H = g->in_h;
  if (g->x_stride[1] != 1 || g->x_stride[3] != C || g->x_stride[2] != W * C || g->x_stride[0] != H * W * C) return false;
  const int64_t OC = g->out_channels, OW = g->out_w, OH = g->out_h;
  if (g->y_stride[1] != 1 || g->y_stride[3] != OC || g->y_stride[2] != OW * OC || g->y_stride[0] != OH * OW * OC) return false;
  const int64_t es = y_dtype == DIMQ_F32 ? 4 : 2;
  if (!aligned(x, 16) || !aligned(w->packed_khwc, 4) || !aligned(y, 16) || (OC * es) % 16 != 0) return false;
  if (residual != nullptr && !aligned(residual, 16)) return false;
  return g->batch >= 1 && OW >= 1 && OH >= 1;
}

int64_t conv_dense_workspace_bytes(int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g) {
  return static_cast<int64_t>(g->out_channels) * g->kernel_h * g->kernel_w * g->in_channels * 2 * passes_for(x_dtype, w);
}

int launch_conv2d_wq_dense(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                           const void* residual, void* y, int y_dtype, const dimq_conv_geom* g, int epilogue,
                           void* workspace, int64_t workspace_bytes, cudaStream_t st) {
  if (!conv_dense_supported(x, x_dtype, w, g, y, y_dtype, residual)) return DIMQ_ERR_UNSUPPORTED;
  if (workspace == nullptr || workspace_bytes < conv_dense_workspace_bytes(x_dtype, w, g)) return DIMQ_ERR_SCRATCH_TOO_SMALL;
  if (!aligned(workspace, 16)) return DIMQ_ERR_ALIGNMENT;
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return DIMQ_ERR_DRIVER;
  const int OW = g->out_w, OH = g->out_h, B = g->batch;
  // Tile = tw x th x tb output pixels with tw * th * tb = 128, so every factor is a power of two and
  // any 32 consecutive tile pixels form a box (the TMA store of the epilogue needs that).  Prefer the
  // shape that wastes the fewest rows on positions outside the image, then the widest.
  int best_tw = 0, best_th = 0, best_tb = 0;
  double best_score = -1.0;
  for (int tw = 1; tw <= kBM; tw *= 2) {
    for (int th = 1; tw * th <= kBM; th *= 2) {
      const int tb = kBM / (tw * th);
      const double covered = static_cast<double>((OW + tw - 1) / tw) * tw * ((OH + th - 1) / th) * th * ((B + tb - 1) / tb) * tb;
      const double score = static_cast<double>(OW) * OH * B / covered + 1e-4 * tw + 1e-6 * th;
      if (score > best_score) { best_score = score; best_tw = tw; best_th = th; best_tb = tb; }
    }
  }
#ifdef DIMQ_B200_DIAG
  if (g_dense_diag >> 16) {   // timing experiments: forced tile shape, log2(tw) | log2(th) << 4 in bits 16..23
    best_tw = 1 << ((g_dense_diag >> 16) & 15);
    best_th = 1 << ((g_dense_diag >> 20) & 15);
    best_tb = kBM / (best_tw * best_th);
  }
#endif
  DenseParams p;
  memset(&p, 0, sizeof(p));
  DenseMaps maps;
  memset(&maps, 0, sizeof(maps));
  p.conv = 1;
  p.tw = best_tw;
  p.th = best_th;
  p.tb = best_tb;
  p.tiles_w = (OW + best_tw - 1) / best_tw;
  p.tiles_h = (OH + best_th - 1) / best_th;
  const int64_t m_tiles = static_cast<int64_t>(p.tiles_w) * p.tiles_h * ((B + best_tb - 1) / best_tb);
  if (m_tiles >= 0x7FFFFFFF) return DIMQ_ERR_TOO_LARGE;
  p.m_tiles = static_cast<int>(m_tiles);
  p.OW = OW;
  p.OH = OH;
  p.Bn = B;
  p.stride = g->stride_h;
  p.pad_h = g->pad_h;
  p.pad_w = g->pad_w;
  p.dil_h = g->dilation_h;
  p.dil_w = g->dilation_w;
  p.KW = g->kernel_w;
  p.c_blocks = g->in_channels / kBK;
  p.M = static_cast<int64_t>(B) * OH * OW;
  p.N = g->out_channels;
  p.passes = passes_for(x_dtype, w);
  p.bn = choose_bn(p.m_tiles, p.N);
  p.n_tiles = static_cast<int>((p.N + p.bn - 1) / p.bn);
  const int64_t K = static_cast<int64_t>(g->kernel_h) * g->kernel_w * g->in_channels;

  const int s = g->stride_h;
  const int64_t C = g->in_channels, W = g->in_w, H = g->in_h;
  const CUtensorMapDataType dt = x_dtype == DIMQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  for (int py = 0; py < s; ++py) {
    for (int px = 0; px < s; ++px) {
      const int64_t Wp = (W - px + s - 1) / s, Hp = (H - py + s - 1) / s;
      const cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(Wp), static_cast<cuuint64_t>(Hp),
                                  static_cast<cuuint64_t>(B)};
      const cuuint64_t strides[3] = {static_cast<cuuint64_t>(s * C * 2), static_cast<cuuint64_t>(s * W * C * 2),
                                     static_cast<cuuint64_t>(H * W * C * 2)};
      const cuuint32_t box[4] = {kBK, static_cast<cuuint32_t>(best_tw), static_cast<cuuint32_t>(best_th),
                                 static_cast<cuuint32_t>(best_tb)};
      const cuuint32_t estr[4] = {1, 1, 1, 1};
      void* base = const_cast<char*>(static_cast<const char*>(x)) + (py * W + px) * C * 2;
      if (encode(&maps.a[py * s + px], dt, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return DIMQ_ERR_DRIVER;
    }
  }
  const int cbw = best_tw < 32 ? best_tw : 32;
  const int cbh = best_th < 32 / cbw ? best_th : 32 / cbw;
  const int cbb = 32 / (cbw * cbh);
  const cuuint64_t odims[4] = {static_cast<cuuint64_t>(g->out_channels), static_cast<cuuint64_t>(OW),
                               static_cast<cuuint64_t>(OH), static_cast<cuuint64_t>(B)};
  const cuuint32_t obox[4] = {32, static_cast<cuuint32_t>(cbw), static_cast<cuuint32_t>(cbh), static_cast<cuuint32_t>(cbb)};
  if (!out_map(encode, &maps.y, y, y_dtype, 4, odims, obox)) return DIMQ_ERR_DRIVER;
  int rc = expand(w, w->packed_khwc, p.N, K, x_dtype == DIMQ_BF16 ? 1 : 0, p.passes, workspace, st);
  if (rc != DIMQ_OK) return rc;
  return launch_dense(maps, p, workspace, K, x_dtype, bias, bias_dtype, residual, y_dtype, epilogue, st);
}

}  // namespace dimq
