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
// Warp roles (448 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM
// allocator, warps 2-5 epilogue, warps 6-13 dequantisation.  Persistent grid:
// one CTA per SM walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...
#include "tc_common.cuh"

namespace dimq {
namespace {

using namespace tc;

constexpr int kTileW = 128;      // weight rows per tile (UMMA M)
constexpr int kTileX = 192;      // activation rows per tile (UMMA N)
constexpr int kBlockK = 64;      // k per stage: 128 bytes of 16-bit elements
constexpr int kXStages = 6;      // shared-memory stages of the activation tile
constexpr int kWStages = 4;      // tensor-memory stages of the dequantised weight tile
constexpr int kAccStages = 2;    // accumulator buffers
constexpr int kTmemCols = 512;
constexpr int kAccCol = 0;                         // accumulators: columns [0, 2*kTileX)
constexpr int kWCol = kAccStages * kTileX;         // weight stages: 32 columns each
static_assert(kWCol + kWStages * (kBlockK / 2) <= kTmemCols, "TMEM layout");
constexpr int kXStageBytes = kTileX * kBlockK * 2;  // 24 KB
constexpr int kNumDequantWarps = 8;
constexpr int kNumEpilogueWarps = 4;
constexpr int kThreads = (2 + kNumEpilogueWarps + kNumDequantWarps) * 32;
constexpr int kMaxTableBytes = 64 * 1024;

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
  int w_fmt;                  // operand format of the dequantised weight: 0 fp16, 1 bf16
  uint32_t idesc;
  int m_tiles, n_tiles;
};

struct SharedHeader {
  uint64_t x_full[kXStages], x_empty[kXStages];
  uint64_t w_full[kWStages], w_empty[kWStages];
  uint64_t d_full[kAccStages], d_empty[kAccStages];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

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

// PAIR: the table holds, per group, 4^BITS words, entry v = {C[v & mask], C[v >> BITS]} as two
// 16-bit operands.  Otherwise it holds 2^BITS 16-bit operands per group.
template <int BITS, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
linear_wq_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // [x stages (1024-aligned)] [header] [tables]
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* x_stage = smem;
  SharedHeader* hdr = reinterpret_cast<SharedHeader*>(smem + kXStages * kXStageBytes);
  uint32_t* table = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(hdr) + 256);
  static_assert(sizeof(SharedHeader) <= 256, "header");

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int num_tiles = p.m_tiles * p.n_tiles;
  const int k_blocks = static_cast<int>(p.K / kBlockK);

  // ---- one-time setup ---------------------------------------------------------
  if (tid == 0) {
    for (int s = 0; s < kXStages; ++s) { mbar_init(smem_u32(&hdr->x_full[s]), 1); mbar_init(smem_u32(&hdr->x_empty[s]), 1); }
    for (int s = 0; s < kWStages; ++s) { mbar_init(smem_u32(&hdr->w_full[s]), kNumDequantWarps * 32); mbar_init(smem_u32(&hdr->w_empty[s]), 1); }
    for (int s = 0; s < kAccStages; ++s) { mbar_init(smem_u32(&hdr->d_full[s]), 1); mbar_init(smem_u32(&hdr->d_empty[s]), kNumEpilogueWarps * 32); }
    hdr->abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&hdr->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  {
    constexpr uint32_t mask = (1u << BITS) - 1u;
    constexpr int per_group = PAIR ? (1 << (2 * BITS)) : (1 << BITS) / 2;  // 32-bit words per group
    const int total = static_cast<int>(p.groups) * per_group;
    for (int i = tid; i < total; i += kThreads) {
      const int g = i / per_group, v = i % per_group;
      uint32_t lo, hi;
      if (PAIR) {
        const int e0 = v & mask, e1 = v >> BITS;
        lo = e0 < p.entries ? to_operand16(load_as_float(p.codebooks, p.cb_dtype, (int64_t)g * p.entries + e0), p.w_fmt) : 0u;
        hi = e1 < p.entries ? to_operand16(load_as_float(p.codebooks, p.cb_dtype, (int64_t)g * p.entries + e1), p.w_fmt) : 0u;
      } else {
        const int e0 = 2 * v, e1 = 2 * v + 1;
        lo = e0 < p.entries ? to_operand16(load_as_float(p.codebooks, p.cb_dtype, (int64_t)g * p.entries + e0), p.w_fmt) : 0u;
        hi = e1 < p.entries ? to_operand16(load_as_float(p.codebooks, p.cb_dtype, (int64_t)g * p.entries + e1), p.w_fmt) : 0u;
      }
      table[i] = lo | (hi << 16);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  volatile uint32_t* abort_flag = &hdr->abort_flag;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = t % p.m_tiles;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&hdr->x_empty[stage]), phase ^ 1u, abort_flag, 0x100u | stage)) { ok = false; break; }
          const uint32_t full = smem_u32(&hdr->x_full[stage]);
          mbar_arrive_expect_tx(full, kXStageBytes);
          tma_load_2d(smem_u32(x_stage + stage * kXStageBytes), &tmap_x, full, kb * kBlockK, m_blk * kTileX);
          ++issued;
          if (++stage == kXStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Gave up: wait (bounded) for the copies still in flight so that no TMA write
        // lands in shared memory after this CTA has exited.
        const uint32_t n_back = issued < (uint32_t)kXStages ? issued : (uint32_t)kXStages;
        uint32_t s = stage, ph = phase;
        for (uint32_t i = 0; i < n_back; ++i) {
          if (s == 0) { s = kXStages - 1; ph ^= 1u; } else { --s; }
          for (uint32_t it = 0; it < kSpinLimit; ++it)
            if (mbar_try_wait(smem_u32(&hdr->x_full[s]), ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      uint32_t xs = 0, xph = 0, ws = 0, wph = 0, as = 0, aph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(smem_u32(&hdr->d_empty[as]), aph ^ 1u, abort_flag, 0x200u | as)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + kAccCol + as * kTileX;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&hdr->x_full[xs]), xph, abort_flag, 0x300u | xs)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&hdr->w_full[ws]), wph, abort_flag, 0x400u | ws)) { ok = false; break; }
          tc_fence_after();
          const uint64_t b_desc = make_smem_desc_sw128(smem_u32(x_stage + xs * kXStageBytes));
          const uint32_t a_tmem = tmem_base + kWCol + ws * (kBlockK / 2);
#pragma unroll
          for (int j = 0; j < kBlockK / 16; ++j) {
            // advance 16 k: 32 bytes inside the swizzled row (encoded >> 4), 8 TMEM columns
            mma_f16_ts(d_tmem, a_tmem + j * 8, b_desc + static_cast<uint64_t>(j * 2), p.idesc,
                       (kb > 0 || j > 0) ? 1u : 0u);
          }
          mma_commit(smem_u32(&hdr->x_empty[xs]));
          mma_commit(smem_u32(&hdr->w_empty[ws]));
          if (++xs == kXStages) { xs = 0; xph ^= 1u; }
          if (++ws == kWStages) { ws = 0; wph ^= 1u; }
        }
        if (!ok) break;
        mma_commit(smem_u32(&hdr->d_full[as]));
        if (++as == kAccStages) { as = 0; aph ^= 1u; }
      }
    }
  } else if (warp < 2 + kNumEpilogueWarps) {
    // ===================== epilogue =====================
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32)
    uint32_t as = 0, aph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m_blk = t % p.m_tiles, n_blk = t / p.m_tiles;
      const int64_t n = static_cast<int64_t>(n_blk) * kTileW + quarter * 32 + lane;
      const int64_t m0 = static_cast<int64_t>(m_blk) * kTileX;
      const bool n_ok = n < p.N;
      const float bias = (p.bias != nullptr && n_ok) ? load_as_float(p.bias, p.bias_dtype, n) : 0.0f;
      // tcgen05.ld is warp-collective: the whole warp proceeds or the whole warp gives up
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->d_full[as]), aph, abort_flag, 0x500u | as))) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kAccCol + as * kTileX;
#pragma unroll 1
      for (int c = 0; c < kTileX / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(d_tmem + c * 32, r);
        tmem_ld_wait();
        if (c == kTileX / 32 - 1) {
          // every column of this buffer is in registers: hand it back to the MMA warp
          tc_fence_before();
          mbar_arrive(smem_u32(&hdr->d_empty[as]));
        }
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int64_t m = m0 + c * 32 + j;
            if (m < p.M) {
              float v = apply_epilogue(__uint_as_float(r[j]) + bias, p.epilogue);
              const int64_t o = m * p.N + n;
              if (p.residual != nullptr) v += load_as_float(p.residual, p.y_dtype, o);
              store_from_float(p.y, p.y_dtype, o, v);
            }
          }
        }
      }
      if (++as == kAccStages) { as = 0; aph ^= 1u; }
    }
  } else {
    // ===================== dequantisation =====================
    const int dw = warp - (2 + kNumEpilogueWarps);  // 0..7
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may write
    const int half = dw >> 2;                       // which 32 of the stage's 64 k
    const int row_in_tile = quarter * 32 + lane;
    const int64_t row_bytes = p.K * BITS / 8;
    constexpr int per_group = PAIR ? (1 << (2 * BITS)) : (1 << BITS) / 2;
    const int64_t total_iters = static_cast<int64_t>((num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * k_blocks;
    auto unit_ptr = [&](int64_t it) -> const uint8_t* {
      const int t = blockIdx.x + static_cast<int>(it / k_blocks) * gridDim.x;
      const int kb = static_cast<int>(it % k_blocks);
      int64_t row = static_cast<int64_t>(t / p.m_tiles) * kTileW + row_in_tile;
      if (row >= p.N) row = p.N - 1;
      return p.packed + row * row_bytes + static_cast<int64_t>(kb) * (8 * BITS) + half * (4 * BITS);
    };
    uint32_t ws = 0, wph = 0;
    uint32_t nxt[BITS];
    if (total_iters > 0) load_unit<BITS>(unit_ptr(0), nxt);
    for (int64_t it = 0; it < total_iters; ++it) {
      uint32_t cur[BITS];
#pragma unroll
      for (int i = 0; i < BITS; ++i) cur[i] = nxt[i];
      if (it + 1 < total_iters) load_unit<BITS>(unit_ptr(it + 1), nxt);
      const int t = blockIdx.x + static_cast<int>(it / k_blocks) * gridDim.x;
      int64_t row = static_cast<int64_t>(t / p.m_tiles) * kTileW + row_in_tile;
      if (row >= p.N) row = p.N - 1;
      const uint32_t* tbl = table + (row / p.group_rows) * per_group;
      uint32_t out[16];
      if (PAIR) {
#pragma unroll
        for (int q = 0; q < 16; ++q) out[q] = tbl[get_field<BITS, 2 * BITS>(cur, q)];
      } else {
        const uint16_t* tbl16 = reinterpret_cast<const uint16_t*>(tbl);
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const uint32_t lo = tbl16[get_field<BITS, BITS>(cur, 2 * q)];
          const uint32_t hi = tbl16[get_field<BITS, BITS>(cur, 2 * q + 1)];
          out[q] = lo | (hi << 16);
        }
      }
      // tcgen05.st is warp-collective: the whole warp proceeds or the whole warp gives up
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&hdr->w_empty[ws]), wph ^ 1u, abort_flag, 0x600u | ws))) break;
      tc_fence_after();
      tmem_st16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kWCol + ws * (kBlockK / 2) + half * 16, out);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&hdr->w_full[ws]));
      if (++ws == kWStages) { ws = 0; wph ^= 1u; }
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

template <int BITS, bool PAIR>
int launch_tc(const CUtensorMap& tmap, const TcParams& p, size_t smem, int grid, cudaStream_t st) {
  auto kern = linear_wq_tc_kernel<BITS, PAIR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  kern<<<grid, kThreads, smem, st>>>(tmap, p);
  return launch_status();
}

size_t table_bytes(int bits, int64_t groups, bool pair) {
  const size_t per_group = pair ? (size_t(1) << (2 * bits)) : (size_t(1) << bits) / 2;
  return groups * per_group * 4;
}

}  // namespace

bool tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K) {
  if (x_dtype != DIMQ_BF16 && x_dtype != DIMQ_F16) return false;
  if (M < 1 || N < 1 || K < kBlockK || K % kBlockK != 0) return false;
  if (!aligned(x, 16) || !aligned(w->packed, 16)) return false;
  if (M > 0x7FFFFFFF / 2 || N > 0x7FFFFFFF / 2) return false;
  if (table_bytes(w->bits, w->groups, false) > (size_t)kMaxTableBytes) return false;
  const int64_t tiles = ((M + kTileX - 1) / kTileX) * ((N + kTileW - 1) / kTileW);
  return tiles < 0x7FFFFFFF;
}

int launch_linear_wq_tc(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                        const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                        int w_fmt, cudaStream_t st) {
  if (!tc_supported(x, x_dtype, w, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  EncodeTiledFn encode = get_encode_tiled();
  if (encode == nullptr) return DIMQ_ERR_DRIVER;
  CUtensorMap tmap;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {kBlockK, kTileX};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(&tmap, x_dtype == DIMQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                            2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return DIMQ_ERR_DRIVER;

  TcParams p;
  p.packed = w->packed;
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
  p.M = M;
  p.N = N;
  p.K = K;
  p.epilogue = epilogue;
  p.w_fmt = w_fmt;
  p.idesc = tc::make_idesc_f16(w_fmt, x_dtype == DIMQ_BF16 ? 1 : 0, kTileW, kTileX);
  p.m_tiles = static_cast<int>((M + kTileX - 1) / kTileX);
  p.n_tiles = static_cast<int>((N + kTileW - 1) / kTileW);
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);

  const bool pair = w->bits != 8 && table_bytes(w->bits, w->groups, true) <= (size_t)kMaxTableBytes;
  const size_t smem = 1024 + static_cast<size_t>(kXStages) * kXStageBytes + 256 + table_bytes(w->bits, w->groups, pair);
  switch (w->bits) {
    case 2: return pair ? launch_tc<2, true>(tmap, p, smem, grid, st) : launch_tc<2, false>(tmap, p, smem, grid, st);
    case 3: return pair ? launch_tc<3, true>(tmap, p, smem, grid, st) : launch_tc<3, false>(tmap, p, smem, grid, st);
    case 4: return pair ? launch_tc<4, true>(tmap, p, smem, grid, st) : launch_tc<4, false>(tmap, p, smem, grid, st);
    case 8: return launch_tc<8, false>(tmap, p, smem, grid, st);
    default: return DIMQ_ERR_BAD_BITS;
  }
}

int read_device_status(uint32_t* status) {
  cudaError_t e = cudaMemcpyFromSymbol(status, tc::g_device_status, sizeof(uint32_t));
  if (e != cudaSuccess) return static_cast<int>(e);
  const uint32_t zero = 0;
  e = cudaMemcpyToSymbol(tc::g_device_status, &zero, sizeof(uint32_t));
  return e == cudaSuccess ? DIMQ_OK : static_cast<int>(e);
}

}  // namespace dimq
