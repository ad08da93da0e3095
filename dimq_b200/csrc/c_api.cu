// Argument validation and kernel selection of the weight-only entry points, plus
// the small utility entry points of the C ABI.
#include "common.cuh"

namespace dimq {
int check_wq_weight(const dimq_wq_weight* w, int64_t out_rows);
int launch_linear_wq_generic(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                             const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                             int epilogue, cudaStream_t st);
int launch_conv2d_direct(bool a4, const void* x, int x_dtype, const dimq_wq_weight* w, float scale, int zp,
                         const void* bias, int bias_dtype, const void* residual, void* y, int y_dtype,
                         const dimq_conv_geom* g, int epilogue, cudaStream_t st);
bool stream_supported(const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K);
int launch_linear_wq_stream(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                            const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                            int epilogue, cudaStream_t st);
bool mma_stream_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K);
int launch_linear_wq_mma_stream(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                int bias_dtype, const void* residual, void* y, int y_dtype, int64_t M, int64_t N,
                                int64_t K, int epilogue, cudaStream_t st);
bool tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K);
int launch_linear_wq_tc(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                        const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                        int precision, cudaStream_t st, void* workspace = nullptr, int64_t workspace_bytes = 0);
int tc_split_k(int64_t M, int64_t N, int64_t K);
bool conv_tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, int y_dtype);
int launch_conv2d_wq_tc(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                        const void* residual, void* y, int y_dtype, const dimq_conv_geom* g, int epilogue,
                        cudaStream_t st);
bool dense_pays(int64_t rows);
bool dense_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const void* y, int y_dtype,
                     const void* residual, int64_t M, int64_t N, int64_t K);
int64_t dense_workspace_bytes(int x_dtype, const dimq_wq_weight* w, int64_t N, int64_t K);
int launch_linear_wq_dense(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                           const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                           void* workspace, int64_t workspace_bytes, cudaStream_t st);
bool conv_dense_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, const void* y,
                          int y_dtype, const void* residual);
int64_t conv_dense_workspace_bytes(int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g);
int launch_conv2d_wq_dense(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                           const void* residual, void* y, int y_dtype, const dimq_conv_geom* g, int epilogue,
                           void* workspace, int64_t workspace_bytes, cudaStream_t st);
bool stem_conv_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, const void* y,
                         int y_dtype, const void* residual);
int64_t stem_conv_workspace_bytes(int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g);
int launch_stem_conv(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                     const void* residual, void* y, int y_dtype, const dimq_conv_geom* g, int epilogue, void* workspace,
                     int64_t workspace_bytes, cudaStream_t st);
int read_device_status(uint32_t* status);
int read_ms_status(uint32_t* status);
bool mma_regs_supported(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K);
bool mma_regs_pays(const dimq_wq_weight* w, int64_t N, int64_t K);
int64_t mma_regs_workspace_bytes(const dimq_wq_weight* w, int64_t M, int64_t N, int64_t K);
int launch_linear_wq_mma_regs(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                              const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                              int epilogue, void* workspace, int64_t workspace_bytes, cudaStream_t st);
int read_rg_status(uint32_t* status);
int launch_linear_prepack(const uint8_t* packed, int bits, int64_t N, int64_t K, uint8_t* out, cudaStream_t st);
int read_dense_status(uint32_t* status);
int launch_bounded_wait_selftest(uint32_t polls, uint32_t* result, cudaStream_t st);
}  // namespace dimq

using namespace dimq;

#ifdef DIMQ_B200_DIAG
namespace dimq { void diag_configure(int dbg, int rep, unsigned long long* prof, int64_t prof_words); }
namespace dimq { void dense_diag_configure(int mode); void stem_diag_prof(unsigned long long* prof); }
extern "C" __attribute__((visibility("default"))) int dimq_diag_stem_prof(void* prof) {
  stem_diag_prof(static_cast<unsigned long long*>(prof));
  return DIMQ_OK;
}
namespace dimq { void set_mma_regs_slices(int ks); void set_mma_regs_trace(uint32_t* trace); }
extern "C" __attribute__((visibility("default"))) int dimq_diag_mma_regs_trace(void* trace) {
  set_mma_regs_trace(static_cast<uint32_t*>(trace));
  return DIMQ_OK;
}
extern "C" __attribute__((visibility("default"))) int dimq_diag_mma_regs_slices(int ks) {
  set_mma_regs_slices(ks);
  return DIMQ_OK;
}
extern "C" __attribute__((visibility("default"))) int dimq_diag_dense(int mode) {
  dense_diag_configure(mode);
  return DIMQ_OK;
}
// Diagnostics build only (not declared in the public header).
extern "C" __attribute__((visibility("default"))) int dimq_diag_configure(int dbg, int rep, void* prof, int64_t prof_words) {
  diag_configure(dbg, rep, static_cast<unsigned long long*>(prof), prof_words);
  return DIMQ_OK;
}
#endif

extern "C" int dimq_version(void) { return 100; }

extern "C" const char* dimq_status_string(int status) {
  switch (status) {
    case DIMQ_OK: return "ok";
    case DIMQ_ERR_NULL_POINTER: return "a required pointer is null";
    case DIMQ_ERR_BAD_SIZE: return "a size or count is out of range";
    case DIMQ_ERR_BAD_DTYPE: return "unsupported element type";
    case DIMQ_ERR_BAD_BITS: return "unsupported index bit width (or more codebook entries than 2^bits)";
    case DIMQ_ERR_BAD_QPARAMS: return "act_scale must be positive and act_zero_point in [0, 15]";
    case DIMQ_ERR_BAD_SHAPE: return "tensor shapes / convolution geometry do not fit together";
    case DIMQ_ERR_UNSUPPORTED: return "the requested algorithm does not support these arguments";
    case DIMQ_ERR_ALIGNMENT: return "a pointer is not aligned as the kernel requires";
    case DIMQ_ERR_DRIVER: return "tensor-map encoding through the CUDA driver failed";
    case DIMQ_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
    case DIMQ_ERR_TOO_LARGE: return "problem too large for this kernel's grid";
    case DIMQ_ERR_SCRATCH_TOO_SMALL: return "scratch too small (the 4 MiB built-in array of dimq_conv2d_wq_static, or the caller's workspace)";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown dimq status";
}

extern "C" int dimq_last_device_status(uint32_t* status) {
  if (status == nullptr) return DIMQ_ERR_NULL_POINTER;
  uint32_t tc = 0, ms = 0, dense = 0, rg = 0;
  int rc = read_device_status(&tc);
  if (rc != DIMQ_OK) return rc;
  rc = read_ms_status(&ms);
  if (rc != DIMQ_OK) return rc;
  rc = read_dense_status(&dense);
  if (rc != DIMQ_OK) return rc;
  rc = read_rg_status(&rg);
  if (rc != DIMQ_OK) return rc;
  *status = tc | ms | dense | rg;
  return DIMQ_OK;
}

extern "C" int dimq_selftest_bounded_wait(uint32_t polls, uint32_t* result, void* stream) {
  if (result == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (polls == 0 || polls > 4096) return DIMQ_ERR_BAD_SIZE;   // at most 4096 polls of <= 20 us each
  return launch_bounded_wait_selftest(polls, result, static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_linear_wq(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                              int bias_dtype, const void* residual, void* y, int y_dtype, int64_t M, int64_t N,
                              int64_t K, int epilogue, int algo, void* stream) {
  if (M < 0 || N <= 0 || K <= 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (epilogue < DIMQ_EPI_NONE || epilogue > DIMQ_EPI_ADD_RELU) return DIMQ_ERR_UNSUPPORTED;
  const int rc = check_wq_weight(w, N);
  if (rc != DIMQ_OK) return rc;
  if (M == 0) return DIMQ_OK;
  if (x == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (algo == DIMQ_ALGO_AUTO) {
    if (mma_regs_supported(x, x_dtype, w, M, N, K) && mma_regs_pays(w, N, K) &&
        mma_regs_workspace_bytes(w, M, N, K) == 0)
      algo = DIMQ_ALGO_MMA_REGS;   // one k slice: no scratch needed
    else if (mma_stream_supported(x, x_dtype, w, M, N, K)) algo = DIMQ_ALGO_MMA_STREAM;
    else if (stream_supported(w, M, N, K)) algo = DIMQ_ALGO_STREAM;
    else if (tc_supported(x, x_dtype, w, M, N, K)) algo = DIMQ_ALGO_TCGEN05;
    else algo = DIMQ_ALGO_GENERIC;
  }
  switch (algo) {
    case DIMQ_ALGO_GENERIC:
      return launch_linear_wq_generic(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, st);
    case DIMQ_ALGO_STREAM:
      return launch_linear_wq_stream(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, st);
    case DIMQ_ALGO_MMA_STREAM:
      return launch_linear_wq_mma_stream(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, st);
    case DIMQ_ALGO_MMA_REGS:
      return launch_linear_wq_mma_regs(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, nullptr,
                                       0, st);   // DIMQ_ERR_SCRATCH_TOO_SMALL where K has several slices
    case DIMQ_ALGO_TCGEN05:
      return launch_linear_wq_tc(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, 0, st);
#ifdef DIMQ_B200_DIAG
    case DIMQ_ALGO_TCGEN05 + 100:  // codewords rounded to the activations' 16-bit format, never split
      return launch_linear_wq_tc(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, 1, st);
#endif
    default:
      return DIMQ_ERR_UNSUPPORTED;
  }
}

extern "C" int dimq_linear_prepack(const uint8_t* packed, int32_t bits, int64_t N, int64_t K, uint8_t* packed_tiled,
                                   void* stream) {
  if (packed == nullptr || packed_tiled == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (N <= 0 || K <= 0) return DIMQ_ERR_BAD_SIZE;
  return launch_linear_prepack(packed, bits, N, K, packed_tiled, static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_linear_wq_regs_workspace_bytes(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M,
                                                   int64_t N, int64_t K, int64_t* bytes) {
  if (bytes == nullptr || w == nullptr) return DIMQ_ERR_NULL_POINTER;
  *bytes = 0;
  const int rc = check_wq_weight(w, N);
  if (rc != DIMQ_OK) return rc;
  if (!mma_regs_supported(x, x_dtype, w, M, N, K)) return DIMQ_ERR_UNSUPPORTED;
  *bytes = mma_regs_workspace_bytes(w, M, N, K);
  return DIMQ_OK;
}

extern "C" int dimq_linear_wq_regs(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                                   const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                                   int epilogue, void* workspace, int64_t workspace_bytes, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (epilogue < DIMQ_EPI_NONE || epilogue > DIMQ_EPI_ADD_RELU) return DIMQ_ERR_UNSUPPORTED;
  const int rc = check_wq_weight(w, N);
  if (rc != DIMQ_OK) return rc;
  if (x == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  return launch_linear_wq_mma_regs(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, workspace,
                                   workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_linear_wq_workspace_bytes(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N,
                                              int64_t K, int64_t* bytes) {
  if (bytes == nullptr || w == nullptr) return DIMQ_ERR_NULL_POINTER;
  *bytes = 0;
  if (M <= 0 || N <= 0 || K <= 0) return DIMQ_OK;
  if (check_wq_weight(w, N) != DIMQ_OK) return DIMQ_OK;
  if (mma_regs_supported(x, x_dtype, w, M, N, K) && mma_regs_pays(w, N, K)) {
    *bytes = mma_regs_workspace_bytes(w, M, N, K);   // the k slices' partial sums (0 with one slice)
    return DIMQ_OK;
  }
  if (mma_stream_supported(x, x_dtype, w, M, N, K) || stream_supported(w, M, N, K)) return DIMQ_OK;
  // many activation rows: the expanded 16-bit weight (the output is taken to be as wide as it may get
  // - 16-bit - and aligned; dimq_linear_wq_ws checks the real one and falls back if it does not fit)
  if (dense_pays(M) && (N * 2) % 16 == 0 && dense_supported(x, x_dtype, w, x, x_dtype, nullptr, M, N, K)) {
    *bytes = dense_workspace_bytes(x_dtype, w, N, K);
    return DIMQ_OK;
  }
  // else only where the automatic choice would take the tcgen05 kernel and splitting K pays
  if (!tc_supported(x, x_dtype, w, M, N, K)) return DIMQ_OK;
  if (tc_split_k(M, N, K) > 1) *bytes = M * N * 4;
  return DIMQ_OK;
}

extern "C" int dimq_linear_wq_ws(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                                 const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                                 int epilogue, void* workspace, int64_t workspace_bytes, void* stream) {
  int64_t need = 0;
  if (w != nullptr && workspace != nullptr && M > 0 && N > 0 && K > 0 && valid_dtype(x_dtype) && valid_dtype(y_dtype) &&
      (bias == nullptr || valid_dtype(bias_dtype)) && epilogue >= DIMQ_EPI_NONE && epilogue <= DIMQ_EPI_ADD_RELU &&
      x != nullptr && y != nullptr &&
      dimq_linear_wq_workspace_bytes(x, x_dtype, w, M, N, K, &need) == DIMQ_OK && need > 0) {
    if (workspace_bytes < need) return DIMQ_ERR_SCRATCH_TOO_SMALL;
    if (mma_regs_supported(x, x_dtype, w, M, N, K) && mma_regs_pays(w, N, K))
      return launch_linear_wq_mma_regs(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, workspace,
                                       workspace_bytes, static_cast<cudaStream_t>(stream));
    if (dense_pays(M)) {
      if (dense_supported(x, x_dtype, w, y, y_dtype, residual, M, N, K))
        return launch_linear_wq_dense(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue,
                                      workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
    } else {
      return launch_linear_wq_tc(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, 0,
                                 static_cast<cudaStream_t>(stream), workspace, workspace_bytes);
    }
  }
  return dimq_linear_wq(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, DIMQ_ALGO_AUTO, stream);
}

extern "C" int dimq_conv2d_wq(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                              int bias_dtype, const void* residual, void* y, int y_dtype,
                              const dimq_conv_geom* geom, int epilogue, int algo, void* stream) {
  if (geom == nullptr) return DIMQ_ERR_NULL_POINTER;
  dimq_conv_geom g = *geom;
  int rc = dimq_conv_out_size(&g);
  if (rc != DIMQ_OK) return rc;
  if (g.out_h != geom->out_h || g.out_w != geom->out_w) return DIMQ_ERR_BAD_SHAPE;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (epilogue < DIMQ_EPI_NONE || epilogue > DIMQ_EPI_ADD_RELU) return DIMQ_ERR_UNSUPPORTED;
  rc = check_wq_weight(w, g.out_channels);
  if (rc != DIMQ_OK) return rc;
  if (static_cast<int64_t>(g.batch) * g.out_channels * g.out_h * g.out_w == 0) return DIMQ_OK;
  if (x == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (algo == DIMQ_ALGO_AUTO) algo = conv_tc_supported(x, x_dtype, w, &g, y_dtype) ? DIMQ_ALGO_TCGEN05 : DIMQ_ALGO_GENERIC;
  if (algo == DIMQ_ALGO_TCGEN05)
    return launch_conv2d_wq_tc(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, &g, epilogue, st);
  if (algo != DIMQ_ALGO_GENERIC) return DIMQ_ERR_UNSUPPORTED;
  return launch_conv2d_direct(false, x, x_dtype, w, 1.0f, 0, bias, bias_dtype, residual, y, y_dtype, &g, epilogue,
                              static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_expand_workspace_bytes(int x_dtype, const dimq_wq_weight* w, int64_t rows, int64_t row_len,
                                           int64_t* bytes) {
  if (bytes == nullptr || w == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (rows < 0 || row_len < 0) return DIMQ_ERR_BAD_SIZE;
  *bytes = dense_workspace_bytes(x_dtype, w, rows, row_len);
  return DIMQ_OK;
}

extern "C" int dimq_linear_wq_expand(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                     int bias_dtype, const void* residual, void* y, int y_dtype, int64_t M, int64_t N,
                                     int64_t K, int epilogue, void* workspace, int64_t workspace_bytes, void* stream) {
  if (M < 0 || N <= 0 || K <= 0) return DIMQ_ERR_BAD_SIZE;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (epilogue < DIMQ_EPI_NONE || epilogue > DIMQ_EPI_ADD_RELU) return DIMQ_ERR_UNSUPPORTED;
  const int rc = check_wq_weight(w, N);
  if (rc != DIMQ_OK) return rc;
  if (M == 0) return DIMQ_OK;
  if (x == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  return launch_linear_wq_dense(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, M, N, K, epilogue, workspace,
                                workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_conv2d_wq_workspace_bytes(const void* x, int x_dtype, const dimq_wq_weight* w,
                                              const dimq_conv_geom* geom, int64_t* bytes) {
  if (bytes == nullptr || w == nullptr || geom == nullptr) return DIMQ_ERR_NULL_POINTER;
  *bytes = 0;
  dimq_conv_geom g = *geom;
  if (dimq_conv_out_size(&g) != DIMQ_OK || check_wq_weight(w, g.out_channels) != DIMQ_OK) return DIMQ_OK;
  if (!dense_pays(static_cast<int64_t>(g.batch) * g.out_h * g.out_w)) return DIMQ_OK;
  if ((static_cast<int64_t>(g.out_channels) * 2) % 16 != 0) return DIMQ_OK;
  if (stem_conv_supported(x, x_dtype, w, &g, x, x_dtype, nullptr)) *bytes = stem_conv_workspace_bytes(x_dtype, w, &g);
  else if (conv_dense_supported(x, x_dtype, w, &g, x, x_dtype, nullptr)) *bytes = conv_dense_workspace_bytes(x_dtype, w, &g);
  return DIMQ_OK;
}

static int conv_wq_checks(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                          void* y, int y_dtype, const dimq_conv_geom* geom, int epilogue, dimq_conv_geom* g, bool* empty) {
  if (geom == nullptr) return DIMQ_ERR_NULL_POINTER;
  *g = *geom;
  int rc = dimq_conv_out_size(g);
  if (rc != DIMQ_OK) return rc;
  if (g->out_h != geom->out_h || g->out_w != geom->out_w) return DIMQ_ERR_BAD_SHAPE;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (epilogue < DIMQ_EPI_NONE || epilogue > DIMQ_EPI_ADD_RELU) return DIMQ_ERR_UNSUPPORTED;
  rc = check_wq_weight(w, g->out_channels);
  if (rc != DIMQ_OK) return rc;
  *empty = static_cast<int64_t>(g->batch) * g->out_channels * g->out_h * g->out_w == 0;
  if (!*empty && (x == nullptr || y == nullptr)) return DIMQ_ERR_NULL_POINTER;
  return DIMQ_OK;
}

extern "C" int dimq_conv2d_wq_expand(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                     int bias_dtype, const void* residual, void* y, int y_dtype,
                                     const dimq_conv_geom* geom, int epilogue, void* workspace, int64_t workspace_bytes,
                                     void* stream) {
  dimq_conv_geom g;
  bool empty = false;
  const int rc = conv_wq_checks(x, x_dtype, w, bias, bias_dtype, y, y_dtype, geom, epilogue, &g, &empty);
  if (rc != DIMQ_OK) return rc;
  if (empty) return DIMQ_OK;
  if (stem_conv_supported(x, x_dtype, w, &g, y, y_dtype, residual))
    return launch_stem_conv(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, &g, epilogue, workspace,
                            workspace_bytes, static_cast<cudaStream_t>(stream));
  return launch_conv2d_wq_dense(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, &g, epilogue, workspace,
                                workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int dimq_conv2d_wq_ws(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                                 const void* residual, void* y, int y_dtype, const dimq_conv_geom* geom, int epilogue,
                                 void* workspace, int64_t workspace_bytes, void* stream) {
  dimq_conv_geom g;
  bool empty = false;
  const int rc = conv_wq_checks(x, x_dtype, w, bias, bias_dtype, y, y_dtype, geom, epilogue, &g, &empty);
  if (rc != DIMQ_OK) return rc;
  if (empty) return DIMQ_OK;
  int64_t need = 0;
  if (workspace != nullptr && dimq_conv2d_wq_workspace_bytes(x, x_dtype, w, geom, &need) == DIMQ_OK && need > 0 &&
      stem_conv_supported(x, x_dtype, w, &g, y, y_dtype, residual)) {
    if (workspace_bytes < need) return DIMQ_ERR_SCRATCH_TOO_SMALL;
    return launch_stem_conv(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, &g, epilogue, workspace,
                            workspace_bytes, static_cast<cudaStream_t>(stream));
  }
  if (workspace != nullptr && need > 0 && conv_dense_supported(x, x_dtype, w, &g, y, y_dtype, residual)) {
    if (workspace_bytes < need) return DIMQ_ERR_SCRATCH_TOO_SMALL;
    return launch_conv2d_wq_dense(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, &g, epilogue, workspace,
                                  workspace_bytes, static_cast<cudaStream_t>(stream));
  }
  return dimq_conv2d_wq(x, x_dtype, w, bias, bias_dtype, residual, y, y_dtype, geom, epilogue, DIMQ_ALGO_AUTO, stream);
}
