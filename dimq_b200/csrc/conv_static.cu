// dimq_conv2d_wq_static: the tensor-core LUT convolution for callers that may not allocate.
//
// The implicit-GEMM convolution reads the weight indices in [OC][KH][KW][ICg] order, a re-ordered
// copy of the packed stream that dimq_conv2d_wq expects its caller to allocate (dimq_conv_prepack).
// Some integrations cannot do that: a plug-in inside a serving runtime that has handed the whole
// device to its own memory pool, a process running under a fixed device-memory budget, or a caller
// that only holds the tensors it was given and has no allocator to ask.  For them this entry point
// keeps the re-ordered indices in a fixed array that is part of the library image itself.
//
// Consequences of that choice, all visible to the caller:
//   * the array is 4 MiB and every GPU on which the library is used carries it until the process
//     exits; a weight whose index stream is larger is rejected (DIMQ_ERR_SCRATCH_TOO_SMALL);
//   * there is ONE array per GPU, shared by every call: a call overwrites what the previous call left
//     there (it rewrites every byte it later reads, so nothing needs clearing), and two calls whose
//     kernels can overlap on the GPU — different streams, or threads racing on one device — corrupt
//     each other.  Issue the calls of one device on one stream, or serialise them yourself;
//   * the first call on a device looks the array's device address up once (with that device
//     current).  Make that first call outside any stream capture.
// No cudaMalloc / cudaFree or allocating library routine is called here.
#include <mutex>

#include "common.cuh"

namespace dimq {
namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_conv_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_ptr[kMaxDevices] = {};  // device address of g_conv_scratch, per device

// The name g_conv_scratch is a host-side handle in host code, not a device address: the address
// kernels can use comes from cudaGetSymbolAddress, asked once per device while it is current.
int scratch_address(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return DIMQ_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_conv_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (ptr == nullptr) return DIMQ_ERR_DRIVER;
    g_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = g_scratch_ptr[dev];
  return DIMQ_OK;
}

}  // namespace

bool conv_tc_supported(const void* x, int x_dtype, const dimq_wq_weight* w, const dimq_conv_geom* g, int y_dtype);
int check_wq_weight(const dimq_wq_weight* w, int64_t out_rows);

}  // namespace dimq

using namespace dimq;

extern "C" int dimq_conv2d_wq_static(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                     int bias_dtype, const void* residual, void* y, int y_dtype,
                                     const dimq_conv_geom* geom, int epilogue, void* stream) {
  if (w == nullptr || geom == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (w->packed == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (!(w->bits == 2 || w->bits == 3 || w->bits == 4 || w->bits == 8)) return DIMQ_ERR_BAD_BITS;
  dimq_conv_geom g = *geom;
  int rc = dimq_conv_out_size(&g);
  if (rc != DIMQ_OK) return rc;
  if (g.out_h != geom->out_h || g.out_w != geom->out_w) return DIMQ_ERR_BAD_SHAPE;
  // every argument check dimq_conv2d_wq would make comes first, so that a negative return code means
  // that nothing was launched and the shared array was not touched
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return DIMQ_ERR_BAD_DTYPE;
  if (epilogue < DIMQ_EPI_NONE || epilogue > DIMQ_EPI_ADD_RELU) return DIMQ_ERR_UNSUPPORTED;
  rc = check_wq_weight(w, g.out_channels);
  if (rc != DIMQ_OK) return rc;
  const int64_t numel = static_cast<int64_t>(g.out_channels) * g.in_channels_per_group * g.kernel_h * g.kernel_w;
  const int64_t bytes = (numel * w->bits + 7) / 8;
  if (bytes > static_cast<int64_t>(kStaticScratchBytes)) return DIMQ_ERR_SCRATCH_TOO_SMALL;
  if (static_cast<int64_t>(g.batch) * g.out_channels * g.out_h * g.out_w == 0) return DIMQ_OK;

  unsigned char* scratch = nullptr;
  rc = scratch_address(&scratch);
  if (rc != DIMQ_OK) return rc;

  dimq_wq_weight ws = *w;
  ws.packed_khwc = scratch;
  // this entry point exists for the kernel that needs the re-ordered indices; other geometries need
  // no scratch at all and belong to dimq_conv2d_wq
  if (x == nullptr || y == nullptr) return DIMQ_ERR_NULL_POINTER;
  if (!conv_tc_supported(x, x_dtype, &ws, &g, y_dtype)) return DIMQ_ERR_UNSUPPORTED;
  rc = dimq_conv_prepack(w->packed, w->bits, g.out_channels, g.in_channels_per_group, g.kernel_h, g.kernel_w,
                         scratch, stream);
  if (rc != DIMQ_OK) return rc;
  return dimq_conv2d_wq(x, x_dtype, &ws, bias, bias_dtype, residual, y, y_dtype, &g, epilogue, DIMQ_ALGO_TCGEN05,
                        stream);
}
