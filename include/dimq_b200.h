/*
 * dimq_b200 — C ABI of the B200 (sm_100a) backend for DIMQ packed-index inference.
 *
 * Every entry point takes raw device pointers, explicit sizes and a CUDA stream
 * (a cudaStream_t passed as void*; NULL is the legacy default stream).  Nothing
 * here allocates device memory, synchronises the stream or takes ownership of a
 * buffer: the caller provides inputs, outputs and (where stated) scratch.
 * Launches go to the device that is current on the calling thread.
 *
 * Return value: 0 on success; a negative DIMQ_ERR_* code for a rejected
 * argument (nothing was launched); a positive value is a cudaError_t reported by
 * the launch.  dimq_status_string() turns either into text.
 *
 * "Replaces" names the function of the DIMQ reference (paths inside that
 * project) whose role the entry point takes over.
 */
#ifndef DIMQ_B200_H_
#define DIMQ_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DIMQ_API __attribute__((visibility("default")))
#else
#define DIMQ_API
#endif

#define DIMQ_OK 0
#define DIMQ_ERR_NULL_POINTER (-1)
#define DIMQ_ERR_BAD_SIZE (-2)
#define DIMQ_ERR_BAD_DTYPE (-3)
#define DIMQ_ERR_BAD_BITS (-4)
#define DIMQ_ERR_BAD_QPARAMS (-5)   /* act_scale <= 0 or act_zp outside [0, 15] */
#define DIMQ_ERR_BAD_SHAPE (-6)     /* channel / group / kernel geometry does not fit */
#define DIMQ_ERR_UNSUPPORTED (-7)   /* the requested algorithm cannot take these arguments */
#define DIMQ_ERR_ALIGNMENT (-8)
#define DIMQ_ERR_DRIVER (-9)        /* a driver entry point (tensor-map encode) is unavailable or failed */
#define DIMQ_ERR_DEVICE_TIMEOUT (-10) /* a bounded wait inside a kernel expired (see dimq_last_device_status) */
#define DIMQ_ERR_TOO_LARGE (-11)
#define DIMQ_ERR_SCRATCH_TOO_SMALL (-12) /* built-in scratch of dimq_conv2d_wq_static or a caller workspace is too small */

/* element types of floating tensors */
#define DIMQ_F32 0
#define DIMQ_F16 1
#define DIMQ_BF16 2

/* kernel selection for the weight-only ops */
#define DIMQ_ALGO_AUTO 0
#define DIMQ_ALGO_GENERIC 1   /* exact fp32 SIMT kernel, any shape */
#define DIMQ_ALGO_STREAM 2    /* small-M index-streaming kernel, fp32 arithmetic (any activation type, M <= 8) */
#define DIMQ_ALGO_TCGEN05 3   /* TMA + in-pipeline dequantisation + tcgen05 MMA (tensor-core regime) */
#define DIMQ_ALGO_MMA_STREAM 4 /* small-M index-streaming kernel for 16-bit activations (M <= 32): pair-table
                                  lookups feeding warp-level MMAs; the HBM-bound regime */
#define DIMQ_ALGO_MMA_REGS 6  /* small-M kernel for weights of 2 MB of indices and more (M <= 16, K a multiple of
                                  128, at least 2048): activations and indices in registers.  Through
                                  dimq_linear_wq only with K = 2048 (one k slice); longer K needs scratch:
                                  dimq_linear_wq_ws / _regs */

/* fused epilogues of the weight-only ops */
#define DIMQ_EPI_NONE 0
#define DIMQ_EPI_RELU 1
#define DIMQ_EPI_GELU 2       /* exact (erf) GELU */
#define DIMQ_EPI_ADD_RELU 3   /* relu(acc + bias + residual): the residual is added before the ReLU */

DIMQ_API int dimq_version(void);
DIMQ_API const char* dimq_status_string(int status);

/* ---- index bit-packing ------------------------------------------------- */

/* packed[j] = idx[2j] & 15 | (idx[2j+1] & 15) << 4; an odd tail leaves the high
 * nibble zero.  `packed` holds (numel + 1) / 2 bytes.
 * Replaces pack_u4_cuda, dimq_cuda_backend/csrc/dimq_pack.cu:52-67. */
DIMQ_API int dimq_pack_u4(const uint8_t* indices, int64_t numel, uint8_t* packed, void* stream);

/* indices[i] = nibble i of `packed` (even i -> low nibble).
 * Replaces unpack_u4_cuda, dimq_cuda_backend/csrc/dimq_pack.cu:69-85. */
DIMQ_API int dimq_unpack_u4(const uint8_t* packed, int64_t numel, uint8_t* indices, void* stream);

/* bits in {1, 2, 3, 4, 8}: index j occupies bits [j*bits, (j+1)*bits) of a
 * little-endian bit stream of (numel*bits + 7) / 8 bytes, tail bits zero.
 * bits == 4 is dimq_pack_u4.  Generalises dimq_pack.cu:11-35 (the reference is
 * 4-bit only). */
DIMQ_API int dimq_pack_bits(const uint8_t* indices, int64_t numel, int bits, uint8_t* packed, void* stream);
DIMQ_API int dimq_unpack_bits(const uint8_t* packed, int64_t numel, int bits, uint8_t* indices, void* stream);

/* ---- W4A4 pieces --------------------------------------------------------- */

/* out[i] = clamp(rint(float(x[i]) / act_scale) + act_zp, 0, 15), IEEE divide,
 * round-half-even.  Replaces quantize_activation_u4_cuda, dimq_pack.cu:87-109. */
DIMQ_API int dimq_quantize_activation_u4(const void* x, int x_dtype, int64_t numel, float act_scale, int act_zp,
                                uint8_t* out, void* stream);

/* table[g][w][a] = float(codebook[g][w]) * (act_scale * float(a - act_zp)), fp32,
 * a in [0, 16).  groups == 1, entries == 16 is the reference op.
 * Replaces build_product_table_cuda, dimq_cuda_backend/csrc/dimq_product_table.cu:29-46. */
DIMQ_API int dimq_build_product_table(const void* codebook, int cb_dtype, int64_t groups, int entries,
                             float act_scale, int act_zp, float* table, void* stream);

/* y[m][n] = sum_k P[widx(n,k)][q(x[m][k])] + bias[n], fp32 out; the product
 * table is built inside the kernel (no temporary).  x is [M, K] row-major,
 * packed_w the u4 stream of the [N, K] index matrix (rows not padded), codebook
 * has 16 entries.  bias may be NULL.
 * Replaces linear_lut_cuda, dimq_cuda_backend/csrc/dimq_gemm_lut.cu:58-117. */
DIMQ_API int dimq_linear_lut(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook, int cb_dtype,
                    float act_scale, int act_zp, const void* bias, int bias_dtype, float* y, int64_t M,
                    int64_t N, int64_t K, void* stream);

/* Geometry of a 2-D convolution.  Strides are in ELEMENTS and describe where
 * element (b, c, h, w) of the logical NCHW tensor lives, so both contiguous
 * NCHW and channels_last (NHWC) storage are addressed without a copy. */
typedef struct dimq_conv_geom {
  int32_t batch, in_channels, in_h, in_w;
  int32_t out_channels, in_channels_per_group, kernel_h, kernel_w;
  int32_t stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w, groups;
  int32_t out_h, out_w;               /* filled by dimq_conv_out_size */
  int64_t x_stride[4];                /* b, c, h, w */
  int64_t y_stride[4];                /* b, oc, oh, ow */
} dimq_conv_geom;

/* out = (in + 2*pad - dilation*(kernel-1) - 1) / stride + 1 for both axes
 * (dimq_cuda_backend/csrc/dimq_conv2d_lut.cu:129-130).  Validates the geometry. */
DIMQ_API int dimq_conv_out_size(dimq_conv_geom* geom);

/* Direct W4A4 convolution over the product table, taps outside the image skipped.
 * Replaces conv2d_lut_cuda, dimq_cuda_backend/csrc/dimq_conv2d_lut.cu:90-186. */
DIMQ_API int dimq_conv2d_lut(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook, int cb_dtype,
                    float act_scale, int act_zp, const void* bias, int bias_dtype, float* y,
                    const dimq_conv_geom* geom, void* stream);

/* ---- export: nearest-codeword assignment (+ packing) -------------------- */

/* idx = argmin_k (float(w) - codebook[g][k])^2 in fp32, first minimum wins, a
 * NaN distance beats every number; row r of the [rows, cols] weight uses
 * codebook g = r / group_rows.  Writes unpacked uint8 indices (may be NULL)
 * and/or the `bits`-wide packed stream of the flattened index matrix (may be
 * NULL; entries <= 2^bits required).
 * Replaces hard_quantize_weight, quant/dimq.py:197-221, and
 * assign_weight_indices + pack_u4_indices, dimq_backend/export.py:24-55. */
DIMQ_API int dimq_hard_quantize(const void* w, int w_dtype, int64_t rows, int64_t cols, const float* codebooks,
                       int entries, int64_t group_rows, uint8_t* indices, uint8_t* packed, int bits,
                       void* stream);

/* Straight-through fake quantisation of the QAT forward: out = w + (codebook[g][idx].to(w's type) - w),
 * every operation rounded to the weight's element type as PyTorch evaluates it, idx as in
 * dimq_hard_quantize; `out` has w's element type, `indices` (uint8, may be NULL) receives idx.  One
 * pass over w instead of argmin + gather + two elementwise kernels.  Its gradient is the identity on w
 * and none on the codebook, so the host side needs no backward kernel.
 * Replaces the forward of fake_quant_weight in "hard_ste" mode, quant/dimq_wrapper.py:72-75, which
 * calls hard_quantize_weight (quant/dimq.py:197-221) on every step. */
DIMQ_API int dimq_fake_quantize_ste(const void* w, int w_dtype, int64_t rows, int64_t cols, const float* codebooks,
                                    int entries, int64_t group_rows, void* out, uint8_t* indices, void* stream);

/* ---- weight-only LUT GEMM / conv ---------------------------------------- */

typedef struct dimq_wq_weight {
  const uint8_t* packed;     /* `bits`-wide stream of the [N, K] (or [OC, ICg, KH, KW]) index tensor */
  int32_t bits;              /* 2, 3, 4 or 8 */
  const void* codebooks;     /* [groups, entries] */
  int32_t cb_dtype;          /* DIMQ_F32 / DIMQ_F16 / DIMQ_BF16 */
  int32_t entries;           /* <= 2^bits */
  int64_t groups;
  int64_t group_rows;        /* output rows (channels) per codebook */
  const uint8_t* packed_khwc; /* optional second copy of the indices in the order a fast kernel reads them.
                                Convolutions: [OC][KH][KW][ICg], written by dimq_conv_prepack; enables the
                                tensor-core conv.  Linear layers: tiles of 16 rows x 128 k, written by
                                dimq_linear_prepack; read by the register-resident small-M kernel only (its index
                                loads become contiguous), every other kernel reads `packed` */
} dimq_wq_weight;

/* y[m][n] = sum_k x[m][k] * codebooks[n / group_rows][idx(n, k)] + bias[n], then
 * the epilogue, then + residual[m][n] (may be NULL).  fp32 accumulation.  The
 * reference computes this as dequantize_packed_weight + F.linear
 * (dimq_backend/reference.py:47-56, quant/dimq_wrapper.py:237-240). */
DIMQ_API int dimq_linear_wq(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                   const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K, int epilogue,
                   int algo, void* stream);

/* Weight-only convolution; same contract as dimq_conv2d_lut without the
 * activation quantiser (dimq_backend/reference.py:113-144 with x left in float,
 * quant/dimq_wrapper.py:189-197).  y has y_dtype elements at geom->y_stride. */
DIMQ_API int dimq_conv2d_wq(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                   const void* residual, void* y, int y_dtype, const dimq_conv_geom* geom, int epilogue,
                   int algo, void* stream);

/* Re-orders the `bits`-wide index stream of a [OC][ICg][KH][KW] convolution weight (the reference's
 * "conv_kcrs" layout, dimq_backend/export.py:232) to [OC][KH][KW][ICg], so that 64 consecutive
 * indices of a row are 64 input channels of one filter tap — the k order of the implicit-GEMM
 * convolution over NHWC activations.  `dst` holds (OC*ICg*KH*KW*bits + 7) / 8 bytes and is scratch
 * the caller owns (typically built once per layer and cached).  No counterpart in the reference
 * (its direct convolution reads the kcrs stream in place). */
DIMQ_API int dimq_conv_prepack(const uint8_t* packed_kcrs, int bits, int64_t out_channels, int64_t in_channels_per_group,
                               int64_t kernel_h, int64_t kernel_w, uint8_t* packed_khwc, void* stream);

/* The tensor-core path of dimq_conv2d_wq for callers that cannot allocate device memory (a plug-in
 * inside a runtime that owns the whole device pool, a process under a fixed memory budget): it takes
 * the canonical packed stream (w->packed; w->packed_khwc is ignored) and keeps the re-ordered indices
 * in a 4 MiB array built into the library, so nothing is allocated by either side.  Limits: the index
 * stream (OC*ICg*KH*KW*bits/8 bytes) must fit 4 MiB (else DIMQ_ERR_SCRATCH_TOO_SMALL); the geometry
 * must be one the tensor-core convolution takes (else DIMQ_ERR_UNSUPPORTED: use dimq_conv2d_wq, which
 * then needs no scratch); the array is shared by all calls on a GPU, so calls that may overlap on the
 * device race — keep them on one stream.  The first call on a device resolves the array's address;
 * make it before any stream capture.  Every GPU the library runs on holds the 4 MiB until exit.
 * This entry point has no counterpart in the reference. */
DIMQ_API int dimq_conv2d_wq_static(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                   int bias_dtype, const void* residual, void* y, int y_dtype,
                                   const dimq_conv_geom* geom, int epilogue, void* stream);

/* dimq_linear_wq with caller-owned scratch memory, which three regimes use:
 *  - a few activation rows (M <= 16, 16-bit x) against 2 MB of 2- to 4-bit indices or more, N a multiple
 *    of 16 and K of 128, K >= 2048: the register-resident small-M kernel cuts K into slices of 2048 worked on by
 *    different CTAs, each writes its partial sums to the workspace (slices * M * N * 4 bytes, at most 8
 *    slices at a time) and a second small kernel adds them in a fixed order and applies bias / epilogue /
 *    residual: no atomics, the same bits every run.
 *  - many activation rows (M >= 1024, 16-bit x, K a multiple of 64, 16-byte aligned y rows): the
 *    indices are expanded ONCE per call into a 16-bit weight matrix in the workspace (N*K*2 bytes; twice
 *    that when bf16 activations meet a codebook that is not stored in bf16 and every codeword is carried
 *    as a hi + lo pair) and a dense TMA + tcgen05 GEMM runs over it.  Looking the indices up inside the
 *    GEMM pipeline instead repeats the N*K lookups once per 192 activation rows.
 *  - a few hundred activation rows against a long K, whose tiles would occupy only a few SMs: the
 *    in-pipeline tcgen05 kernel cuts K into slices (split-K), adds the partial sums into the workspace
 *    (M*N*4 bytes, float atomics: the last bits can differ from run to run) and a second small kernel
 *    applies bias / epilogue / residual.
 * dimq_linear_wq_workspace_bytes reports the bytes of the regime that applies and 0 otherwise (then
 * dimq_linear_wq_ws is dimq_linear_wq with DIMQ_ALGO_AUTO and the workspace is not touched).  The
 * workspace must be 16-byte aligned; its contents after the call are unspecified.  The reference has no
 * counterpart: it dequantises the whole weight per call (dimq_backend/reference.py:47-56) or reads
 * nibbles in its innermost loop (csrc/dimq_gemm_lut.cu:45-49). */
DIMQ_API int dimq_linear_wq_workspace_bytes(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M, int64_t N,
                                            int64_t K, int64_t* bytes);
DIMQ_API int dimq_linear_wq_ws(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                               const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                               int epilogue, void* workspace, int64_t workspace_bytes, void* stream);

/* The same for dimq_conv2d_wq: with w->packed_khwc, channels_last 16-bit x and y, groups 1, input
 * channels a multiple of 64, stride 1 or 2 and at least 1024 output pixels, the re-ordered indices are
 * expanded once into the workspace (OC*KH*KW*IC*2 bytes, doubled for hi + lo pairs as above) and the
 * dense implicit-GEMM kernel runs; otherwise dimq_conv2d_wq_workspace_bytes reports 0 and
 * dimq_conv2d_wq_ws is dimq_conv2d_wq with DIMQ_ALGO_AUTO. */
DIMQ_API int dimq_conv2d_wq_workspace_bytes(const void* x, int x_dtype, const dimq_wq_weight* w,
                                            const dimq_conv_geom* geom, int64_t* bytes);
DIMQ_API int dimq_conv2d_wq_ws(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                               const void* residual, void* y, int y_dtype, const dimq_conv_geom* geom, int epilogue,
                               void* workspace, int64_t workspace_bytes, void* stream);

/* The expand-then-GEMM form requested explicitly, at any M (DIMQ_ERR_UNSUPPORTED where it cannot run:
 * see the conditions above, without the row threshold).  dimq_expand_workspace_bytes gives the scratch
 * size for `rows` weight rows of `row_len` indices each (linear: N rows of K; convolution: OC rows of
 * KH*KW*IC).  No counterpart in the reference. */
DIMQ_API int dimq_expand_workspace_bytes(int x_dtype, const dimq_wq_weight* w, int64_t rows, int64_t row_len,
                                         int64_t* bytes);
DIMQ_API int dimq_linear_wq_expand(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                   int bias_dtype, const void* residual, void* y, int y_dtype, int64_t M, int64_t N,
                                   int64_t K, int epilogue, void* workspace, int64_t workspace_bytes, void* stream);
DIMQ_API int dimq_conv2d_wq_expand(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias,
                                   int bias_dtype, const void* residual, void* y, int y_dtype,
                                   const dimq_conv_geom* geom, int epilogue, void* workspace, int64_t workspace_bytes,
                                   void* stream);

/* The register-resident small-M kernel requested explicitly, whatever the size of the weight
 * (DIMQ_ERR_UNSUPPORTED outside M <= 16, 16-bit x, 2- to 4-bit indices, N % 16 == 0, K % 128 == 0, K >= 2048).
 * dimq_linear_wq_regs_workspace_bytes gives the scratch it needs (0 when K = 2048).  Replaces the
 * reference's per-call dequantisation (dimq_backend/reference.py:47-56) in the decode regime. */
/* packed_tiled = the [N, K] index stream re-ordered into tiles of 16 rows x 128 k ([row block][128-k range][row]
 * [16 * bits bytes]); same size as the input.  2-, 3- or 4-bit, N a multiple of 16, K of 128; once per layer. */
DIMQ_API int dimq_linear_prepack(const uint8_t* packed, int32_t bits, int64_t N, int64_t K, uint8_t* packed_tiled,
                                 void* stream);
DIMQ_API int dimq_linear_wq_regs_workspace_bytes(const void* x, int x_dtype, const dimq_wq_weight* w, int64_t M,
                                                 int64_t N, int64_t K, int64_t* bytes);
DIMQ_API int dimq_linear_wq_regs(const void* x, int x_dtype, const dimq_wq_weight* w, const void* bias, int bias_dtype,
                                 const void* residual, void* y, int y_dtype, int64_t M, int64_t N, int64_t K,
                                 int epilogue, void* workspace, int64_t workspace_bytes, void* stream);

/* ---- W4A4 product-table ops on the tensor cores ------------------------- */

/* Same operation as dimq_linear_lut / dimq_conv2d_lut (csrc/dimq_gemm_lut.cu:58-117,
 * csrc/dimq_conv2d_lut.cu:90-186), computed as sum_k (s*C[w_idx]) * (a_idx - z) on the tcgen05
 * weight-only kernel: the activation codes are the reference's exactly, the scaled codewords go in as
 * a hi + lo pair of bf16 values (about 2^-17 relative), accumulation is fp32.  The result is in the
 * tolerance class of the weight-only ops (max-abs 1e-2, relative L2 1e-3), not bit-equal to the table
 * lookup; dimq_linear_lut / dimq_conv2d_lut stay the exact path.
 *
 * `workspace` is caller-owned device memory, 256-byte aligned, of at least
 * dimq_a4_workspace_bytes(x_numel, conv_weight_numel) bytes (conv_weight_numel = 0 for the linear op);
 * it holds the centred activation codes (bf16), the 16 scaled codewords and, for the convolution,
 * the indices re-ordered to [OC][KH][KW][ICg].  DIMQ_ERR_SCRATCH_TOO_SMALL if it is smaller,
 * DIMQ_ERR_UNSUPPORTED where the tensor-core kernel does not apply (linear: K a multiple of 64;
 * convolution: channels_last x and y, groups 1, in_channels a multiple of 64, stride 1 or 2). */
DIMQ_API int dimq_a4_workspace_bytes(int64_t x_numel, int64_t conv_weight_numel, int64_t* bytes);

/* The first half of the two calls above on its own: codes[i] = bf16(clamp(rint(x[i] / act_scale) + act_zp,
 * 0, 15) - act_zp), the reference's activation quantiser (csrc/dimq_pack.cu:37-48, dimq_common.cuh:17-21)
 * with the zero point already subtracted; an integer in [-15, 15], exact in bf16, element order of x kept.
 * A caller that keeps per-layer state (the scaled codebook act_scale * C, the re-ordered indices) feeds
 * these codes to dimq_linear_wq_ws / dimq_conv2d_wq_ws and gets the W4A4 result without the per-call
 * index re-order of dimq_conv2d_lut_tc. */
DIMQ_API int dimq_centre_quantize_u4(const void* x, int x_dtype, int64_t numel, float act_scale, int act_zp,
                                     void* codes_bf16, void* stream);
DIMQ_API int dimq_linear_lut_tc(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook,
                                int cb_dtype, float act_scale, int act_zp, const void* bias, int bias_dtype,
                                float* y, int64_t M, int64_t N, int64_t K, void* workspace,
                                int64_t workspace_bytes, void* stream);
DIMQ_API int dimq_conv2d_lut_tc(const void* x, int x_dtype, const uint8_t* packed_w, const void* codebook,
                                int cb_dtype, float act_scale, int act_zp, const void* bias, int bias_dtype,
                                float* y, const dimq_conv_geom* geom, void* workspace, int64_t workspace_bytes,
                                void* stream);

/* ---- dense helper of the whole-model harness --------------------------- */

/* h_out = LayerNorm(x [+ delta]) * gamma + beta over rows of `cols` 16-bit elements (DIMQ_BF16 or
 * DIMQ_F16), statistics in fp32; with delta != NULL the sum x + delta (rounded to the element type)
 * is also written to x_out (the residual stream).  cols % 8 == 0, cols <= 1024, 16-byte aligned rows.
 * No counterpart in the reference: its models use torch.nn.LayerNorm; this fuses the residual add of
 * a transformer block with the normalisation that follows it. */
DIMQ_API int dimq_add_layer_norm(const void* x, const void* delta, const void* gamma, const void* beta,
                                 void* x_out, void* h_out, int64_t rows, int64_t cols, float eps, int dtype,
                                 void* stream);

/* cols[(b, oh, ow)][k] = x[b][c][ih][iw] with k = (kh * KW + kw) * C + c (zero outside the image and in
 * the padding columns k >= KH*KW*C up to padded_k, a multiple of 8): the explicit patch matrix of a
 * groups == 1 convolution over 16-bit activations addressed by geom->x_stride.  Used for the 3-channel
 * stem of ResNet, whose k blocks do not fit the implicit-GEMM convolution; the result feeds
 * dimq_linear_wq with the weight re-ordered by dimq_conv_prepack.  `cols` is caller-owned scratch of
 * batch*out_h*out_w*padded_k elements.  No counterpart in the reference. */
DIMQ_API int dimq_im2col(const void* x, int dtype, const dimq_conv_geom* geom, int64_t padded_k, void* cols,
                         void* stream);

/* Max-pool over NHWC 16-bit activations (channels % 8 == 0); dense helper of the ResNet harness, in the
 * reference's models this is torch.nn.MaxPool2d. */
DIMQ_API int dimq_max_pool_nhwc(const void* x, void* y, int dtype, int64_t batch, int64_t height, int64_t width,
                                int64_t channels, int kernel, int stride, int pad, void* stream);

/* Image batch NCHW (3 channels, fp32 / fp16 / bf16, contiguous) -> NHWC 16-bit (`y_dtype` bf16 or fp16), the
 * layout the stem convolution reads; height * width must be a multiple of 8.  Dense helper of the ResNet
 * harness (in the reference's pipeline: `images.to(dtype).contiguous(memory_format=channels_last)`). */
DIMQ_API int dimq_images_to_nhwc(const void* x, int x_dtype, void* y, int y_dtype, int64_t batch, int64_t height,
                                 int64_t width, void* stream);

/* Status word written by the last tensor-core kernel on this thread's device that
 * gave up a bounded wait (0 = none; bit 31 set plus a code naming the waiter otherwise).  Reading it
 * synchronises the device and clears the word. */
DIMQ_API int dimq_last_device_status(uint32_t* status);

/* Health check of the bounded-wait mechanism every pipeline barrier of the tensor-core kernels uses:
 * one warp waits on a barrier that nothing arrives at, gives up after `polls` polls (1..4096, each at
 * most 20 us), and writes result[0] = 1 (the wait reported "gave up") and result[1] = the CTA's abort
 * flag to the two device words at `result`.  dimq_last_device_status then returns 0x80007E57 once.
 * The kernel returns normally: nothing traps or hangs.  No counterpart in the reference (its kernels
 * have no device-side waits). */
DIMQ_API int dimq_selftest_bounded_wait(uint32_t polls, uint32_t* result, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DIMQ_B200_H_ */
