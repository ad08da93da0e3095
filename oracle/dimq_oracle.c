/*
 * CPU restatement (plain C, OpenMP) of the DIMQ packed-index inference path.
 *
 * TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared with and
 * the timed CPU baseline.  The product library never links or loads it.
 * Parity status: pinned — tests/test_oracle_golden.py checks every function
 * against vectors produced by the reference's own Python code.
 *
 * Each function cites the reference file:line it follows (paths inside the
 * DIMQ project).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Index j occupies stream bits [j*bits, (j+1)*bits); little-endian stream.
 * bits == 4 is dimq_cuda_backend/csrc/dimq_pack.cu:11-25 / dimq_backend/export.py:38-55. */
void dimq_oracle_pack_bits(const uint8_t* idx, int64_t n, int bits, uint8_t* packed) {
  int64_t nbytes = (n * bits + 7) / 8;
  memset(packed, 0, (size_t)nbytes);
  uint32_t mask = (1u << bits) - 1u;
  for (int64_t j = 0; j < n; ++j) {
    uint32_t v = idx[j] & mask;
    int64_t bit = j * bits;
    int64_t byte = bit >> 3;
    int sh = (int)(bit & 7);
    packed[byte] |= (uint8_t)(v << sh);
    if (sh + bits > 8) packed[byte + 1] |= (uint8_t)(v >> (8 - sh));
  }
}

/* dimq_cuda_backend/csrc/dimq_common.cuh:9-15 (get_u4) generalised to `bits`. */
void dimq_oracle_unpack_bits(const uint8_t* packed, int64_t n, int bits, uint8_t* idx) {
  uint32_t mask = (1u << bits) - 1u;
  int64_t nbytes = (n * bits + 7) / 8;
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < n; ++j) {
    int64_t bit = j * bits;
    int64_t byte = bit >> 3;
    int sh = (int)(bit & 7);
    uint32_t v = packed[byte];
    if (byte + 1 < nbytes) v |= (uint32_t)packed[byte + 1] << 8;
    idx[j] = (uint8_t)((v >> sh) & mask);
  }
}

/* argmin_k (w - c_k)^2 in fp32, first minimum wins, a NaN distance beats every
 * number (first NaN wins): quant/dimq.py:197-221 with Tensor.argmin semantics.
 * Row r of the [rows, cols] weight uses codebook (r / group_rows). */
void dimq_oracle_hard_quantize(const float* w, int64_t rows, int64_t cols, const float* codebooks,
                               int K, int64_t group_rows, uint8_t* idx) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* c = codebooks + (r / group_rows) * K;
    for (int64_t j = 0; j < cols; ++j) {
      volatile float x = w[r * cols + j];
      int best = 0;
      volatile float d0 = x - c[0];
      float bestd = d0 * d0;
      for (int k = 1; k < K; ++k) {
        volatile float d = x - c[k];
        float dd = d * d;
        if (dd < bestd || (isnan(dd) && !isnan(bestd))) { bestd = dd; best = k; }
      }
      idx[r * cols + j] = (uint8_t)best;
    }
  }
}

/* clamp(rint(x / s) + z, 0, 15): dimq_backend/reference.py:11-21,
 * dimq_cuda_backend/csrc/dimq_common.cuh:17-21.  IEEE divide, round-half-even. */
static inline uint8_t quant_u4(float x, float s, int z) {
  float q = nearbyintf(x / s) + (float)z;
  if (isnan(q)) return 0;
  if (q < 0.0f) q = 0.0f;
  if (q > 15.0f) q = 15.0f;
  return (uint8_t)q;
}

void dimq_oracle_quantize_activation_u4(const float* x, int64_t n, float s, int z, uint8_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = quant_u4(x[i], s, z);
}

/* P[w,a] = C[w] * (s * (a - z)): dimq_cuda_backend/csrc/dimq_product_table.cu:11-25. */
void dimq_oracle_product_table(const float* codebook, int K, float s, int z, float* table) {
  for (int w = 0; w < K; ++w)
    for (int a = 0; a < 16; ++a) {
      volatile float ah = s * (float)(a - z);
      table[w * 16 + a] = codebook[w] * ah;
    }
}

static inline uint8_t get_u4(const uint8_t* p, int64_t i) {
  uint8_t b = p[i >> 1];
  return (i & 1) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0x0F);
}

/* y[m,n] = sum_k P[w(n,k)][q(x[m,k])] + bias[n], ascending k, fp32:
 * dimq_cuda_backend/csrc/dimq_gemm_lut.cu:16-54. */
void dimq_oracle_linear_lut_a4(const float* x, const uint8_t* packed_w, const float* codebook, float s,
                               int z, const float* bias, float* y, int64_t M, int64_t N, int64_t K) {
  float table[256];
  dimq_oracle_product_table(codebook, 16, s, z, table);
  uint8_t* q = (uint8_t*)malloc((size_t)(M * K ? M * K : 1));
  dimq_oracle_quantize_activation_u4(x, M * K, s, z, q);
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) acc += table[get_u4(packed_w, n * K + k) * 16 + q[m * K + k]];
      if (bias) acc += bias[n];
      y[m * N + n] = acc;
    }
  free(q);
}

/* Direct NCHW convolution over the product table, taps outside the image
 * skipped: dimq_cuda_backend/csrc/dimq_conv2d_lut.cu:14-86. */
void dimq_oracle_conv2d_lut_a4(const float* x, const uint8_t* packed_w, const float* codebook, float s,
                               int z, const float* bias, float* y, int B, int C, int H, int W, int OC,
                               int ICG, int KH, int KW, int sh, int sw, int ph, int pw, int dh, int dw,
                               int groups) {
  float table[256];
  dimq_oracle_product_table(codebook, 16, s, z, table);
  int OH = (H + 2 * ph - dh * (KH - 1) - 1) / sh + 1;
  int OW = (W + 2 * pw - dw * (KW - 1) - 1) / sw + 1;
  int ocg = OC / groups;
  int64_t total = (int64_t)B * OC * OH * OW;
#pragma omp parallel for schedule(static)
  for (int64_t lin = 0; lin < total; ++lin) {
    int ow = (int)(lin % OW);
    int oh = (int)((lin / OW) % OH);
    int co = (int)((lin / ((int64_t)OW * OH)) % OC);
    int b = (int)(lin / ((int64_t)OW * OH * OC));
    int g = co / ocg;
    float acc = 0.0f;
    int64_t wb = (int64_t)co * ICG * KH * KW;
    for (int cg = 0; cg < ICG; ++cg) {
      int ci = g * ICG + cg;
      for (int kh = 0; kh < KH; ++kh) {
        int ih = oh * sh + kh * dh - ph;
        if (ih < 0 || ih >= H) continue;
        for (int kw = 0; kw < KW; ++kw) {
          int iw = ow * sw + kw * dw - pw;
          if (iw < 0 || iw >= W) continue;
          float xv = x[(((int64_t)b * C + ci) * H + ih) * W + iw];
          uint8_t wi = get_u4(packed_w, wb + ((int64_t)cg * KH + kh) * KW + kw);
          acc += table[wi * 16 + quant_u4(xv, s, z)];
        }
      }
    }
    if (bias) acc += bias[co];
    y[lin] = acc;
  }
}

/* Weight-only linear: y = x . C[g(n)][idx(n,k)]^T + bias, fp32 — the
 * dequantize-then-F.linear path of dimq_backend/reference.py:47-56, with the
 * bit-width and grouped-codebook generalisations. */
void dimq_oracle_linear_wq(const float* x, const uint8_t* packed_w, int bits, const float* codebooks,
                           int Kc, int64_t group_rows, const float* bias, float* y, int64_t M, int64_t N,
                           int64_t K) {
  uint8_t* idx = (uint8_t*)malloc((size_t)(N * K ? N * K : 1));
  float* wh = (float*)malloc(sizeof(float) * (size_t)(N * K ? N * K : 1));
  dimq_oracle_unpack_bits(packed_w, N * K, bits, idx);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t k = 0; k < K; ++k) wh[n * K + k] = codebooks[(n / group_rows) * Kc + idx[n * K + k]];
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      const float* xr = x + m * K;
      const float* wr = wh + n * K;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      int64_t k = 0;
      for (; k + 8 <= K; k += 8)
        for (int u = 0; u < 8; ++u) acc[u] += xr[k + u] * wr[k + u];
      float t = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      for (; k < K; ++k) t += xr[k] * wr[k];
      y[m * N + n] = t + (bias ? bias[n] : 0.0f);
    }
  free(idx);
  free(wh);
}
