"""CPU restatement (numpy) of the DIMQ packed-index inference path.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA kernels are
compared against; nothing in the product package imports it.  Every function
names the file:line of the DIMQ reference it restates.

Parity status: pinned.  ``tests/golden/*.npz`` were produced by importing the
reference's own Python functions (``tests/golden/make_golden.py``) and
``tests/test_oracle_golden.py`` checks every function here against them.  The
2-/3-/8-bit packing layouts and grouped codebooks have no counterpart in the
reference (it is 4-bit, per-layer only); they are defined here as the
little-endian bit-stream generalisation of the 4-bit rule and are pinned by
round trips and by agreement with the 4-bit reference layout at ``bits == 4``.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# index bit-packing
# --------------------------------------------------------------------------

def pack_bits(indices: np.ndarray, bits: int) -> np.ndarray:
    """Pack ``bits``-wide indices into a little-endian bit stream.

    Index ``j`` occupies stream bits ``[j*bits, (j+1)*bits)``; stream bit ``t``
    is bit ``t % 8`` of byte ``t // 8``; unused tail bits are zero.  For
    ``bits == 4`` this is ``packed[j] = idx[2j] | idx[2j+1] << 4`` with a zero
    high nibble on an odd tail, i.e. dimq_backend/export.py:38-55 and
    csrc/dimq_pack.cu:11-25.  Values are masked to ``bits`` bits the way the
    CUDA kernel masks (``& 0x0F``, csrc/dimq_pack.cu:19,22).
    """
    if bits not in (1, 2, 3, 4, 8):
        raise ValueError(f"unsupported bit width {bits}")
    flat = np.ascontiguousarray(indices).reshape(-1).astype(np.uint8)
    n = flat.size
    if n == 0:
        return np.zeros((0,), dtype=np.uint8)
    flat = flat & np.uint8((1 << bits) - 1)
    # bit matrix [n, bits], least-significant bit first
    bitmat = (flat[:, None] >> np.arange(bits, dtype=np.uint8)[None, :]) & 1
    stream = bitmat.reshape(-1)
    nbytes = (n * bits + 7) // 8
    pad = nbytes * 8 - stream.size
    if pad:
        stream = np.concatenate([stream, np.zeros(pad, dtype=np.uint8)])
    return np.packbits(stream.reshape(nbytes, 8), axis=1, bitorder="little").reshape(-1)


def unpack_bits(packed: np.ndarray, numel: int, bits: int) -> np.ndarray:
    """Inverse of :func:`pack_bits`; ``numel`` trims the pad bits.

    ``bits == 4`` restates dimq_backend/export.py:58-78 and ``get_u4``
    (csrc/dimq_common.cuh:9-15): even index -> low nibble.
    """
    if bits not in (1, 2, 3, 4, 8):
        raise ValueError(f"unsupported bit width {bits}")
    if numel < 0:
        raise ValueError("numel must be non-negative")
    flat = np.ascontiguousarray(packed).reshape(-1).astype(np.uint8)
    needed = (numel * bits + 7) // 8
    if flat.size < needed:
        raise ValueError(f"packed tensor has {flat.size} bytes, expected at least {needed}")
    if numel == 0:
        return np.zeros((0,), dtype=np.uint8)
    stream = np.unpackbits(flat[:needed], bitorder="little")[: numel * bits]
    bitmat = stream.reshape(numel, bits).astype(np.uint16)
    weights = (1 << np.arange(bits, dtype=np.uint16))[None, :]
    return (bitmat * weights).sum(axis=1).astype(np.uint8)


def pack_u4(indices: np.ndarray) -> np.ndarray:
    """dimq_backend/export.py:38-55 (range check included, as the Python twin does)."""
    flat = np.ascontiguousarray(indices).reshape(-1)
    if flat.size and (int(flat.max()) > 15 or int(flat.min()) < 0):
        raise ValueError("u4 indices must be in [0, 15]")
    return pack_bits(flat, 4)


def unpack_u4(packed: np.ndarray, numel: int) -> np.ndarray:
    """dimq_backend/export.py:58-78."""
    return unpack_bits(packed, numel, 4)


# --------------------------------------------------------------------------
# hard quantisation (nearest codeword, ties to the lowest index)
# --------------------------------------------------------------------------

def hard_quantize(w: np.ndarray, centers: np.ndarray) -> np.ndarray:
    """``argmin_k (float(w) - float(c_k))**2`` with torch.argmin semantics.

    Restates quant/dimq.py:197-221 (and dimq_backend/export.py:24-35): the
    squared distance is formed in fp32 (subtract, then multiply), the first
    minimum wins, and a NaN distance beats every number (first NaN wins), which
    is what ``Tensor.argmin`` does.  Chunking in the reference does not change
    the result, so none is done here.  Returns uint8 indices shaped like ``w``.
    """
    wf = np.asarray(w, dtype=F32).reshape(-1)
    c = np.asarray(centers, dtype=F32).reshape(-1)
    if c.size == 0:
        raise ValueError("centers must be non-empty")
    out = np.empty(wf.size, dtype=np.uint8)
    step = 1 << 18
    with np.errstate(invalid="ignore", over="ignore"):
        for s in range(0, wf.size, step):
            part = wf[s : s + step]
            d = part[:, None] - c[None, :]
            d = d * d
            nan = np.isnan(d)
            idx = np.argmin(np.where(nan, F32(np.inf), d), axis=1)
            has_nan = nan.any(axis=1)
            if has_nan.any():
                idx = np.where(has_nan, np.argmax(nan, axis=1), idx)
            out[s : s + step] = idx.astype(np.uint8)
    return out.reshape(np.shape(w))


def group_of_row(n_rows: int, group_rows: int) -> np.ndarray:
    """Codebook group of output row ``n``: ``n // group_rows`` (extension; the
    reference has one codebook per layer, dimq_backend/export.py:218)."""
    return np.arange(n_rows) // int(group_rows)


def hard_quantize_grouped(w2d: np.ndarray, codebooks: np.ndarray, group_rows: int) -> np.ndarray:
    """Slice-by-slice application of :func:`hard_quantize` for ``[G, K]``
    codebooks: rows ``[g*group_rows, (g+1)*group_rows)`` use ``codebooks[g]``."""
    w2d = np.asarray(w2d, dtype=F32)
    rows = w2d.shape[0]
    flat = w2d.reshape(rows, -1)
    out = np.empty(flat.shape, dtype=np.uint8)
    for g in range(codebooks.shape[0]):
        lo, hi = g * group_rows, min((g + 1) * group_rows, rows)
        if lo >= hi:
            break
        out[lo:hi] = hard_quantize(flat[lo:hi], codebooks[g])
    return out.reshape(w2d.shape)


def dequantize(indices: np.ndarray, codebooks: np.ndarray, group_rows: int | None = None) -> np.ndarray:
    """``codebook.float()[indices]`` (dimq_backend/reference.py:47-56), grouped
    by output row when ``codebooks`` is ``[G, K]``."""
    cb = np.asarray(codebooks, dtype=F32)
    idx = np.asarray(indices).astype(np.int64)
    if cb.ndim == 1 or cb.shape[0] == 1:
        return cb.reshape(-1)[idx]
    rows = idx.shape[0]
    g = group_of_row(rows, group_rows if group_rows else rows)
    flat = idx.reshape(rows, -1)
    return cb[g[:, None], flat].reshape(idx.shape)


# --------------------------------------------------------------------------
# W4A4 pieces
# --------------------------------------------------------------------------

def quantize_activation_u4(x: np.ndarray, act_scale: float, act_zero_point: int) -> np.ndarray:
    """``clamp(round(x.float() / scale) + zp, 0, 15)`` as uint8.

    dimq_backend/reference.py:11-21.  The divide is an IEEE fp32 divide by the
    fp32-rounded scale (what the CPU ``Tensor / float`` does) and ``round`` is
    round-half-to-even; csrc/dimq_common.cuh:17-21 is the CUDA twin.
    """
    if float(act_scale) <= 0.0:
        raise ValueError("act_scale must be positive")
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        q = np.rint(np.asarray(x, dtype=F32) / F32(act_scale)) + F32(int(act_zero_point))
        q = np.clip(q, F32(0), F32(15))
        # NaN stays NaN through clip; the uint8 cast of NaN is 0 in torch on x86
        q = np.where(np.isnan(q), F32(0), q)
    return q.astype(np.uint8)


def build_product_table(codebook: np.ndarray, act_scale: float, act_zero_point: int) -> np.ndarray:
    """``P[w, a] = C[w] * (s * (a - z))`` in fp32 — association as in
    dimq_backend/reference.py:32-44 and csrc/dimq_product_table.cu:11-25.
    ``codebook`` may be ``[K]`` or ``[G, K]``; the result is ``[..., K, 16]``."""
    c = np.asarray(codebook, dtype=F32)
    a = np.arange(16, dtype=F32)
    a_hat = F32(act_scale) * (a - F32(int(act_zero_point)))
    return (c[..., :, None] * a_hat).astype(F32)


def linear_lut_a4(x, packed_w, codebook, act_scale, act_zero_point, out_features, in_features, bias=None):
    """W4A4 LUT linear: ``y[m,n] = sum_k P[widx[n,k], q(x[m,k])] + bias[n]``.

    dimq_backend/reference.py:59-88; accumulation in fp32 in ascending ``k``
    like csrc/dimq_gemm_lut.cu:45-49 (the torch oracle sums in another order;
    the reference's own tolerance between the two is 1e-5/1e-6).
    """
    x2 = np.asarray(x, dtype=F32).reshape(-1, in_features)
    widx = unpack_u4(packed_w, out_features * in_features).reshape(out_features, in_features).astype(np.int64)
    table = build_product_table(np.asarray(codebook).reshape(-1), act_scale, act_zero_point)
    aidx = quantize_activation_u4(x2, act_scale, act_zero_point).astype(np.int64)
    y = np.zeros((x2.shape[0], out_features), dtype=F32)
    for k in range(in_features):
        y += table[widx[None, :, k], aidx[:, None, k]]
    if bias is not None:
        y = y + np.asarray(bias, dtype=F32).reshape(1, -1)
    return y.reshape(*np.shape(x)[:-1], out_features)


def conv_out_size(size, pad, dil, k, stride):
    """csrc/dimq_conv2d_lut.cu:129-130."""
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


def _im2col(x, kh, kw, stride, padding, dilation):
    """NCHW -> [B, C, KH, KW, OH, OW] with zero padding (taps outside the image
    contribute nothing: csrc/dimq_conv2d_lut.cu:66-73)."""
    b, c, h, w = x.shape
    sh, sw = stride
    ph, pw = padding
    dh, dw = dilation
    oh = conv_out_size(h, ph, dh, kh, sh)
    ow = conv_out_size(w, pw, dw, kw, sw)
    xp = np.zeros((b, c, h + 2 * ph, w + 2 * pw), dtype=x.dtype)
    xp[:, :, ph : ph + h, pw : pw + w] = x
    cols = np.zeros((b, c, kh, kw, max(oh, 0), max(ow, 0)), dtype=x.dtype)
    for i in range(kh):
        for j in range(kw):
            cols[:, :, i, j] = xp[:, :, i * dh : i * dh + sh * oh : sh, j * dw : j * dw + sw * ow : sw][:, :, :oh, :ow]
    return cols, oh, ow


def conv2d_dense(x, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    """fp32 ``F.conv2d`` restated with im2col + matmul (NCHW in, NCHW out)."""
    x = np.asarray(x, dtype=F32)
    weight = np.asarray(weight, dtype=F32)
    oc, icg, kh, kw = weight.shape
    b = x.shape[0]
    cols, oh, ow = _im2col(x, kh, kw, stride, padding, dilation)
    y = np.zeros((b, oc, oh, ow), dtype=F32)
    ocg = oc // groups
    for g in range(groups):
        cg = cols[:, g * icg : (g + 1) * icg].reshape(b, icg * kh * kw, oh * ow)
        wg = weight[g * ocg : (g + 1) * ocg].reshape(ocg, icg * kh * kw)
        y[:, g * ocg : (g + 1) * ocg] = np.einsum("ok,bkp->bop", wg, cg, optimize=True).reshape(b, ocg, oh, ow)
    if bias is not None:
        y = y + np.asarray(bias, dtype=F32).reshape(1, -1, 1, 1)
    return y


def conv2d_lut_a4(x, packed_w, codebook, act_scale, act_zero_point, weight_shape, bias=None,
                  stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    """W4A4 conv: dequantise both operands, then a dense fp32 conv
    (dimq_backend/reference.py:113-144)."""
    weight_shape = tuple(int(v) for v in weight_shape)
    numel = int(np.prod(weight_shape))
    widx = unpack_u4(packed_w, numel).reshape(weight_shape)
    w_hat = dequantize(widx, np.asarray(codebook).reshape(-1))
    q = quantize_activation_u4(x, act_scale, act_zero_point)
    x_hat = F32(act_scale) * (q.astype(F32) - F32(int(act_zero_point)))
    return conv2d_dense(x_hat, w_hat, bias, stride, padding, dilation, groups)


# --------------------------------------------------------------------------
# weight-only path (what the throughput configurations time)
# --------------------------------------------------------------------------

def linear_wq(x, packed_w, codebooks, bits, out_features, in_features, bias=None, group_rows=None):
    """``F.linear(x.float(), dequantize_packed_weight(...), bias.float())``:
    dimq_backend/reference.py:47-56 followed by a dense fp32 linear, with the
    grouped-codebook and bit-width generalisations."""
    idx = unpack_bits(packed_w, out_features * in_features, bits).reshape(out_features, in_features)
    w_hat = dequantize(idx, codebooks, group_rows)
    x2 = np.asarray(x, dtype=F32).reshape(-1, in_features)
    y = x2 @ w_hat.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=F32).reshape(1, -1)
    return y.reshape(*np.shape(x)[:-1], out_features).astype(F32)


def conv2d_wq(x, packed_w, codebooks, bits, weight_shape, bias=None, stride=(1, 1), padding=(0, 0),
              dilation=(1, 1), groups=1, group_rows=None):
    """``F.conv2d(x.float(), dequantize_packed_weight(...), ...)`` on
    NCHW-logical tensors (dimq_backend/reference.py:113-144 without the
    activation quantiser)."""
    weight_shape = tuple(int(v) for v in weight_shape)
    idx = unpack_bits(packed_w, int(np.prod(weight_shape)), bits).reshape(weight_shape)
    w_hat = dequantize(idx, codebooks, group_rows)
    return conv2d_dense(x, w_hat, bias, stride, padding, dilation, groups)


def parity_metrics(y: np.ndarray, y_ref: np.ndarray) -> tuple[float, float]:
    """``(max_abs, rel_l2)`` over the whole tensor, both in float64."""
    a = np.asarray(y, dtype=np.float64).reshape(-1)
    b = np.asarray(y_ref, dtype=np.float64).reshape(-1)
    if a.size == 0:
        return 0.0, 0.0
    max_abs = float(np.max(np.abs(a - b)))
    denom = float(np.linalg.norm(b))
    rel = float(np.linalg.norm(a - b) / denom) if denom > 0 else float(np.linalg.norm(a - b))
    return max_abs, rel


# --------------------------------------------------------------------------
# codebook construction used by the synthetic workloads
# --------------------------------------------------------------------------

def quantile_codebook(w: np.ndarray, k: int) -> np.ndarray:
    """Quantile initialisation of a sorted ``k``-entry codebook.

    Follows quant/dimq.py:132-137 (probabilities ``linspace(0,1,k+2)[1:-1]``,
    linear interpolation) and the post-processing at quant/dimq.py:175-194
    (sort, enforce strictly increasing with a ``1e-6`` relative gap, keep the
    mean, sort).  The reference subsamples above 200 000 values with the global
    RNG; the synthetic workloads here use every value instead.
    """
    flat = np.asarray(w, dtype=F32).reshape(-1)
    flat = flat[np.isfinite(flat)]
    q = np.linspace(0.0, 1.0, k + 2, dtype=F32)[1:-1]
    centers = np.quantile(flat.astype(np.float64), q.astype(np.float64)).astype(F32)
    centers = np.sort(centers)
    span = abs(float(flat.max()) - float(flat.min()))
    sigma = abs(float(flat.std()))
    min_gap = F32(max(max(span, sigma), 1e-6) * 1e-6)
    fixed = centers.copy()
    for i in range(1, k):
        if fixed[i] <= fixed[i - 1]:
            fixed[i] = fixed[i - 1] + min_gap
    fixed = fixed - (fixed.mean(dtype=F32) - centers.mean(dtype=F32))
    return np.sort(fixed).astype(F32)


def linear_prepack(packed_w, out_features, in_features, bits):
    """Byte order of ``dimq_linear_prepack``: the canonical ``[N][K * bits / 8]`` index stream cut into tiles of
    16 rows x 128 k, stored ``[row block][128-k range][row][16 * bits bytes]``.  No counterpart in the
    reference (its kernels read the canonical stream, csrc/dimq_gemm_lut.cu:45-49); the layout is this
    library's own and the oracle states it so that the kernel can be checked against something."""
    piece = 16 * bits
    rows = np.asarray(packed_w, dtype=np.uint8).reshape(out_features, in_features * bits // 8)
    assert out_features % 16 == 0 and in_features % 128 == 0
    tiles = rows.reshape(out_features // 16, 16, in_features // 128, piece)
    return np.ascontiguousarray(tiles.transpose(0, 2, 1, 3)).reshape(-1)

