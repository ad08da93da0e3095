"""Python entry points of the B200 backend — a drop-in for ``dimq_backend.ops``.

The six operators of the reference (dimq_cuda_backend/csrc/dimq_ops.cpp:37-44)
are registered under ``torch.ops.dimq`` with the same schemas and, like there,
only for CUDA tensors; the wrappers below keep the positional signatures of
dimq_cuda_backend/dimq_backend/ops.py:36-119.  Additional operators (any bit
width, grouped codebooks, weight-only GEMM/conv, hard-quantise + pack) are
separate functions and never change the meaning of the frozen ones.

Everything runs in ``libdimq_b200.so``; there is no CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib
from ._lib import ALGO_AUTO, ALGO_GENERIC, ALGO_STREAM, ALGO_TCGEN05, EPI_GELU, EPI_NONE, EPI_RELU  # noqa: F401

_EPILOGUES = {None: EPI_NONE, "none": EPI_NONE, "relu": EPI_RELU, "gelu": EPI_GELU, "add_relu": _lib.EPI_ADD_RELU}
_ALGOS = {None: ALGO_AUTO, "auto": ALGO_AUTO, "generic": ALGO_GENERIC, "stream": ALGO_STREAM,
          "tcgen05": ALGO_TCGEN05, "mma_stream": 4, "expand": 5, "mma_regs": 6}


def is_available() -> bool:
    """Whether the compiled sm_100a library can be loaded."""
    return _lib.is_available()


def require_extension() -> None:
    _lib.lib()


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} expects a CUDA tensor")


def _pair(value) -> tuple[int, int]:
    if isinstance(value, int):
        return int(value), int(value)
    if len(value) != 2:
        raise ValueError(f"expected pair, got {value!r}")
    return int(value[0]), int(value[1])


# ---------------------------------------------------------------------------
# implementations (CUDA tensors in, CUDA tensors out)
# ---------------------------------------------------------------------------

def _pack_bits_impl(indices: torch.Tensor, bits: int) -> torch.Tensor:
    _require_cuda(indices, "pack")
    if indices.dtype != torch.uint8:
        raise RuntimeError("pack expects uint8 indices")
    flat = indices.contiguous().view(-1)
    n = flat.numel()
    packed = torch.empty(((n * bits + 7) // 8,), dtype=torch.uint8, device=flat.device)
    with torch.cuda.device(flat.device):
        st = _lib.lib().dimq_pack_bits(_lib.ptr(flat), C.c_int64(n), C.c_int(bits), _lib.ptr(packed),
                                       _lib.stream_ptr(flat.device))
    _lib.check(st, "pack_bits")
    return packed


def _unpack_bits_impl(packed: torch.Tensor, numel: int, bits: int) -> torch.Tensor:
    _require_cuda(packed, "unpack")
    if packed.dtype != torch.uint8:
        raise RuntimeError("unpack expects uint8 packed data")
    if numel < 0:
        raise RuntimeError("numel must be non-negative")
    if packed.numel() < (numel * bits + 7) // 8:
        raise RuntimeError("packed tensor is too small for requested numel")
    flat = packed.contiguous().view(-1)
    out = torch.empty((numel,), dtype=torch.uint8, device=flat.device)
    with torch.cuda.device(flat.device):
        st = _lib.lib().dimq_unpack_bits(_lib.ptr(flat), C.c_int64(numel), C.c_int(bits), _lib.ptr(out),
                                         _lib.stream_ptr(flat.device))
    _lib.check(st, "unpack_bits")
    return out


def _pack_u4_impl(indices: torch.Tensor) -> torch.Tensor:
    return _pack_bits_impl(indices, 4)


def _unpack_u4_impl(packed: torch.Tensor, numel: int) -> torch.Tensor:
    return _unpack_bits_impl(packed, int(numel), 4)


def _check_qparams(act_scale: float, act_zp: int) -> None:
    if not act_scale > 0.0:
        raise RuntimeError("act_scale must be positive")
    if act_zp < 0 or act_zp > 15:
        raise RuntimeError("act_zero_point must be in [0, 15]")


def _quantize_activation_u4_impl(x: torch.Tensor, act_scale: float, act_zp: int) -> torch.Tensor:
    _require_cuda(x, "quantize_activation_u4")
    if not x.is_floating_point():
        raise RuntimeError("quantize_activation_u4 expects floating input")
    _check_qparams(act_scale, act_zp)
    xc = x.contiguous()
    out = torch.empty(xc.shape, dtype=torch.uint8, device=xc.device)
    with torch.cuda.device(xc.device):
        st = _lib.lib().dimq_quantize_activation_u4(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.c_int64(xc.numel()),
                                                    C.c_float(act_scale), C.c_int(act_zp), _lib.ptr(out),
                                                    _lib.stream_ptr(xc.device))
    _lib.check(st, "quantize_activation_u4")
    return out


def _build_product_table_impl(codebook: torch.Tensor, act_scale: float, act_zp: int) -> torch.Tensor:
    _require_cuda(codebook, "build_product_table")
    if not codebook.is_floating_point():
        raise RuntimeError("build_product_table expects floating codebook")
    if codebook.numel() != 16:
        raise RuntimeError("build_product_table expects exactly 16 codebook entries")
    _check_qparams(act_scale, act_zp)
    return build_product_table_grouped(codebook.reshape(1, 16), act_scale, act_zp).view(16, 16)


def _bias_arg(bias: torch.Tensor | None, n: int, device: torch.device, what: str):
    if bias is None:
        return None, 0
    if not bias.is_cuda:
        raise RuntimeError("bias must be CUDA when provided")
    if bias.numel() != n:
        raise RuntimeError(f"bias numel must equal {what}")
    b = bias.contiguous().view(-1)
    return b, _lib.dtype_code(b, "bias")


# W4A4 problems with at least this many activation rows (output pixels for the convolution) take the
# tensor-core path (operands rounded to a hi + lo bf16 pair); smaller ones the exact table-lookup kernel.
A4_TC_MIN_ROWS = 512
_UNSUPPORTED = -7


def _a4_workspace(x_numel: int, conv_weight_numel: int, device: torch.device) -> torch.Tensor:
    need = C.c_int64(0)
    st = _lib.lib().dimq_a4_workspace_bytes(C.c_int64(x_numel), C.c_int64(conv_weight_numel), C.byref(need))
    if st != 0:
        raise RuntimeError(f"dimq_b200.a4_workspace_bytes failed (status {st})")
    return torch.empty(need.value, dtype=torch.uint8, device=device)


def centre_quantize_u4(x: torch.Tensor, act_scale: float, act_zero_point: int) -> torch.Tensor:
    """``clamp(rint(x / act_scale) + z, 0, 15) - z`` as bf16, same shape and memory format as ``x``:
    the activation codes of the W4A4 ops with the zero point removed (integers in [-15, 15])."""
    require_extension()
    _require_cuda(x, "centre_quantize_u4")
    if not x.is_floating_point():
        raise RuntimeError("centre_quantize_u4 expects floating input")
    _check_qparams(act_scale, act_zero_point)
    dense = x.is_contiguous() or (x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last))
    xc = x if dense else x.contiguous()
    out = torch.empty_like(xc, dtype=torch.bfloat16)       # keeps the strides of a dense tensor
    with torch.cuda.device(xc.device):
        st = _lib.lib().dimq_centre_quantize_u4(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.c_int64(xc.numel()),
                                                C.c_float(act_scale), C.c_int(act_zero_point), _lib.ptr(out),
                                                _lib.stream_ptr(xc.device))
    _lib.check(st, "centre_quantize_u4")
    return out


def _linear_lut_impl(x, packed_w, codebook, act_scale, act_zp, bias, out_features, in_features):
    _require_cuda(x, "linear_lut")
    _require_cuda(packed_w, "linear_lut")
    _require_cuda(codebook, "linear_lut")
    if not x.is_floating_point():
        raise RuntimeError("linear_lut expects floating input")
    if packed_w.dtype != torch.uint8:
        raise RuntimeError("packed_weight must be uint8")
    if not codebook.is_floating_point():
        raise RuntimeError("codebook must be floating point")
    if codebook.numel() != 16:
        raise RuntimeError("codebook must have 16 entries for W4")
    _check_qparams(act_scale, act_zp)
    if out_features <= 0 or in_features <= 0:
        raise RuntimeError("linear dimensions must be positive")
    if x.numel() % in_features != 0:
        raise RuntimeError("input numel must be divisible by in_features")
    if packed_w.numel() < (out_features * in_features + 1) // 2:
        raise RuntimeError("packed_weight is too small for out_features * in_features")
    if x.dim() == 0 or x.size(-1) != in_features:
        raise RuntimeError("input last dimension must equal in_features")
    xc = x.contiguous()
    pw = packed_w.contiguous().view(-1)
    cb = codebook.contiguous().view(-1)
    b, b_dt = _bias_arg(bias, out_features, xc.device, "out_features")
    m = xc.numel() // in_features
    y = torch.empty((m, out_features), dtype=torch.float32, device=xc.device)
    if m >= A4_TC_MIN_ROWS and in_features % 64 == 0 and pw.data_ptr() % 16 == 0:
        ws = _a4_workspace(xc.numel(), 0, xc.device)
        with torch.cuda.device(xc.device):
            st = _lib.lib().dimq_linear_lut_tc(_lib.ptr(xc), _lib.dtype_code(xc, "x"), _lib.ptr(pw), _lib.ptr(cb),
                                               _lib.dtype_code(cb, "codebook"), C.c_float(act_scale), C.c_int(act_zp),
                                               _lib.ptr(b), b_dt, _lib.ptr(y), C.c_int64(m), C.c_int64(out_features),
                                               C.c_int64(in_features), _lib.ptr(ws), C.c_int64(ws.numel()),
                                               _lib.stream_ptr(xc.device))
        if st != _UNSUPPORTED:
            _lib.check(st, "linear_lut_tc")
            _lib.LAUNCH_COUNT[0] += 1  # the activation quantiser and the GEMM
            return y.view(*x.shape[:-1], out_features)
    with torch.cuda.device(xc.device):
        st = _lib.lib().dimq_linear_lut(_lib.ptr(xc), _lib.dtype_code(xc, "x"), _lib.ptr(pw), _lib.ptr(cb),
                                        _lib.dtype_code(cb, "codebook"), C.c_float(act_scale), C.c_int(act_zp),
                                        _lib.ptr(b), b_dt, _lib.ptr(y), C.c_int64(m), C.c_int64(out_features),
                                        C.c_int64(in_features), _lib.stream_ptr(xc.device))
    _lib.check(st, "linear_lut")
    return y.view(*x.shape[:-1], out_features)


def _conv_geom(x: torch.Tensor, weight_shape, stride, padding, dilation, groups) -> _lib.ConvGeom:
    oc, icg, kh, kw = (int(v) for v in weight_shape)
    g = _lib.ConvGeom()
    g.batch, g.in_channels, g.in_h, g.in_w = (int(v) for v in x.shape)
    g.out_channels, g.in_channels_per_group, g.kernel_h, g.kernel_w = oc, icg, kh, kw
    g.stride_h, g.stride_w = stride
    g.pad_h, g.pad_w = padding
    g.dilation_h, g.dilation_w = dilation
    g.groups = int(groups)
    if oc <= 0 or icg <= 0:
        raise RuntimeError("channel counts must be positive")
    if kh <= 0 or kw <= 0:
        raise RuntimeError("kernel size must be positive")
    if g.stride_h <= 0 or g.stride_w <= 0:
        raise RuntimeError("stride must be positive")
    if g.dilation_h <= 0 or g.dilation_w <= 0:
        raise RuntimeError("dilation must be positive")
    if g.groups <= 0:
        raise RuntimeError("groups must be positive")
    if g.in_channels != icg * g.groups:
        raise RuntimeError("input channels do not match weight/groups")
    if oc % g.groups != 0:
        raise RuntimeError("out_channels must be divisible by groups")
    st = _lib.lib().dimq_conv_out_size(C.byref(g))
    if st != 0:
        raise RuntimeError("computed negative output size")
    return g


def _conv_io(x: torch.Tensor, g: _lib.ConvGeom, out_dtype: torch.dtype):
    """Input as stored (NCHW-contiguous or channels_last, no copy) and an output in the same format."""
    channels_last = x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous()
    xc = x if (channels_last or x.is_contiguous()) else x.contiguous()
    y = torch.empty((g.batch, g.out_channels, g.out_h, g.out_w), dtype=out_dtype, device=x.device,
                    memory_format=torch.channels_last if channels_last else torch.contiguous_format)
    for i in range(4):
        g.x_stride[i] = xc.stride(i)
        g.y_stride[i] = y.stride(i)
    return xc, y


def _conv2d_lut_impl(x, packed_w, codebook, act_scale, act_zp, bias, out_channels, in_channels_per_group,
                     kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w, groups):
    _require_cuda(x, "conv2d_lut")
    if x.dim() != 4:
        raise RuntimeError("conv2d_lut expects NCHW input")
    _require_cuda(packed_w, "conv2d_lut")
    _require_cuda(codebook, "conv2d_lut")
    if not x.is_floating_point():
        raise RuntimeError("conv2d_lut expects floating input")
    if packed_w.dtype != torch.uint8:
        raise RuntimeError("packed_weight must be uint8")
    if not codebook.is_floating_point():
        raise RuntimeError("codebook must be floating point")
    if codebook.numel() != 16:
        raise RuntimeError("codebook must have 16 entries for W4")
    _check_qparams(act_scale, act_zp)
    g = _conv_geom(x, (out_channels, in_channels_per_group, kernel_h, kernel_w), (stride_h, stride_w),
                   (pad_h, pad_w), (dilation_h, dilation_w), groups)
    numel = out_channels * in_channels_per_group * kernel_h * kernel_w
    if packed_w.numel() < (numel + 1) // 2:
        raise RuntimeError("packed_weight is too small for requested conv weight shape")
    b, b_dt = _bias_arg(bias, out_channels, x.device, "out_channels")
    xc, y = _conv_io(x, g, torch.float32)
    if y.numel() == 0:
        return y
    pw = packed_w.contiguous().view(-1)
    cb = codebook.contiguous().view(-1)
    channels_last = g.x_stride[1] == 1 and g.y_stride[1] == 1
    if (channels_last and groups == 1 and g.in_channels % 64 == 0
            and g.batch * g.out_h * g.out_w >= A4_TC_MIN_ROWS):
        ws = _a4_workspace(xc.numel(), numel, x.device)
        with torch.cuda.device(x.device):
            st = _lib.lib().dimq_conv2d_lut_tc(_lib.ptr(xc), _lib.dtype_code(xc, "x"), _lib.ptr(pw), _lib.ptr(cb),
                                               _lib.dtype_code(cb, "codebook"), C.c_float(act_scale), C.c_int(act_zp),
                                               _lib.ptr(b), b_dt, _lib.ptr(y), C.byref(g), _lib.ptr(ws),
                                               C.c_int64(ws.numel()), _lib.stream_ptr(x.device))
        if st != _UNSUPPORTED:
            _lib.check(st, "conv2d_lut_tc")
            _lib.LAUNCH_COUNT[0] += 2  # index re-order, activation quantiser, convolution
            return y
    with torch.cuda.device(x.device):
        st = _lib.lib().dimq_conv2d_lut(_lib.ptr(xc), _lib.dtype_code(xc, "x"), _lib.ptr(pw), _lib.ptr(cb),
                                        _lib.dtype_code(cb, "codebook"), C.c_float(act_scale), C.c_int(act_zp),
                                        _lib.ptr(b), b_dt, _lib.ptr(y), C.byref(g), _lib.stream_ptr(x.device))
    _lib.check(st, "conv2d_lut")
    return y


# ---------------------------------------------------------------------------
# torch.ops.dimq registration: the reference's six schemas, CUDA key only
# ---------------------------------------------------------------------------

_SCHEMAS = (
    ("pack_u4(Tensor indices) -> Tensor", _pack_u4_impl),
    ("unpack_u4(Tensor packed, int numel) -> Tensor", _unpack_u4_impl),
    ("quantize_activation_u4(Tensor x, float act_scale, int act_zp) -> Tensor", _quantize_activation_u4_impl),
    ("build_product_table(Tensor codebook, float act_scale, int act_zp) -> Tensor", _build_product_table_impl),
    ("linear_lut(Tensor x, Tensor packed_w, Tensor codebook, float act_scale, int act_zp, Tensor? bias, "
     "int out_features, int in_features) -> Tensor", _linear_lut_impl),
    ("conv2d_lut(Tensor x, Tensor packed_w, Tensor codebook, float act_scale, int act_zp, Tensor? bias, "
     "int out_channels, int in_channels_per_group, int kernel_h, int kernel_w, int stride_h, int stride_w, "
     "int pad_h, int pad_w, int dilation_h, int dilation_w, int groups) -> Tensor", _conv2d_lut_impl),
)

_TORCH_LIBRARY = None


def _register() -> None:
    global _TORCH_LIBRARY
    if _TORCH_LIBRARY is not None:
        return
    library = torch.library.Library("dimq", "DEF")
    for schema, fn in _SCHEMAS:
        library.define(schema)
        library.impl(schema.split("(", 1)[0], fn, "CUDA")
    _TORCH_LIBRARY = library


_register()


# ---------------------------------------------------------------------------
# the reference's Python signatures (dimq_backend/ops.py:36-119)
# ---------------------------------------------------------------------------

def pack_u4(indices: torch.Tensor) -> torch.Tensor:
    require_extension()
    return torch.ops.dimq.pack_u4(indices)


def unpack_u4(packed: torch.Tensor, numel: int) -> torch.Tensor:
    require_extension()
    return torch.ops.dimq.unpack_u4(packed, int(numel))


def quantize_activation_u4(x: torch.Tensor, act_scale: float, act_zero_point: int) -> torch.Tensor:
    require_extension()
    return torch.ops.dimq.quantize_activation_u4(x, float(act_scale), int(act_zero_point))


def build_product_table(codebook: torch.Tensor, act_scale: float, act_zero_point: int) -> torch.Tensor:
    require_extension()
    return torch.ops.dimq.build_product_table(codebook, float(act_scale), int(act_zero_point))


def dimq_linear_lut(x, packed_weight, codebook, act_scale, act_zero_point, bias, out_features, in_features):
    require_extension()
    return torch.ops.dimq.linear_lut(x, packed_weight, codebook, float(act_scale), int(act_zero_point), bias,
                                     int(out_features), int(in_features))


def dimq_conv2d_lut(x, packed_weight, codebook, act_scale, act_zero_point, bias, weight_shape: Sequence[int],
                    stride: Sequence[int], padding: Sequence[int], dilation: Sequence[int], groups: int):
    require_extension()
    out_channels, cin_per_group, kernel_h, kernel_w = [int(v) for v in weight_shape]
    stride_h, stride_w = _pair(stride)
    pad_h, pad_w = _pair(padding)
    dil_h, dil_w = _pair(dilation)
    return torch.ops.dimq.conv2d_lut(x, packed_weight, codebook, float(act_scale), int(act_zero_point), bias,
                                     out_channels, cin_per_group, kernel_h, kernel_w, stride_h, stride_w, pad_h,
                                     pad_w, dil_h, dil_w, int(groups))


# ---------------------------------------------------------------------------
# additional operators
# ---------------------------------------------------------------------------

def pack_bits(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """Little-endian bit-stream packing for ``bits`` in {1, 2, 3, 4, 8}; ``bits == 4`` is ``pack_u4``."""
    require_extension()
    if bits not in (1, 2, 3, 4, 8):
        raise RuntimeError(f"unsupported bit width {bits}")
    return _pack_bits_impl(indices, int(bits))


def unpack_bits(packed: torch.Tensor, numel: int, bits: int) -> torch.Tensor:
    require_extension()
    if bits not in (1, 2, 3, 4, 8):
        raise RuntimeError(f"unsupported bit width {bits}")
    return _unpack_bits_impl(packed, int(numel), int(bits))


def build_product_table_grouped(codebooks: torch.Tensor, act_scale: float, act_zero_point: int) -> torch.Tensor:
    """``[G, K]`` codebooks -> fp32 ``[G, K, 16]`` product tables."""
    require_extension()
    _require_cuda(codebooks, "build_product_table")
    _check_qparams(float(act_scale), int(act_zero_point))
    cb = codebooks.contiguous()
    if cb.dim() != 2:
        raise RuntimeError("codebooks must be [groups, entries]")
    groups, entries = cb.shape
    table = torch.empty((groups, entries, 16), dtype=torch.float32, device=cb.device)
    with torch.cuda.device(cb.device):
        st = _lib.lib().dimq_build_product_table(_lib.ptr(cb), _lib.dtype_code(cb, "codebook"), C.c_int64(groups),
                                                 C.c_int(entries), C.c_float(act_scale), C.c_int(act_zero_point),
                                                 _lib.ptr(table), _lib.stream_ptr(cb.device))
    _lib.check(st, "build_product_table")
    return table


def hard_quantize(w: torch.Tensor, codebooks: torch.Tensor, *, group_rows: int | None = None,
                  bits: int | None = None, return_indices: bool = True):
    """Nearest-codeword indices of ``w`` (ties to the lowest index), optionally packed.

    ``codebooks`` is ``[K]`` (one codebook for the tensor) or ``[G, K]`` with
    ``group_rows`` leading-dimension rows of ``w`` per codebook.  Returns
    ``(indices uint8 shaped like w | None, packed uint8 | None)``.
    """
    require_extension()
    _require_cuda(w, "hard_quantize")
    if not w.is_floating_point():
        raise RuntimeError("hard_quantize expects floating weights")
    wc = w.contiguous()
    cb = codebooks.to(device=wc.device, dtype=torch.float32).contiguous()
    if cb.dim() == 1:
        cb = cb.view(1, -1)
    entries = cb.shape[1]
    if entries == 0:
        raise RuntimeError("centers must be non-empty")
    if entries > 256:
        raise RuntimeError("hard_quantize supports at most 256 centres")
    if cb.shape[0] == 1:
        rows, cols, grp = 1, wc.numel(), 1
    else:
        if group_rows is None or wc.dim() < 1:
            raise RuntimeError("grouped codebooks need group_rows")
        rows = wc.shape[0]
        cols = wc.numel() // max(rows, 1)
        grp = int(group_rows)
        if cb.shape[0] * grp < rows:
            raise RuntimeError("not enough codebooks for the rows of w")
    if bits is not None and (bits not in (1, 2, 3, 4, 8) or entries > (1 << bits)):
        raise RuntimeError(f"cannot pack {entries}-entry indices into {bits} bits")
    idx = torch.empty(wc.shape, dtype=torch.uint8, device=wc.device) if return_indices else None
    packed = None
    if bits is not None:
        packed = torch.empty(((wc.numel() * bits + 7) // 8,), dtype=torch.uint8, device=wc.device)
    if idx is None and packed is None:
        raise RuntimeError("nothing to compute: ask for indices, packed bytes or both")
    with torch.cuda.device(wc.device):
        st = _lib.lib().dimq_hard_quantize(_lib.ptr(wc), _lib.dtype_code(wc, "w"), C.c_int64(rows), C.c_int64(cols),
                                           _lib.ptr(cb), C.c_int(entries), C.c_int64(grp), _lib.ptr(idx),
                                           _lib.ptr(packed), C.c_int(bits if bits is not None else 8),
                                           _lib.stream_ptr(wc.device))
    _lib.check(st, "hard_quantize")
    return idx, packed


def fake_quantize_ste(w: torch.Tensor, codebooks: torch.Tensor, *, group_rows: int | None = None,
                      return_indices: bool = False):
    """``w + (codebook[idx].to(w.dtype) - w)`` with ``idx`` the nearest codeword (ties to the lowest
    index), in one kernel: the value of the straight-through fake quantisation of
    quant/dimq_wrapper.py:72-75.  Returns ``out`` or ``(out, idx uint8)``."""
    require_extension()
    _require_cuda(w, "fake_quantize_ste")
    if not w.is_floating_point() or w.dtype == torch.float64:
        raise RuntimeError("fake_quantize_ste expects float32, float16 or bfloat16 weights")
    wc = w.contiguous()
    cb = codebooks.detach().to(device=wc.device, dtype=torch.float32).contiguous()
    if cb.dim() == 1:
        cb = cb.view(1, -1)
    entries = cb.shape[1]
    if entries == 0:
        raise RuntimeError("centers must be non-empty")
    if entries > 256:
        raise RuntimeError("fake_quantize_ste supports at most 256 centres")
    if cb.shape[0] == 1:
        rows, cols, grp = 1, wc.numel(), 1
    else:
        if group_rows is None or wc.dim() < 1:
            raise RuntimeError("grouped codebooks need group_rows")
        rows = wc.shape[0]
        cols = wc.numel() // max(rows, 1)
        grp = int(group_rows)
        if cb.shape[0] * grp < rows:
            raise RuntimeError("not enough codebooks for the rows of w")
    out = torch.empty_like(wc)
    idx = torch.empty(wc.shape, dtype=torch.uint8, device=wc.device) if return_indices else None
    with torch.cuda.device(wc.device):
        st = _lib.lib().dimq_fake_quantize_ste(_lib.ptr(wc), _lib.dtype_code(wc, "w"), C.c_int64(rows), C.c_int64(cols),
                                               _lib.ptr(cb), C.c_int(entries), C.c_int64(grp), _lib.ptr(out),
                                               _lib.ptr(idx), _lib.stream_ptr(wc.device))
    _lib.check(st, "fake_quantize_ste")
    return (out, idx) if return_indices else out


def _wq_weight(packed_weight: torch.Tensor, codebooks: torch.Tensor, bits: int, out_rows: int, numel: int,
               group_rows: int | None, packed_khwc: torch.Tensor | None = None):
    _require_cuda(packed_weight, "weight-only op")
    _require_cuda(codebooks, "weight-only op")
    if packed_weight.dtype != torch.uint8:
        raise RuntimeError("packed_weight must be uint8")
    if not codebooks.is_floating_point():
        raise RuntimeError("codebook must be floating point")
    if bits not in (2, 3, 4, 8):
        raise RuntimeError(f"unsupported weight bit width {bits}")
    pw = packed_weight.contiguous().view(-1)
    if pw.numel() < (numel * bits + 7) // 8:
        raise RuntimeError("packed_weight is too small for the weight shape")
    cb = codebooks.contiguous()
    if cb.dim() == 1:
        cb = cb.view(1, -1)
    groups, entries = cb.shape
    if entries > (1 << bits):
        raise RuntimeError(f"{entries} codebook entries do not fit {bits}-bit indices")
    if groups == 1:
        grp = out_rows
    else:
        if group_rows is None:
            raise RuntimeError("grouped codebooks need group_rows")
        grp = int(group_rows)
        if groups * grp < out_rows:
            raise RuntimeError("not enough codebooks for the output rows")
    khwc = None
    if packed_khwc is not None:
        khwc = packed_khwc.contiguous().view(-1)
        if khwc.dtype != torch.uint8 or not khwc.is_cuda or khwc.numel() < (numel * bits + 7) // 8:
            raise RuntimeError("packed_khwc must be a CUDA uint8 tensor as large as packed_weight")
    w = _lib.WqWeight(pw.data_ptr(), bits, cb.data_ptr(), _lib.dtype_code(cb, "codebook"), entries, groups, grp,
                      0 if khwc is None else khwc.data_ptr())
    return w, (pw, cb, khwc)


def dimq_linear_wq(x: torch.Tensor, packed_weight: torch.Tensor, codebooks: torch.Tensor,
                   bias: torch.Tensor | None, out_features: int, in_features: int, *, bits: int = 4,
                   group_rows: int | None = None, out_dtype: torch.dtype | None = None,
                   epilogue: str | None = None, residual: torch.Tensor | None = None,
                   algo: str | None = None, packed_tiled: torch.Tensor | None = None) -> torch.Tensor:
    """Weight-only LUT linear: ``x @ codebook[idx].T + bias`` with fp32 accumulation.

    The result the reference gets from ``dequantize_packed_weight`` + ``F.linear``
    (dimq_backend/reference.py:47-56), without materialising the weight.  ``packed_tiled`` (the indices
    re-ordered by :func:`linear_prepack`) speeds up the small-M kernel for large weights; the result is the
    same bits with and without it.
    """
    require_extension()
    _require_cuda(x, "linear_wq")
    if not x.is_floating_point():
        raise RuntimeError("linear_wq expects floating input")
    out_features, in_features = int(out_features), int(in_features)
    if out_features <= 0 or in_features <= 0:
        raise RuntimeError("linear dimensions must be positive")
    if x.dim() == 0 or x.size(-1) != in_features:
        raise RuntimeError("input last dimension must equal in_features")
    xc = x.contiguous()
    w, keep = _wq_weight(packed_weight, codebooks, int(bits), out_features, out_features * in_features, group_rows,
                         packed_tiled)
    b, b_dt = _bias_arg(bias, out_features, xc.device, "out_features")
    out_dtype = out_dtype or torch.float32
    m = xc.numel() // in_features
    y = torch.empty((m, out_features), dtype=out_dtype, device=xc.device)
    res = None
    if residual is not None:
        if residual.dtype != out_dtype or residual.numel() != y.numel():
            raise RuntimeError("residual must match the output shape and dtype")
        res = residual.contiguous()
    if algo == "expand":
        # always the two-step form: expand the indices to a 16-bit weight in scratch, then the dense
        # TMA + tcgen05 GEMM
        need = C.c_int64(0)
        _lib.check(_lib.lib().dimq_expand_workspace_bytes(_lib.dtype_code(xc, "x"), C.byref(w), C.c_int64(out_features),
                                                          C.c_int64(in_features), C.byref(need)), "expand_workspace_bytes")
        ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device=xc.device)
        with torch.cuda.device(xc.device):
            st = _lib.lib().dimq_linear_wq_expand(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), _lib.ptr(b), b_dt,
                                                  _lib.ptr(res), _lib.ptr(y), _lib.dtype_code(y, "y"), C.c_int64(m),
                                                  C.c_int64(out_features), C.c_int64(in_features),
                                                  _EPILOGUES[epilogue], _lib.ptr(ws), C.c_int64(ws.numel()),
                                                  _lib.stream_ptr(xc.device))
        _lib.check(st, "linear_wq_expand")
        _lib.LAUNCH_COUNT[0] += 1  # the expansion and the GEMM
        del keep
        return y.view(*x.shape[:-1], out_features)
    if algo == "mma_regs":
        # the register-resident small-M kernel at any weight size; its k slices meet in scratch memory
        need = C.c_int64(0)
        st = _lib.lib().dimq_linear_wq_regs_workspace_bytes(
            _lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), C.c_int64(m), C.c_int64(out_features),
            C.c_int64(in_features), C.byref(need))
        if st != 0:
            _lib.check(st, "linear_wq_regs_workspace_bytes")   # raises: a size query launches nothing
        ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device=xc.device)
        with torch.cuda.device(xc.device):
            st = _lib.lib().dimq_linear_wq_regs(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), _lib.ptr(b), b_dt,
                                                _lib.ptr(res), _lib.ptr(y), _lib.dtype_code(y, "y"), C.c_int64(m),
                                                C.c_int64(out_features), C.c_int64(in_features), _EPILOGUES[epilogue],
                                                _lib.ptr(ws), C.c_int64(ws.numel()), _lib.stream_ptr(xc.device))
        _lib.check(st, "linear_wq_regs")
        if need.value > 0:
            _lib.LAUNCH_COUNT[0] += 1  # the kernel that adds the k slices
        del keep
        return y.view(*x.shape[:-1], out_features)
    if algo is None:
        # Three shapes get scratch memory: a few activation rows against a large weight (the k slices of
        # the small-M kernel meet there), many activation rows (the indices are expanded once to a
        # 16-bit weight and a dense tensor-core GEMM follows) and a few hundred rows against a long K
        # (the kernel splits K and sums partial tiles there).
        need = C.c_int64(0)
        _lib.lib().dimq_linear_wq_workspace_bytes(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), C.c_int64(m),
                                                  C.c_int64(out_features), C.c_int64(in_features), C.byref(need))
        if need.value > 0:
            ws = torch.empty(need.value, dtype=torch.uint8, device=xc.device)
            with torch.cuda.device(xc.device):
                st = _lib.lib().dimq_linear_wq_ws(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), _lib.ptr(b), b_dt,
                                                  _lib.ptr(res), _lib.ptr(y), _lib.dtype_code(y, "y"), C.c_int64(m),
                                                  C.c_int64(out_features), C.c_int64(in_features),
                                                  _EPILOGUES[epilogue], _lib.ptr(ws), C.c_int64(need.value),
                                                  _lib.stream_ptr(xc.device))
            _lib.check(st, "linear_wq_ws")
            _lib.LAUNCH_COUNT[0] += 1  # two kernels: expansion + GEMM, or GEMM + the kernel that finishes the sums
            del keep
            return y.view(*x.shape[:-1], out_features)
    with torch.cuda.device(xc.device):
        st = _lib.lib().dimq_linear_wq(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), _lib.ptr(b), b_dt,
                                       _lib.ptr(res), _lib.ptr(y), _lib.dtype_code(y, "y"), C.c_int64(m),
                                       C.c_int64(out_features), C.c_int64(in_features), _EPILOGUES[epilogue],
                                       _ALGOS[algo], _lib.stream_ptr(xc.device))
    _lib.check(st, "linear_wq")
    del keep
    return y.view(*x.shape[:-1], out_features)


def dimq_conv2d_wq(x: torch.Tensor, packed_weight: torch.Tensor, codebooks: torch.Tensor,
                   bias: torch.Tensor | None, weight_shape: Sequence[int], stride=(1, 1), padding=(0, 0),
                   dilation=(1, 1), groups: int = 1, *, bits: int = 4, group_rows: int | None = None,
                   out_dtype: torch.dtype | None = None, epilogue: str | None = None,
                   residual: torch.Tensor | None = None, algo: str | None = None,
                   packed_khwc: torch.Tensor | None = None) -> torch.Tensor:
    """Weight-only LUT convolution (logical NCHW; channels_last storage is used as is).

    With ``packed_khwc`` (the indices re-ordered by :func:`conv_prepack`), channels_last bf16/fp16
    activations, ``groups == 1``, a multiple of 64 input channels and stride 1 or 2, the convolution
    runs as an implicit GEMM on the tensor cores; otherwise as a direct convolution.
    """
    require_extension()
    _require_cuda(x, "conv2d_wq")
    if x.dim() != 4:
        raise RuntimeError("conv2d_wq expects NCHW input")
    if not x.is_floating_point():
        raise RuntimeError("conv2d_wq expects floating input")
    g = _conv_geom(x, weight_shape, _pair(stride), _pair(padding), _pair(dilation), groups)
    numel = 1
    for v in weight_shape:
        numel *= int(v)
    w, keep = _wq_weight(packed_weight, codebooks, int(bits), g.out_channels, numel, group_rows, packed_khwc)
    b, b_dt = _bias_arg(bias, g.out_channels, x.device, "out_channels")
    out_dtype = out_dtype or torch.float32
    xc, y = _conv_io(x, g, out_dtype)
    if y.numel() == 0:
        return y
    res = None
    if residual is not None:
        if residual.dtype != out_dtype or residual.shape != y.shape or residual.stride() != y.stride():
            raise RuntimeError("residual must match the output shape, dtype and memory format")
        res = residual
    if algo in (None, "expand"):
        # Many output pixels: expand the indices once to a 16-bit weight in scratch and run a dense
        # tensor-core kernel - the implicit GEMM over the re-ordered indices (packed_khwc), or the stem
        # kernel for a 3-channel stride-2 convolution.  "expand" forces that form at any size.
        need = C.c_int64(0)
        if algo == "expand":
            # the larger of the two layouts: [OC][KH*KW*IC] and the stem's [OC][192]
            numel_k = max(numel // g.out_channels, 192)
            _lib.check(_lib.lib().dimq_expand_workspace_bytes(_lib.dtype_code(xc, "x"), C.byref(w),
                                                              C.c_int64(g.out_channels), C.c_int64(numel_k),
                                                              C.byref(need)), "expand_workspace_bytes")
        else:
            _lib.lib().dimq_conv2d_wq_workspace_bytes(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), C.byref(g),
                                                      C.byref(need))
        if need.value > 0:
            ws = torch.empty(need.value, dtype=torch.uint8, device=x.device)
            fn = _lib.lib().dimq_conv2d_wq_expand if algo == "expand" else _lib.lib().dimq_conv2d_wq_ws
            with torch.cuda.device(x.device):
                st = fn(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), _lib.ptr(b), b_dt, _lib.ptr(res), _lib.ptr(y),
                        _lib.dtype_code(y, "y"), C.byref(g), _EPILOGUES[epilogue], _lib.ptr(ws), C.c_int64(need.value),
                        _lib.stream_ptr(x.device))
            _lib.check(st, "conv2d_wq_ws")
            _lib.LAUNCH_COUNT[0] += 1  # the expansion and the convolution
            del keep
            return y
    with torch.cuda.device(x.device):
        st = _lib.lib().dimq_conv2d_wq(_lib.ptr(xc), _lib.dtype_code(xc, "x"), C.byref(w), _lib.ptr(b), b_dt,
                                       _lib.ptr(res), _lib.ptr(y), _lib.dtype_code(y, "y"), C.byref(g),
                                       _EPILOGUES[epilogue], _ALGOS[algo], _lib.stream_ptr(x.device))
    _lib.check(st, "conv2d_wq")
    del keep
    return y


def linear_prepack(packed_weight: torch.Tensor, out_features: int, in_features: int, bits: int = 4) -> torch.Tensor:
    """Indices of an ``[N, K]`` weight re-ordered into tiles of 16 rows x 128 k (same bit width and size): what
    ``dimq_linear_wq(..., packed_tiled=...)`` takes.  2-, 3- or 4-bit, N a multiple of 16, K of 128."""
    require_extension()
    _require_cuda(packed_weight, "linear_prepack")
    nbytes = out_features * in_features * bits // 8
    src = packed_weight.contiguous().view(-1)
    if src.dtype != torch.uint8 or src.numel() < nbytes:
        raise RuntimeError("packed_weight is too small for the weight shape")
    dst = torch.empty((nbytes,), dtype=torch.uint8, device=src.device)
    with torch.cuda.device(src.device):
        st = _lib.lib().dimq_linear_prepack(_lib.ptr(src), C.c_int(bits), C.c_int64(out_features),
                                            C.c_int64(in_features), _lib.ptr(dst), _lib.stream_ptr(src.device))
    _lib.check(st, "linear_prepack")
    return dst


def conv_prepack(packed_weight: torch.Tensor, weight_shape: Sequence[int], bits: int = 4) -> torch.Tensor:
    """Indices of a ``[OC, ICg, KH, KW]`` weight re-ordered to ``[OC, KH, KW, ICg]`` (same bit width)."""
    require_extension()
    _require_cuda(packed_weight, "conv_prepack")
    oc, icg, kh, kw = (int(v) for v in weight_shape)
    numel = oc * icg * kh * kw
    src = packed_weight.contiguous().view(-1)
    if src.dtype != torch.uint8 or src.numel() < (numel * bits + 7) // 8:
        raise RuntimeError("packed_weight is too small for the weight shape")
    dst = torch.empty(((numel * bits + 7) // 8,), dtype=torch.uint8, device=src.device)
    with torch.cuda.device(src.device):
        st = _lib.lib().dimq_conv_prepack(_lib.ptr(src), C.c_int(bits), C.c_int64(oc), C.c_int64(icg), C.c_int64(kh),
                                          C.c_int64(kw), _lib.ptr(dst), _lib.stream_ptr(src.device))
    _lib.check(st, "conv_prepack")
    return dst


def im2col(x: torch.Tensor, weight_shape: Sequence[int], stride, padding, dilation=(1, 1), padded_k: int | None = None):
    """Patch matrix ``[B*OH*OW, padded_k]`` of a ``groups == 1`` convolution, columns in (kh, kw, c) order."""
    require_extension()
    _require_cuda(x, "im2col")
    g = _conv_geom(x, weight_shape, _pair(stride), _pair(padding), _pair(dilation), 1)
    k_real = g.kernel_h * g.kernel_w * g.in_channels
    kp = int(padded_k) if padded_k is not None else (k_real + 7) // 8 * 8
    for i in range(4):
        g.x_stride[i] = x.stride(i)
    cols = torch.empty((g.batch * g.out_h * g.out_w, kp), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.lib().dimq_im2col(_lib.ptr(x), _lib.dtype_code(x, "x"), C.byref(g), C.c_int64(kp), _lib.ptr(cols),
                                    _lib.stream_ptr(x.device))
    _lib.check(st, "im2col")
    return cols, (g.out_h, g.out_w)


def max_pool_nhwc(x: torch.Tensor, kernel: int, stride: int, padding: int) -> torch.Tensor:
    """Max-pool of a channels_last 16-bit tensor (logical NCHW in, logical NCHW / channels_last out)."""
    require_extension()
    _require_cuda(x, "max_pool_nhwc")
    if x.dim() != 4 or not x.is_contiguous(memory_format=torch.channels_last):
        raise RuntimeError("max_pool_nhwc expects a channels_last 4-D tensor")
    b, c, h, w = x.shape
    oh = (h + 2 * padding - kernel) // stride + 1
    ow = (w + 2 * padding - kernel) // stride + 1
    y = torch.empty((b, c, oh, ow), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    with torch.cuda.device(x.device):
        st = _lib.lib().dimq_max_pool_nhwc(_lib.ptr(x), _lib.ptr(y), _lib.dtype_code(x, "x"), C.c_int64(b), C.c_int64(h),
                                           C.c_int64(w), C.c_int64(c), C.c_int(kernel), C.c_int(stride),
                                           C.c_int(padding), _lib.stream_ptr(x.device))
    _lib.check(st, "max_pool_nhwc")
    return y


def images_to_nhwc(images: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``images.to(dtype).contiguous(memory_format=torch.channels_last)`` for a contiguous NCHW batch of
    3-channel images (fp32 / fp16 / bf16) in one pass of 16-byte loads and stores."""
    require_extension()
    _require_cuda(images, "images_to_nhwc")
    if images.dim() != 4 or images.shape[1] != 3 or not images.is_contiguous() or (images.shape[2] * images.shape[3]) % 8:
        raise RuntimeError("images_to_nhwc expects a contiguous [B, 3, H, W] tensor with H * W a multiple of 8")
    if dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError("images_to_nhwc writes bf16 or fp16")
    b, _, h, w = images.shape
    y = torch.empty((b, 3, h, w), dtype=dtype, device=images.device, memory_format=torch.channels_last)
    with torch.cuda.device(images.device):
        st = _lib.lib().dimq_images_to_nhwc(_lib.ptr(images), _lib.dtype_code(images, "images"), _lib.ptr(y),
                                            _lib.dtype_code(y, "y"), C.c_int64(b), C.c_int64(h), C.c_int64(w),
                                            _lib.stream_ptr(images.device))
    _lib.check(st, "images_to_nhwc")
    return y


def add_layer_norm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor,
                   eps: float = 1e-6):
    """``(x + delta, LayerNorm(x + delta))`` over the last dimension (``delta=None``: ``(x, LayerNorm(x))``).

    bf16 / fp16 CUDA tensors with a last dimension that is a multiple of 8 and at most 1024.
    """
    require_extension()
    _require_cuda(x, "add_layer_norm")
    cols = x.shape[-1]
    xc = x.contiguous()
    dc = None if delta is None else delta.contiguous()
    if dc is not None and (dc.shape != xc.shape or dc.dtype != xc.dtype):
        raise RuntimeError("delta must match x in shape and dtype")
    w = weight.to(xc.dtype).contiguous()
    b = bias.to(xc.dtype).contiguous()
    if w.numel() != cols or b.numel() != cols:
        raise RuntimeError("weight / bias must have one element per column")
    x_out = torch.empty_like(xc) if dc is not None else xc
    h = torch.empty_like(xc)
    with torch.cuda.device(xc.device):
        st = _lib.lib().dimq_add_layer_norm(_lib.ptr(xc), _lib.ptr(dc), _lib.ptr(w), _lib.ptr(b),
                                            _lib.ptr(x_out) if dc is not None else C.c_void_p(0), _lib.ptr(h),
                                            C.c_int64(xc.numel() // cols), C.c_int64(cols), C.c_float(eps),
                                            _lib.dtype_code(xc, "x"), _lib.stream_ptr(xc.device))
    _lib.check(st, "add_layer_norm")
    return x_out, h


def last_device_status() -> int:
    """Status word left by a tensor-core kernel that gave up a bounded wait (0 = none); clears it."""
    require_extension()
    word = C.c_uint32(0)
    _lib.check(_lib.lib().dimq_last_device_status(C.byref(word)), "last_device_status")
    return int(word.value)
