"""Runtime modules for packed DIMQ layers — drop-ins for ``dimq_backend.modules``.

Constructor and ``from_export_layer`` signatures follow
dimq_cuda_backend/dimq_backend/modules.py:14-150.  Differences, all additive:

* ``act_scale=None`` selects the weight-only mode (activations stay in floating
  point; ``y = x @ codebook[idx].T + bias``) instead of the W4A4 product-table mode;
* ``bits`` / ``group_rows`` describe 2-, 3-, 4- or 8-bit indices and one codebook per
  ``group_rows`` output rows (``codebook`` is then ``[G, K]``);
* ``out_dtype`` / ``epilogue`` choose the output type and a fused ReLU / GELU.

There is no Python fallback: inputs must be CUDA tensors and the compiled library
must be present, otherwise ``forward`` raises.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch
import torch.nn as nn

from . import ops


def _pair(value) -> tuple[int, int]:
    if isinstance(value, int):
        return int(value), int(value)
    if len(value) != 2:
        raise ValueError(f"expected pair, got {value!r}")
    return int(value[0]), int(value[1])


class _PackedBase(nn.Module):
    def _init_common(self, packed_weight, codebook, act_scale, act_zero_point, bias, use_cuda_kernel, bits,
                     group_rows, out_dtype, epilogue):
        self.register_buffer("packed_weight", packed_weight.contiguous().to(torch.uint8))
        self.register_buffer("codebook", codebook.contiguous())
        self.register_buffer("bias", None if bias is None else bias.contiguous())
        self.act_scale = None if act_scale is None else float(act_scale)
        self.act_zero_point = int(act_zero_point) if act_zero_point is not None else 0
        self.use_cuda_kernel = bool(use_cuda_kernel)
        self.bits = int(bits)
        self.group_rows = None if group_rows is None else int(group_rows)
        self.out_dtype = out_dtype
        self.epilogue = epilogue
        if self.act_scale is not None and (self.bits != 4 or codebook.numel() != 16):
            raise ValueError("the W4A4 mode needs 4-bit indices and one 16-entry codebook; "
                             "pass act_scale=None for weight-only layers")

    def _scaled_codebook(self) -> torch.Tensor:
        """``act_scale * codebook`` in fp32 (the weight operand of the tensor-core W4A4 form), built once
        and rebuilt when the codebook buffer or the scale changes."""
        cb = self.codebook
        key = (cb.data_ptr(), cb._version, cb.device, self.act_scale)
        if getattr(self, "_scaled_cb_key", None) != key:
            self._scaled_cb = cb.detach().float().reshape(-1) * torch.tensor(self.act_scale, dtype=torch.float32,
                                                                               device=cb.device)
            self._scaled_cb_key = key
        return self._scaled_cb

    def _check_input(self, x: torch.Tensor) -> None:
        if not self.use_cuda_kernel:
            raise RuntimeError("dimq_b200 has no Python fallback path (use_cuda_kernel=False is not supported)")
        if not (x.is_cuda and self.packed_weight.is_cuda):
            raise RuntimeError("dimq_b200 layers run on CUDA tensors only; move the module and its input to a B200")
        ops.require_extension()


class DIMQLinear(_PackedBase):
    """Linear layer backed by packed weight indices and a learned codebook."""

    def __init__(self, packed_weight, codebook, act_scale, act_zero_point, out_features, in_features, bias=None, *,
                 use_cuda_kernel: bool = True, bits: int = 4, group_rows: int | None = None,
                 out_dtype: torch.dtype | None = None, epilogue: str | None = None) -> None:
        super().__init__()
        self._init_common(packed_weight, codebook, act_scale, act_zero_point, bias, use_cuda_kernel, bits,
                          group_rows, out_dtype, epilogue)
        self.out_features = int(out_features)
        self.in_features = int(in_features)
        # indices re-ordered for the small-M kernel: built the first time a call with at most 16 activation
        # rows meets a weight that kernel takes (a second copy of the indices), rebuilt whenever the
        # packed_weight buffer is replaced, moved or written in place
        self._tiled = None
        self._tiled_key = None

    def _prepacked(self, rows: int, x: torch.Tensor) -> torch.Tensor | None:
        if (rows > 16 or self.bits not in (2, 3, 4) or self.out_features % 16 != 0 or self.in_features % 128 != 0
                or self.in_features < 2048
                or x.dtype not in (torch.float16, torch.bfloat16)
                or self.out_features * self.in_features * self.bits < (1 << 24)):
            return None
        pw = self.packed_weight
        key = (pw.data_ptr(), pw._version, pw.device)
        if self._tiled is None or self._tiled_key != key:
            self._tiled = ops.linear_prepack(pw, self.out_features, self.in_features, self.bits)
            self._tiled_key = key
        return self._tiled

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        self._check_input(x)
        if self.act_scale is None:
            tiled = self._prepacked(x.numel() // self.in_features, x)
            return ops.dimq_linear_wq(x, self.packed_weight, self.codebook, self.bias, self.out_features,
                                      self.in_features, bits=self.bits, group_rows=self.group_rows,
                                      out_dtype=self.out_dtype, epilogue=self.epilogue, residual=residual,
                                      packed_tiled=tiled)
        rows = x.numel() // self.in_features
        if rows >= ops.A4_TC_MIN_ROWS and self.in_features % 64 == 0:
            # many rows: centred activation codes (exact in bf16) times the scaled codebook through the
            # weight-only tensor-core path; per-layer state is cached, nothing is re-derived per call
            codes = ops.centre_quantize_u4(x, self.act_scale, self.act_zero_point)
            return ops.dimq_linear_wq(codes, self.packed_weight, self._scaled_codebook(), self.bias,
                                      self.out_features, self.in_features, bits=4, out_dtype=self.out_dtype,
                                      epilogue=self.epilogue, residual=residual)
        if residual is not None or self.epilogue is not None:
            raise RuntimeError("a fused epilogue or residual needs the weight-only mode or at least "
                               f"{ops.A4_TC_MIN_ROWS} activation rows")
        return ops.dimq_linear_lut(x, self.packed_weight, self.codebook, self.act_scale, self.act_zero_point,
                                   self.bias, self.out_features, self.in_features)

    @classmethod
    def from_export_layer(cls, layer: Mapping[str, Any], *, use_cuda_kernel: bool = True, **extra) -> "DIMQLinear":
        return cls(layer["packed_weight"], layer["codebook"], layer.get("act_scale"), layer.get("act_zero_point"),
                   layer["out_features"], layer["in_features"], layer.get("bias"), use_cuda_kernel=use_cuda_kernel,
                   bits=layer.get("bit_w", 4), group_rows=layer.get("group_rows"), **extra)

    def extra_repr(self) -> str:
        mode = "weight-only" if self.act_scale is None else "W4A4"
        return f"{self.in_features} -> {self.out_features}, bits={self.bits}, mode={mode}"


class DIMQConv2d(_PackedBase):
    """Conv2d layer backed by packed weight indices and a learned codebook."""

    def __init__(self, packed_weight, codebook, act_scale, act_zero_point, weight_shape, bias=None, *, stride=1,
                 padding=0, dilation=1, groups: int = 1, use_cuda_kernel: bool = True, bits: int = 4,
                 group_rows: int | None = None, out_dtype: torch.dtype | None = None,
                 epilogue: str | None = None) -> None:
        super().__init__()
        self._init_common(packed_weight, codebook, act_scale, act_zero_point, bias, use_cuda_kernel, bits,
                          group_rows, out_dtype, epilogue)
        self.weight_shape = tuple(int(v) for v in weight_shape)
        self.stride = _pair(stride)
        self.padding = _pair(padding)
        self.dilation = _pair(dilation)
        self.groups = int(groups)
        # indices re-ordered for the tensor-core conv: built on first use on the GPU and rebuilt
        # whenever the packed_weight buffer is replaced, moved or written in place
        self._khwc = None
        self._khwc_key = None

    def _prepacked(self) -> torch.Tensor | None:
        if self.groups != 1 or self.weight_shape[1] % 64 != 0:
            return None
        pw = self.packed_weight
        key = (pw.data_ptr(), pw._version, pw.device)
        if self._khwc is None or self._khwc_key != key:
            self._khwc = ops.conv_prepack(pw, self.weight_shape, self.bits)
            self._khwc_key = key
        return self._khwc

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        self._check_input(x)
        if self.act_scale is None:
            return ops.dimq_conv2d_wq(x, self.packed_weight, self.codebook, self.bias, self.weight_shape,
                                      self.stride, self.padding, self.dilation, self.groups, bits=self.bits,
                                      group_rows=self.group_rows, out_dtype=self.out_dtype, epilogue=self.epilogue,
                                      residual=residual, packed_khwc=self._prepacked())
        khwc = self._prepacked()
        channels_last = x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous()
        if khwc is not None and channels_last and self.stride[0] == self.stride[1] and self.stride[0] in (1, 2):
            oh = (x.shape[2] + 2 * self.padding[0] - self.dilation[0] * (self.weight_shape[2] - 1) - 1) // self.stride[0] + 1
            ow = (x.shape[3] + 2 * self.padding[1] - self.dilation[1] * (self.weight_shape[3] - 1) - 1) // self.stride[1] + 1
            if x.shape[0] * oh * ow >= ops.A4_TC_MIN_ROWS:
                # many output pixels: centred activation codes times the scaled codebook through the
                # weight-only implicit-GEMM path, with the re-ordered indices and the scaled codebook
                # cached on the module (no per-call index re-order)
                codes = ops.centre_quantize_u4(x, self.act_scale, self.act_zero_point)
                return ops.dimq_conv2d_wq(codes, self.packed_weight, self._scaled_codebook(), self.bias,
                                          self.weight_shape, self.stride, self.padding, self.dilation, self.groups,
                                          bits=4, out_dtype=self.out_dtype, epilogue=self.epilogue, residual=residual,
                                          packed_khwc=khwc)
        if residual is not None or self.epilogue is not None:
            raise RuntimeError("a fused epilogue or residual needs the weight-only mode, or channels_last input "
                               f"with at least {ops.A4_TC_MIN_ROWS} output pixels")
        return ops.dimq_conv2d_lut(x, self.packed_weight, self.codebook, self.act_scale, self.act_zero_point,
                                   self.bias, self.weight_shape, self.stride, self.padding, self.dilation,
                                   self.groups)

    @classmethod
    def from_export_layer(cls, layer: Mapping[str, Any], *, use_cuda_kernel: bool = True, **extra) -> "DIMQConv2d":
        return cls(layer["packed_weight"], layer["codebook"], layer.get("act_scale"), layer.get("act_zero_point"),
                   layer["weight_shape"], layer.get("bias"), stride=layer.get("stride", (1, 1)),
                   padding=layer.get("padding", (0, 0)), dilation=layer.get("dilation", (1, 1)),
                   groups=layer.get("groups", 1), use_cuda_kernel=use_cuda_kernel, bits=layer.get("bit_w", 4),
                   group_rows=layer.get("group_rows"), **extra)

    def extra_repr(self) -> str:
        mode = "weight-only" if self.act_scale is None else "W4A4"
        return f"weight_shape={self.weight_shape}, stride={self.stride}, bits={self.bits}, mode={mode}"


def make_packed_layer(layer: Mapping[str, Any], *, use_cuda_kernel: bool = True, **extra) -> nn.Module:
    if layer["type"] == "linear":
        return DIMQLinear.from_export_layer(layer, use_cuda_kernel=use_cuda_kernel, **extra)
    if layer["type"] == "conv2d":
        return DIMQConv2d.from_export_layer(layer, use_cuda_kernel=use_cuda_kernel, **extra)
    raise ValueError(f"unsupported packed DIMQ layer type {layer['type']!r}")


def replace_modules_with_packed_dimq(model: nn.Module, packed_state: Mapping[str, Any], *,
                                     use_cuda_kernel: bool = True, **extra) -> nn.Module:
    """Replace matching modules in ``model`` with packed DIMQ runtime layers
    (dimq_backend/modules.py:161-172).  As in the reference, the non-quantised
    tensors of the checkpoint are not loaded here."""
    for name, layer in packed_state["layers"].items():
        parts = name.split(".")
        parent = model
        for part in parts[:-1]:
            parent = parent._modules[part]
        parent._modules[parts[-1]] = make_packed_layer(layer, use_cuda_kernel=use_cuda_kernel, **extra)
    return model
