"""dimq_b200 — B200 (sm_100a) backend for DIMQ packed-index inference.

Drop-in for the ``dimq_backend`` package of the DIMQ reference
(dimq_cuda_backend/dimq_backend/__init__.py:21-37): same operator, module and
export names.  The compute runs in hand-written CUDA behind a C ABI
(include/dimq_b200.h); there is no CPU or PyTorch fallback.
"""

from .export import (
    activation_qparams_from_minmax,
    assign_weight_indices,
    default_activation_qparams,
    export_compact_checkpoint,
    export_packed_dimq_checkpoint,
    hard_quantize_weight,
    infer_module_hparams,
    load_compact_checkpoint,
    pack_u4_indices,
    unpack_u4_indices,
)
from .calibration import ActivationRangeCollector, apply_activation_qparams, calibrate_activation_qparams
from .modules import DIMQConv2d, DIMQLinear, make_packed_layer, replace_modules_with_packed_dimq
from .ops import (
    build_product_table,
    dimq_conv2d_lut,
    dimq_conv2d_wq,
    dimq_linear_lut,
    dimq_linear_wq,
    hard_quantize,
    is_available,
    pack_bits,
    pack_u4,
    quantize_activation_u4,
    require_extension,
    unpack_bits,
    unpack_u4,
)

__all__ = [
    "ActivationRangeCollector", "DIMQConv2d", "DIMQLinear", "activation_qparams_from_minmax", "apply_activation_qparams",
    "calibrate_activation_qparams", "assign_weight_indices", "build_product_table",
    "default_activation_qparams", "dimq_conv2d_lut", "dimq_conv2d_wq", "dimq_linear_lut", "dimq_linear_wq",
    "export_compact_checkpoint", "export_packed_dimq_checkpoint", "hard_quantize", "hard_quantize_weight",
    "infer_module_hparams", "is_available", "load_compact_checkpoint", "make_packed_layer", "pack_bits", "pack_u4",
    "pack_u4_indices", "quantize_activation_u4", "replace_modules_with_packed_dimq", "require_extension",
    "unpack_bits", "unpack_u4", "unpack_u4_indices",
]
