"""``dimq_backend`` import path of the DIMQ reference, served by the B200 backend.

Code written against the reference's packed-index backend imports ``dimq_backend``,
``dimq_backend.ops``, ``dimq_backend.modules`` and ``dimq_backend.export``
(dimq_cuda_backend/dimq_backend/__init__.py:3-37, dimq_cuda_backend/tests/test_cuda_ops.py:22-28).
This package makes those imports resolve to :mod:`dimq_b200`: the three submodules ARE the
``dimq_b200`` ones, and the package exports the reference's names.

Two names of the reference package are left out on purpose: ``dimq_linear_reference`` and
``dimq_conv2d_reference`` are its slow pure-PyTorch CPU oracles (``dimq_backend/reference.py``), and
this backend has no CPU path.  ``build_product_table`` and ``quantize_activation_u4`` are the CUDA
ops here (in the reference package root they are the PyTorch oracle versions, ``__init__.py:14-19``;
its CUDA ones live in ``dimq_backend.ops``, as they also do here).
"""

import sys

from dimq_b200 import export, modules, ops
from dimq_b200 import (
    DIMQConv2d,
    DIMQLinear,
    activation_qparams_from_minmax,
    assign_weight_indices,
    build_product_table,
    default_activation_qparams,
    export_packed_dimq_checkpoint,
    infer_module_hparams,
    is_available,
    pack_u4_indices,
    quantize_activation_u4,
    replace_modules_with_packed_dimq,
    unpack_u4_indices,
)

for _name, _module in (("ops", ops), ("modules", modules), ("export", export)):
    sys.modules[f"{__name__}.{_name}"] = _module

__all__ = [
    "DIMQConv2d",
    "DIMQLinear",
    "activation_qparams_from_minmax",
    "assign_weight_indices",
    "build_product_table",
    "default_activation_qparams",
    "export_packed_dimq_checkpoint",
    "infer_module_hparams",
    "is_available",
    "pack_u4_indices",
    "quantize_activation_u4",
    "replace_modules_with_packed_dimq",
    "unpack_u4_indices",
]
