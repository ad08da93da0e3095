"""The reference's import surface (``import dimq_backend`` ...) served by this backend, and the
reference's four CUDA tests (dimq_cuda_backend/tests/test_cuda_ops.py:31-93) run through it.

Expected values are the reference's own outputs for the same seeded inputs, stored by
tests/golden/make_golden.py (the reference's PyTorch oracles do not exist in this package)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

REFERENCE_EXPORTS = [   # dimq_cuda_backend/dimq_backend/__init__.py:21-37
    "DIMQConv2d", "DIMQLinear", "activation_qparams_from_minmax", "assign_weight_indices", "build_product_table",
    "default_activation_qparams", "dimq_conv2d_reference", "dimq_linear_reference", "export_packed_dimq_checkpoint",
    "infer_module_hparams", "is_available", "pack_u4_indices", "quantize_activation_u4",
    "replace_modules_with_packed_dimq", "unpack_u4_indices",
]
CPU_ORACLES = {"dimq_conv2d_reference", "dimq_linear_reference"}


def test_import_surface_of_the_reference_package():
    import dimq_b200
    import dimq_backend
    from dimq_backend import export, modules, ops
    from dimq_backend.export import pack_u4_indices, unpack_u4_indices  # noqa: F401
    from dimq_backend.modules import DIMQLinear  # noqa: F401
    from dimq_backend.ops import dimq_conv2d_lut, dimq_linear_lut, is_available  # noqa: F401

    assert ops is dimq_b200.ops and modules is dimq_b200.modules and export is dimq_b200.export
    for name in REFERENCE_EXPORTS:
        if name in CPU_ORACLES:
            assert not hasattr(dimq_backend, name)       # no CPU path in this backend
        else:
            assert getattr(dimq_backend, name) is getattr(dimq_b200, name), name
    assert sorted(dimq_backend.__all__) == sorted(set(REFERENCE_EXPORTS) - CPU_ORACLES)
    # frozen positional signatures of the six ops (dimq_backend/ops.py:36-119)
    import inspect

    def names(fn, n):
        return list(inspect.signature(fn).parameters)[:n]

    assert names(ops.pack_u4, 1) == ["indices"]
    assert names(ops.unpack_u4, 2) == ["packed", "numel"]
    assert names(ops.quantize_activation_u4, 3) == ["x", "act_scale", "act_zero_point"]
    assert names(ops.build_product_table, 3) == ["codebook", "act_scale", "act_zero_point"]
    assert names(ops.dimq_linear_lut, 8) == ["x", "packed_weight", "codebook", "act_scale", "act_zero_point", "bias",
                                              "out_features", "in_features"]
    assert names(ops.dimq_conv2d_lut, 11) == ["x", "packed_weight", "codebook", "act_scale", "act_zero_point", "bias",
                                               "weight_shape", "stride", "padding", "dilation", "groups"]


def test_cpu_tensors_are_refused_like_the_reference():
    """The reference registers its ops for the CUDA dispatch key only (csrc/dimq_ops.cpp:46-53): a CPU
    tensor raises instead of running some fallback."""
    from dimq_backend import ops

    if not ops.is_available():
        pytest.skip("library not built")
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.pack_u4(torch.zeros(4, dtype=torch.uint8))


@pytest.fixture()
def cuda_backend(cuda_device):
    from dimq_backend import ops

    ops.require_extension()
    return ops


@pytest.mark.gpu
def test_cuda_pack_unpack_matches_python(cuda_backend, golden):
    from dimq_backend.export import pack_u4_indices

    indices = (torch.arange(257, dtype=torch.uint8, device="cuda") * 7) % 16
    packed_cuda = cuda_backend.pack_u4(indices)
    restored = cuda_backend.unpack_u4(packed_cuda, indices.numel())
    packed_py = pack_u4_indices(indices.cpu()).cuda()
    torch.testing.assert_close(packed_cuda, packed_py)
    torch.testing.assert_close(restored, indices)
    assert np.array_equal(packed_cuda.cpu().numpy(), golden["pack_arange257x7_packed"])


@pytest.mark.gpu
def test_cuda_product_table_matches_reference(cuda_backend, golden):
    codebook = torch.linspace(-1.0, 1.0, 16, device="cuda", dtype=torch.float16)
    assert np.array_equal(codebook.float().cpu().numpy(), golden["pt_cb_f16_as_f32"])
    table = cuda_backend.build_product_table(codebook, 0.125, 8)
    torch.testing.assert_close(table.cpu(), torch.from_numpy(golden["pt_table_f16"]), rtol=1e-3, atol=1e-4)


@pytest.mark.gpu
def test_cuda_linear_lut_matches_reference(cuda_backend, golden):
    y = cuda_backend.dimq_linear_lut(torch.from_numpy(golden["lin_x"]).cuda(), torch.from_numpy(golden["lin_packed"]).cuda(),
                                     torch.from_numpy(golden["lin_cb"]).cuda(), 0.2, 7,
                                     torch.from_numpy(golden["lin_bias"]).cuda(), 6, 11)
    torch.testing.assert_close(y.cpu(), torch.from_numpy(golden["lin_y_lut"]), rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
def test_cuda_conv2d_lut_matches_reference(cuda_backend, golden):
    y = cuda_backend.dimq_conv2d_lut(torch.from_numpy(golden["conv_x"]).cuda(), torch.from_numpy(golden["conv_packed"]).cuda(),
                                     torch.from_numpy(golden["conv_cb"]).cuda(), 0.25, 7,
                                     torch.from_numpy(golden["conv_bias"]).cuda(), (5, 3, 3, 3), (2, 1), (1, 1), (1, 1), 1)
    torch.testing.assert_close(y.cpu(), torch.from_numpy(golden["conv_y_lut"]), rtol=1e-5, atol=1e-5)
