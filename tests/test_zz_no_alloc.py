"""The allocation-free convolution entry point (dimq_conv2d_wq_static) against dimq_conv2d_wq.

A runtime that owns all device memory, or runs under a fixed budget, cannot give this library a
scratch buffer for the re-ordered weight indices; the static entry point keeps them in an array built
into the library instead.  Both entry points launch the same kernels on the same inputs, so their
outputs must be identical.  Two calls in a row, with different layers, check that the shared array
is rewritten correctly from one call to the next.  This file is collected last on purpose.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

from tests._cases import make_weight

pytestmark = pytest.mark.gpu


def _run_both(ops, _lib, b, c, h, w, oc, k, stride, pad, seed, bits=4):
    cw = make_weight(oc, c * k * k, bits, seed=seed, group_rows=1, std=(2.0 / (c * k * k)) ** 0.5)
    wshape = (oc, c, k, k)
    torch.manual_seed(seed)
    x = torch.relu(torch.randn(b, c, h, w, device="cuda")).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    packed = torch.from_numpy(cw["packed"]).cuda()
    books = torch.from_numpy(cw["codebooks"]).cuda().half()
    bias = torch.randn(oc, device="cuda")
    want = ops.dimq_conv2d_wq(x, packed, books, bias, wshape, (stride, stride), (pad, pad), (1, 1), 1, bits=bits,
                              group_rows=1, out_dtype=torch.bfloat16, epilogue="relu",
                              packed_khwc=ops.conv_prepack(packed, wshape, bits), algo="tcgen05")
    geom = ops._conv_geom(x, wshape, (stride, stride), (pad, pad), (1, 1), 1)
    xc, y = ops._conv_io(x, geom, torch.bfloat16)
    y.fill_(-7.0)
    weight = _lib.WqWeight(packed.data_ptr(), bits, books.data_ptr(), _lib.F16, 1 << bits, oc, 1, 0)
    status = _lib.lib().dimq_conv2d_wq_static(
        _lib.ptr(xc), _lib.BF16, C.byref(weight), _lib.ptr(bias), _lib.F32, C.c_void_p(0), _lib.ptr(y), _lib.BF16,
        C.byref(geom), _lib.EPI_RELU, _lib.stream_ptr(x.device))
    assert status == 0, _lib.lib().dimq_status_string(status).decode()
    torch.cuda.synchronize()
    assert ops.last_device_status() == 0
    assert torch.equal(y, want), float((y.float() - want.float()).abs().max())
    return y


def test_static_entry_point_matches_regular_entry_point_twice(cuda_device):
    from dimq_b200 import _lib, ops

    ops.require_extension()
    first = _run_both(ops, _lib, 3, 64, 28, 28, 128, 3, 1, 1, seed=21)
    second = _run_both(ops, _lib, 2, 128, 14, 14, 64, 3, 2, 1, seed=22)   # another layer reuses the array
    assert first.shape == (3, 128, 28, 28) and second.shape == (2, 64, 7, 7)
    assert np.isfinite(first.float().cpu().numpy()).all() and np.isfinite(second.float().cpu().numpy()).all()


def test_static_entry_point_three_bit_indices(cuda_device):
    """3-bit streams: groups of eight indices straddle bytes in the re-ordered copy as well."""
    from dimq_b200 import _lib, ops

    ops.require_extension()
    out = _run_both(ops, _lib, 2, 64, 20, 20, 64, 3, 1, 1, seed=23, bits=3)
    assert out.shape == (2, 64, 20, 20)
    # a rejected argument (unknown element type) returns before the shared array is touched
    geom = ops._conv_geom(torch.zeros(1, 64, 8, 8, device="cuda"), (64, 64, 3, 3), (1, 1), (1, 1), (1, 1), 1)
    dummy = torch.zeros(64 * 64 * 9, dtype=torch.uint8, device="cuda")
    books = torch.zeros(16, dtype=torch.float16, device="cuda")
    weight = _lib.WqWeight(dummy.data_ptr(), 4, books.data_ptr(), _lib.F16, 16, 1, 64, 0)
    status = _lib.lib().dimq_conv2d_wq_static(_lib.ptr(dummy), 9, C.byref(weight), C.c_void_p(0), 0, C.c_void_p(0),
                                              _lib.ptr(dummy), _lib.BF16, C.byref(geom), 0, _lib.stream_ptr(dummy.device))
    assert status == -3


def test_static_entry_point_limits(cuda_device):
    from dimq_b200 import _lib, ops

    ops.require_extension()
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    books = torch.zeros(16, dtype=torch.float16, device="cuda")
    # 2048 x 2048 x 3 x 3 at 4 bits is an 18 MiB index stream: larger than the built-in 4 MiB
    x = torch.zeros(1, 2048, 8, 8, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    geom = ops._conv_geom(x, (2048, 2048, 3, 3), (1, 1), (1, 1), (1, 1), 1)
    xc, y = ops._conv_io(x, geom, torch.bfloat16)
    weight = _lib.WqWeight(dummy.data_ptr(), 4, books.data_ptr(), _lib.F16, 16, 1, 2048, 0)
    status = _lib.lib().dimq_conv2d_wq_static(_lib.ptr(xc), _lib.BF16, C.byref(weight), C.c_void_p(0), 0,
                                              C.c_void_p(0), _lib.ptr(y), _lib.BF16, C.byref(geom), 0,
                                              _lib.stream_ptr(x.device))
    assert status == -12
    assert "4 MiB" in _lib.lib().dimq_status_string(status).decode()
    # a geometry the tensor-core convolution does not take (3 input channels) is refused, not computed wrongly
    x3 = torch.zeros(1, 3, 8, 8, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    geom3 = ops._conv_geom(x3, (8, 3, 3, 3), (1, 1), (1, 1), (1, 1), 1)
    xc3, y3 = ops._conv_io(x3, geom3, torch.bfloat16)
    weight3 = _lib.WqWeight(dummy.data_ptr(), 4, books.data_ptr(), _lib.F16, 16, 1, 8, 0)
    status = _lib.lib().dimq_conv2d_wq_static(_lib.ptr(xc3), _lib.BF16, C.byref(weight3), C.c_void_p(0), 0,
                                              C.c_void_p(0), _lib.ptr(y3), _lib.BF16, C.byref(geom3), 0,
                                              _lib.stream_ptr(x3.device))
    assert status == -7
