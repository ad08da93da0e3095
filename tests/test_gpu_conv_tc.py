"""GPU parity of the tensor-core (implicit-GEMM) weight-only convolution against the CPU oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import dimq_oracle as o
from tests._cases import bf16_round, make_weight

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda_device):
    from dimq_b200 import ops as _ops

    _ops.require_extension()
    return _ops


def _cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_conv_prepack_is_a_transposition(ops, bits):
    oc, icg, kh, kw = 5, 64, 3, 2
    idx = np.random.default_rng(bits).integers(0, 1 << bits, size=(oc, icg, kh, kw), dtype=np.uint8)
    got = ops.conv_prepack(_cuda(o.pack_bits(idx, bits)), idx.shape, bits)
    want = o.pack_bits(idx.transpose(0, 2, 3, 1), bits)
    assert np.array_equal(got.cpu().numpy(), want)


CASES = [
    # batch, C, H, W, OC, k, stride, pad, dilation
    (4, 64, 56, 56, 64, 3, 1, 1, 1),     # config 2 geometry at a smaller batch
    (3, 64, 56, 56, 128, 3, 2, 1, 1),    # stride-2 3x3
    (3, 64, 56, 56, 128, 1, 2, 0, 1),    # 1x1 stride-2 downsample
    (2, 128, 28, 28, 128, 3, 1, 1, 1),
    (5, 128, 14, 14, 192, 3, 1, 1, 1),
    (6, 128, 7, 7, 130, 3, 1, 1, 1),     # OC not a multiple of the 128-row tile
    (2, 64, 13, 9, 64, 3, 2, 1, 1),      # odd sizes with stride 2
    (2, 64, 12, 10, 64, 3, 1, 2, 2),     # dilation 2
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mode", ["per_channel_fp16cb", "per_layer_bf16cb"])
def test_conv2d_wq_tcgen05(ops, case, mode):
    b, c, h, w, oc, k, s, pad, dil = case
    rng = np.random.default_rng(hash(case) % 1000)
    if mode == "per_channel_fp16cb":
        cw = make_weight(oc, c * k * k, 4, seed=7, group_rows=1, std=(2.0 / (c * k * k)) ** 0.5)
        grp, cb_t = 1, torch.float16
    else:
        cw = make_weight(oc, c * k * k, 4, seed=8, group_rows=None, std=(2.0 / (c * k * k)) ** 0.5, cb_dtype="bf16")
        grp, cb_t = None, torch.bfloat16
    x = bf16_round(np.maximum(rng.standard_normal((b, c, h, w)).astype(np.float32), 0))
    bias = rng.standard_normal(oc).astype(np.float32)
    wshape = (oc, c, k, k)
    want = o.conv2d_wq(x, cw["packed"], cw["codebooks"], 4, wshape, bias, stride=(s, s), padding=(pad, pad),
                       dilation=(dil, dil), group_rows=cw["group_rows"])
    packed = _cuda(cw["packed"])
    khwc = ops.conv_prepack(packed, wshape, 4)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    got = ops.dimq_conv2d_wq(x_cl, packed, _cuda(cw["codebooks"], cb_t), _cuda(bias), wshape, (s, s), (pad, pad),
                             (dil, dil), 1, bits=4, group_rows=grp, packed_khwc=khwc, algo="tcgen05")
    assert ops.last_device_status() == 0
    assert got.is_contiguous(memory_format=torch.channels_last) and got.dtype == torch.float32
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= 1e-2 and rel <= 1e-3, (case, mode, max_abs, rel)
    # the direct kernel agrees too (same inputs, generic path)
    ref = ops.dimq_conv2d_wq(x_cl, packed, _cuda(cw["codebooks"], cb_t), _cuda(bias), wshape, (s, s), (pad, pad),
                             (dil, dil), 1, bits=4, group_rows=grp, algo="generic")
    max_abs, rel = o.parity_metrics(ref.cpu().numpy(), want)
    assert max_abs <= 1e-2 and rel <= 1e-3


def test_conv2d_wq_tcgen05_residual_relu_bf16_out(ops):
    b, c, h, w, oc = 4, 64, 28, 28, 64
    rng = np.random.default_rng(3)
    cw = make_weight(oc, c * 9, 4, seed=5, std=(2.0 / (c * 9)) ** 0.5, cb_dtype="bf16")
    x = bf16_round(np.maximum(rng.standard_normal((b, c, h, w)).astype(np.float32), 0))
    res = bf16_round(rng.standard_normal((b, oc, h, w)).astype(np.float32))
    bias = rng.standard_normal(oc).astype(np.float32)
    lin = o.conv2d_wq(x, cw["packed"], cw["codebooks"], 4, (oc, c, 3, 3), bias, stride=(1, 1), padding=(1, 1))
    packed = _cuda(cw["packed"])
    khwc = ops.conv_prepack(packed, (oc, c, 3, 3), 4)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    r_cl = _cuda(res, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    for epi, want in (("add_relu", np.maximum(lin + res, 0)), ("relu", np.maximum(lin, 0) + res)):
        got = ops.dimq_conv2d_wq(x_cl, packed, _cuda(cw["codebooks"], torch.bfloat16), _cuda(bias), (oc, c, 3, 3),
                                 (1, 1), (1, 1), (1, 1), 1, bits=4, out_dtype=torch.bfloat16, epilogue=epi,
                                 residual=r_cl, packed_khwc=khwc)
        assert got.dtype == torch.bfloat16
        max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
        assert max_abs <= 3e-2 and rel <= 4e-3, (epi, max_abs, rel)   # bf16 output rounding included
    assert ops.last_device_status() == 0


def test_conv_module_uses_tensor_core_path(ops):
    from dimq_b200.modules import DIMQConv2d

    oc, c = 64, 64
    cw = make_weight(oc, c * 9, 4, seed=11, group_rows=1, std=(2.0 / (c * 9)) ** 0.5)
    layer = DIMQConv2d(torch.from_numpy(cw["packed"]), torch.from_numpy(cw["codebooks"]).half(), None, None,
                       (oc, c, 3, 3), None, stride=1, padding=1, bits=4, group_rows=1, out_dtype=torch.bfloat16,
                       epilogue="relu").cuda()
    x = torch.relu(torch.randn(2, c, 56, 56, device="cuda")).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = layer(x)
    want = np.maximum(o.conv2d_wq(x.float().cpu().numpy(), cw["packed"], cw["codebooks"], 4, (oc, c, 3, 3), None,
                                  stride=(1, 1), padding=(1, 1), group_rows=1), 0)
    max_abs, rel = o.parity_metrics(y.float().cpu().numpy(), want)
    assert max_abs <= 3e-2 and rel <= 4e-3
    assert layer._khwc is not None and ops.last_device_status() == 0
