"""Activation calibration and the W4A4 whole model: ranges collected by hooks, u4 parameters from the
reference's formula (dimq_backend/export.py:81-111), the calibrated ResNet-18 against the oracle that
quantises activations the way dimq_conv2d_reference does (dimq_backend/reference.py:113-144)."""

from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import dimq_oracle as o

pytestmark = pytest.mark.gpu

# Twice the values measured on a B200 (3.8e-2 and 4.5e-2, argmax 16/16; the test prints them).  A 4-bit
# activation quantiser amplifies rounding noise: an activation within rounding distance (2^-9 relative, bf16
# storage and summation order) of a step boundary takes the neighbouring code, one fifteenth of the range
# away, and a few percent of the activations of every layer sit that close.  Layer by layer, on identical
# inputs, the W4A4 form holds 1e-2 / 1e-3 (test_w4a4_module_matches_exact_kernel_and_caches_its_state).
W4A4_REL_BF16, W4A4_REL_FP32, W4A4_ARGMAX = 8.0e-2, 9.0e-2, 0.75


def test_collector_ranges_and_formula(cuda_device):
    from dimq_b200 import ActivationRangeCollector, activation_qparams_from_minmax, calibrate_activation_qparams

    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 8)).cuda()
    batches = [torch.randn(5, 16, device="cuda") for _ in range(3)]
    with ActivationRangeCollector(net) as col:
        for b in batches:
            net(b)
        ranges = col.ranges()
    allx = torch.cat(batches)
    assert set(ranges) == {"0", "2"}
    assert ranges["0"] == (float(allx.min()), float(allx.max()))
    hidden = torch.relu(net[0](allx)).detach()
    assert ranges["2"] == pytest.approx((float(hidden.min()), float(hidden.max())))
    q = calibrate_activation_qparams(net, batches)
    want = activation_qparams_from_minmax(*ranges["0"])
    assert q["0"]["scale"] == want["scale"] and q["0"]["zero_point"] == want["zero_point"]
    assert q["0"]["source"] == "calibrated_minmax" and 0 <= q["2"]["zero_point"] <= 15
    # the reference's formula on a few ranges (export.py:81-111): scale = (max - min) / 15, zp = round(-min / scale)
    assert activation_qparams_from_minmax(0.0, 15.0)["scale"] == 1.0
    assert activation_qparams_from_minmax(-8.0, 7.0)["zero_point"] == 8
    assert activation_qparams_from_minmax(3.0, 3.0) == {**activation_qparams_from_minmax(3.0, 3.0), "scale": 1.0, "zero_point": 0}


def test_w4a4_module_matches_exact_kernel_and_caches_its_state(cuda_device, monkeypatch):
    """The cached tensor-core W4A4 form of the modules against the exact product-table kernel, and no
    index re-order after the first forward."""
    from dimq_b200 import ops
    from dimq_b200.modules import DIMQConv2d
    from tests._cases import make_weight

    oc, c = 64, 64
    cw = make_weight(oc, c * 9, 4, seed=11, std=(2.0 / (c * 9)) ** 0.5)
    rng = np.random.default_rng(1)
    x = np.maximum(rng.standard_normal((4, c, 28, 28)).astype(np.float32), 0)
    bias = rng.standard_normal(oc).astype(np.float32)
    scale, zp = float(x.max()) / 15.0, 0
    mod = DIMQConv2d(torch.from_numpy(cw["packed"]), torch.from_numpy(cw["codebooks"]).reshape(-1).half(), scale, zp,
                     (oc, c, 3, 3), torch.from_numpy(bias), stride=1, padding=1).cuda()
    x_cl = torch.from_numpy(x).cuda().contiguous(memory_format=torch.channels_last)
    calls = []
    real = ops.conv_prepack
    monkeypatch.setattr(ops, "conv_prepack", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    got = mod(x_cl)
    assert len(calls) == 1 and got.dtype == torch.float32
    got2 = mod(x_cl)
    assert len(calls) == 1 and torch.equal(got, got2)                  # cached: no second re-order
    want = o.conv2d_lut_a4(x, cw["packed"], cw["codebooks"].reshape(-1), scale, zp, (oc, c, 3, 3), bias,
                           stride=(1, 1), padding=(1, 1))
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= 1e-2 and rel <= 1e-3, (max_abs, rel)
    assert ops.last_device_status() == 0


def test_calibrated_w4a4_resnet18_matches_oracle(cuda_device, monkeypatch):
    from dimq_b200 import _lib, ops
    from dimq_b200.workloads import DIMQResNet18, build_resnet18_checkpoint
    from oracle.models_oracle import ResNet18Oracle

    ckpt = build_resnet18_checkpoint(seed=4, device=cuda_device)
    model = DIMQResNet18(ckpt).to(cuda_device).eval()
    gen = torch.Generator().manual_seed(21)
    calib = [torch.randn(8, 3, 224, 224, generator=gen).to(torch.bfloat16).cuda() for _ in range(2)]
    qparams = model.calibrate(calib)
    assert len(qparams) == 19 and all(q["scale"] > 0 for q in qparams.values())
    assert model.set_activation_qparams(qparams) == 19
    images = torch.randn(16, 3, 224, 224, generator=gen).to(torch.bfloat16)
    calls = []
    real = ops.conv_prepack
    monkeypatch.setattr(ops, "conv_prepack", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    with torch.no_grad():
        model(images.cuda())                      # the weight-only calibration run already built the re-ordered indices
        before = _lib.LAUNCH_COUNT[0]
        got = model(images.cuda()).float().cpu().numpy()
        per_forward = _lib.LAUNCH_COUNT[0] - before
        model(images.cuda())
        again = _lib.LAUNCH_COUNT[0] - before - per_forward
    assert calls == []                            # no per-forward index re-order
    # every forward launches the same kernels: per 4-bit convolution the activation codes, the weight
    # expansion (layers with at least 1024 output pixels) and the convolution - and nothing else
    assert per_forward == again and per_forward <= 3 + 1 + 19 * 3 + 1, (per_forward, again)
    cpu = {"config": None, "layers": {k: {kk: (vv.cpu() if hasattr(vv, "cpu") else vv) for kk, vv in v.items()}
                                      for k, v in ckpt["layers"].items()}, "non_quantized_state_dict": {}}
    want_b = ResNet18Oracle(cpu, round_dtype=torch.bfloat16, act_qparams=qparams).forward(images).numpy()
    want_f = ResNet18Oracle(cpu, act_qparams=qparams).forward(images).numpy()
    abs_b, rel_b = o.parity_metrics(got, want_b)
    abs_f, rel_f = o.parity_metrics(got, want_f)
    agree = float((got.argmax(1) == want_f.argmax(1)).mean())
    print(f"W4A4 ResNet-18, 16 images: vs bf16-rounding oracle max_abs={abs_b:.3e} rel_l2={rel_b:.3e}; "
          f"vs fp32 oracle max_abs={abs_f:.3e} rel_l2={rel_f:.3e}; argmax agreement {agree:.3f}")
    assert rel_b <= W4A4_REL_BF16 and rel_f <= W4A4_REL_FP32 and agree >= W4A4_ARGMAX
    assert ops.last_device_status() == 0
