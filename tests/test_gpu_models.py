"""Whole-model parity: the packed DIMQ ViT on the GPU against the CPU oracle (dequantised
weights, PyTorch CPU ops).

The GPU path keeps activations in bf16, so it is compared (a) with an oracle that rounds its
activations to bf16 at the same points — the tolerance below covers the remaining difference in
accumulation order and in the bf16 attention kernel — and (b) layer by layer at the strict
max-abs 1e-2 / relative-L2 1e-3 of the LUT-GEMM contract.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import dimq_oracle as o

pytestmark = pytest.mark.gpu

# Whole-model thresholds: at most twice the values measured on a B200, which the tests print.
# ViT-B/16, 12 layers, 16 images: 1.02e-2 against the oracle that rounds to bf16 at the same points
# (1.17e-2 with GELU / residual as separate kernels), 8.96e-3 against the fp32 oracle, argmax 16/16.
# ResNet-18, 16 images: 2.1e-3 (2.3e-3 unfused) and 2.0e-3, argmax 16/16.
VIT_REL_BF16, VIT_REL_FP32, VIT_ARGMAX = 2.0e-2, 1.8e-2, 0.9
RESNET_REL_BF16, RESNET_REL_FP32, RESNET_ARGMAX = 4.5e-3, 4.0e-3, 0.9


@pytest.fixture(scope="module")
def vit(cuda_device):
    from dimq_b200.workloads import DIMQViT, build_vit_b16_checkpoint

    ckpt = build_vit_b16_checkpoint(seed=3, device=cuda_device)   # all 12 layers
    return ckpt, DIMQViT(ckpt).to(cuda_device).eval()


def test_vit_export_is_bit_exact(vit):
    """Indices assigned and packed on the GPU while building the model equal the CPU oracle's."""
    from oracle import c_oracle

    ckpt, _ = vit
    layer = ckpt["layers"]["blocks.0.mlp.fc1"]
    # rebuild the float weight the builder drew: same generator order is not needed — the packed
    # stream must decode, with the stored codebooks, to values that are nearest-codeword consistent
    idx = o.unpack_bits(layer["packed_weight"].cpu().numpy(), 3072 * 768, 3).reshape(3072, 768)
    books = layer["codebook"].float().cpu().numpy()
    w_hat = o.dequantize(idx, books, 128)
    # idempotence: hard-quantising the dequantised weight gives the same indices back
    again = c_oracle.hard_quantize(w_hat, books, 128)
    assert np.array_equal(again, idx)
    assert idx.max() < 8 and books.shape == (24, 8)


def test_vit_layers_match_oracle_strictly(vit):
    from oracle.models_oracle import dequantize_layer

    ckpt, model = vit
    torch.manual_seed(0)
    for name in ("blocks.0.attn.qkv", "blocks.5.attn.proj", "blocks.11.mlp.fc1", "blocks.1.mlp.fc2", "head"):
        layer = ckpt["layers"][name]
        k = layer["in_features"]
        x = torch.randn(300, k).to(torch.bfloat16)
        want = torch.nn.functional.linear(x.float(), dequantize_layer(layer), layer["bias"].float().cpu()).numpy()
        mod = model.q[name.replace(".", "__")]
        from dimq_b200 import ops
        got = ops.dimq_linear_wq(x.cuda(), mod.packed_weight, mod.codebook, mod.bias, mod.out_features, k, bits=3,
                                 group_rows=128)
        max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
        assert max_abs <= 1e-2 and rel <= 1e-3, (name, max_abs, rel)


def test_vit_forward_matches_cpu_oracle(vit):
    from oracle.models_oracle import ViTOracle

    ckpt, model = vit
    n_img = 16
    images = torch.randn(n_img, 3, 224, 224, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    with torch.no_grad():
        got = model(images.cuda()).float().cpu().numpy()
    cpu_ckpt = {"config": ckpt["config"],
                "layers": {k: {kk: (vv.cpu() if hasattr(vv, "cpu") else vv) for kk, vv in v.items()}
                           for k, v in ckpt["layers"].items()},
                "non_quantized_state_dict": {k: v.cpu() for k, v in ckpt["non_quantized_state_dict"].items()}}
    want_bf16 = ViTOracle(cpu_ckpt, round_dtype=torch.bfloat16).forward(images).numpy()
    want_fp32 = ViTOracle(cpu_ckpt).forward(images).numpy()
    assert got.shape == (n_img, 1000)
    abs_b, rel_b = o.parity_metrics(got, want_bf16)
    abs_f, rel_f = o.parity_metrics(got, want_fp32)
    agree = float((got.argmax(1) == want_fp32.argmax(1)).mean())
    print(f"ViT-B/16, 12 layers, {n_img} images: vs bf16-rounding oracle max_abs={abs_b:.3e} rel_l2={rel_b:.3e}; "
          f"vs fp32 oracle max_abs={abs_f:.3e} rel_l2={rel_f:.3e}; argmax agreement {agree:.3f}")
    # bf16 activations: every stored activation carries 2^-9 rounding, which 12 layers compound; the
    # thresholds are twice the measured values (printed above), the strict 1e-2 / 1e-3 bar is held
    # layer by layer in test_vit_layers_match_oracle_strictly and at full size in test_gpu_expand_gemm.py
    assert rel_b <= VIT_REL_BF16, rel_b
    assert rel_f <= VIT_REL_FP32, rel_f
    assert agree >= VIT_ARGMAX
    # the variant with GELU and the residual add as separate kernels computes the same thing
    from dimq_b200.workloads import DIMQViT

    fused = DIMQViT(ckpt, fuse_epilogues=False).to("cuda").eval()
    with torch.no_grad():
        got_fused = fused(images.cuda()).float().cpu().numpy()
    _, rel_fused = o.parity_metrics(got_fused, want_bf16)
    print(f"  unfused variant vs bf16-rounding oracle rel_l2={rel_fused:.3e}")
    assert rel_fused <= VIT_REL_BF16, rel_fused


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_add_layer_norm_matches_torch(cuda_device, dtype):
    from dimq_b200 import ops

    torch.manual_seed(1)
    x = torch.randn(5, 197, 768, device="cuda").to(dtype)
    d = torch.randn(5, 197, 768, device="cuda").to(dtype)
    w = (1 + 0.1 * torch.randn(768, device="cuda")).to(dtype)
    b = (0.1 * torch.randn(768, device="cuda")).to(dtype)
    x_out, h = ops.add_layer_norm(x, d, w, b, 1e-6)
    want_x = x + d
    assert torch.equal(x_out, want_x)
    want_h = torch.nn.functional.layer_norm(want_x.float(), (768,), w.float(), b.float(), 1e-6)
    assert (h.float() - want_h).abs().max().item() <= (4e-2 if dtype == torch.bfloat16 else 6e-3)
    same, h2 = ops.add_layer_norm(x, None, w, b, 1e-6)
    assert same.data_ptr() == x.data_ptr()
    want_h2 = torch.nn.functional.layer_norm(x.float(), (768,), w.float(), b.float(), 1e-6)
    assert (h2.float() - want_h2).abs().max().item() <= (4e-2 if dtype == torch.bfloat16 else 6e-3)
    _, h3 = ops.add_layer_norm(x[:, 0, :264].contiguous(), None, w[:264], b[:264], 1e-6)   # ragged: 33 vectors
    want_h3 = torch.nn.functional.layer_norm(x[:, 0, :264].float(), (264,), w[:264].float(), b[:264].float(), 1e-6)
    assert (h3.float() - want_h3).abs().max().item() <= (4e-2 if dtype == torch.bfloat16 else 6e-3)
    with pytest.raises(RuntimeError):
        ops.add_layer_norm(x[..., :100].contiguous(), None, w[:100], b[:100])


def _cpu_ckpt(ckpt):
    return {"config": ckpt.get("config"),
            "layers": {k: {kk: (vv.cpu() if hasattr(vv, "cpu") else vv) for kk, vv in v.items()}
                       for k, v in ckpt["layers"].items()},
            "non_quantized_state_dict": {k: v.cpu() for k, v in ckpt["non_quantized_state_dict"].items()}}


@pytest.mark.parametrize("fuse", [True, False])
def test_resnet18_forward_matches_cpu_oracle(cuda_device, fuse):
    from dimq_b200.workloads import DIMQResNet18, build_resnet18_checkpoint
    from oracle.models_oracle import ResNet18Oracle

    ckpt = build_resnet18_checkpoint(seed=2, device=cuda_device)
    model = DIMQResNet18(ckpt, fuse_residual=fuse).to(cuda_device).eval()
    n_img = 16
    images = torch.randn(n_img, 3, 224, 224, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    with torch.no_grad():
        got = model(images.cuda()).float().cpu().numpy()
    cpu = _cpu_ckpt(ckpt)
    want_bf16 = ResNet18Oracle(cpu, round_dtype=torch.bfloat16).forward(images).numpy()
    want_fp32 = ResNet18Oracle(cpu).forward(images).numpy()
    assert got.shape == (n_img, 1000)
    from dimq_b200 import ops
    assert ops.last_device_status() == 0
    abs_b, rel_b = o.parity_metrics(got, want_bf16)
    abs_f, rel_f = o.parity_metrics(got, want_fp32)
    agree = float((got.argmax(1) == want_fp32.argmax(1)).mean())
    print(f"ResNet-18 (fused residual: {fuse}), {n_img} images: vs bf16-rounding oracle max_abs={abs_b:.3e} "
          f"rel_l2={rel_b:.3e}; vs fp32 oracle max_abs={abs_f:.3e} rel_l2={rel_f:.3e}; argmax agreement {agree:.3f}")
    assert rel_b <= RESNET_REL_BF16, rel_b      # twice the measured values; bf16 activations: see the module docstring
    assert rel_f <= RESNET_REL_FP32, rel_f
    assert agree >= RESNET_ARGMAX
    assert abs(model.lut_flops(256) - 928.8e9) / 928.8e9 < 0.01   # per-batch work of the reference config


@pytest.mark.parametrize("src", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dst", [torch.bfloat16, torch.float16])
def test_images_to_nhwc_matches_torch(cuda_device, src, dst):
    from dimq_b200 import ops

    x = torch.randn(5, 3, 12, 10, generator=torch.Generator().manual_seed(3)).to(src).cuda()
    got = ops.images_to_nhwc(x, dst)
    want = x.to(dst).contiguous(memory_format=torch.channels_last)
    assert got.is_contiguous(memory_format=torch.channels_last) and got.dtype == dst
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError):
        ops.images_to_nhwc(x[:, :, :, :9].contiguous(), dst)     # 12 * 9 pixels: not a multiple of 8


def test_im2col_and_max_pool_helpers(cuda_device):
    from dimq_b200 import ops

    torch.manual_seed(4)
    x = torch.randn(3, 3, 19, 23, device="cuda").to(torch.bfloat16)
    cols, (oh, ow) = ops.im2col(x, (8, 3, 7, 7), (2, 2), (3, 3), padded_k=192)
    want = torch.nn.functional.unfold(x.float(), (7, 7), padding=3, stride=2)       # [B, C*49, L], (c, kh, kw) order
    want = want.view(3, 3, 49, oh * ow).permute(0, 3, 2, 1).reshape(3 * oh * ow, 147)  # -> (kh, kw, c) order
    assert cols.shape == (3 * oh * ow, 192)
    assert torch.equal(cols[:, :147].float(), want) and not cols[:, 147:].any()
    xcl = torch.randn(2, 16, 13, 11, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    got = ops.max_pool_nhwc(xcl, 3, 2, 1)
    assert torch.equal(got, torch.nn.functional.max_pool2d(xcl, 3, 2, 1))
    assert got.is_contiguous(memory_format=torch.channels_last)
    for dtype, (k, s, p) in ((torch.float16, (3, 2, 1)), (torch.bfloat16, (2, 2, 0)), (torch.float16, (5, 3, 2)),
                             (torch.bfloat16, (3, 1, 1))):          # 3x3 takes the unrolled window, the rest the loop
        xcl = torch.randn(3, 24, 17, 14, device="cuda").to(dtype).contiguous(memory_format=torch.channels_last)
        assert torch.equal(ops.max_pool_nhwc(xcl, k, s, p), torch.nn.functional.max_pool2d(xcl, k, s, p)), (dtype, k, s, p)


def test_resnet_layers_match_oracle_strictly(cuda_device):
    """Every quantised layer of the model's own checkpoint (the 19 tensor-core convolutions and the
    classifier), run alone on a random bf16 input with fp32 output, at max-abs 1e-2 / relative L2 1e-3
    against dequantise + fp32 F.conv2d / F.linear on the CPU."""
    from dimq_b200 import ops
    from dimq_b200.modules import DIMQConv2d, DIMQLinear
    from dimq_b200.workloads import build_resnet18_checkpoint
    from oracle.models_oracle import dequantize_layer

    ckpt = build_resnet18_checkpoint(seed=2, device=cuda_device)
    gen = torch.Generator().manual_seed(3)
    sizes = {"layer1": 56, "layer2": 56, "layer3": 28, "layer4": 14}   # input size of a stage's first block
    worst = (0.0, 0.0, "")
    for name, layer in ckpt["layers"].items():
        if name == "conv1":
            continue          # the 3-channel stem has its own test (patch matrix + GEMM)
        w_hat = dequantize_layer(layer)
        bias = layer["bias"].float().cpu()
        if name == "fc":
            x = torch.randn(64, 512, generator=gen).to(torch.bfloat16)
            want = torch.nn.functional.linear(x.float(), w_hat, bias)
            mod = DIMQLinear.from_export_layer(layer, out_dtype=torch.float32).to(cuda_device)
            got = mod(x.cuda()).cpu()
        else:
            stage = name.split(".")[0]
            first = name.split(".")[1] == "0" and (name.endswith("conv1") or name.endswith("downsample"))
            hw = sizes[stage] if first or stage == "layer1" else sizes[stage] // 2
            s, pad = layer["stride"][0], layer["padding"][0]
            x = torch.relu(torch.randn(8, layer["weight_shape"][1], hw, hw, generator=gen)).to(torch.bfloat16)
            want = torch.nn.functional.conv2d(x.float(), w_hat, bias, s, pad)
            mod = DIMQConv2d.from_export_layer(layer, out_dtype=torch.float32).to(cuda_device)
            got = mod(x.cuda().contiguous(memory_format=torch.channels_last)).cpu()
        diff = got - want
        max_abs, rel = float(diff.abs().max()), float(diff.norm() / want.norm())
        assert max_abs <= 1e-2 and rel <= 1e-3, (name, max_abs, rel)
        if rel > worst[1]:
            worst = (max_abs, rel, name)
    print(f"ResNet-18 per-layer check, worst layer {worst[2]}: max_abs={worst[0]:.3e} rel_l2={worst[1]:.3e}")
    assert ops.last_device_status() == 0
