"""Synthetic whole-model workloads built from packed DIMQ layers.

``build_vit_b16_checkpoint`` creates a random-init ViT-B/16 (12 layers, hidden 768,
12 heads, MLP 3072, 197 tokens, 1000 classes), quantises every qkv / proj / fc1 /
fc2 / head Linear to ``bits``-bit indices with one quantile codebook per
``group_rows`` output rows — the nearest-codeword assignment and the packing run in
the CUDA library (the export path of dimq_backend/export.py:159-260) — and returns
a ``dimq_packed_lut`` style dictionary.  ``DIMQViT`` runs it: the quantised Linears
go through the weight-only LUT GEMM, attention / LayerNorm / patch embedding stay
dense bf16 PyTorch ops.

The codebooks are rounded to ``codebook_dtype`` *before* the indices are assigned, so
the stored codebook is exactly what the kernels and any CPU check dequantise with.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .modules import DIMQLinear

VIT_B16 = dict(layers=12, hidden=768, heads=12, mlp=3072, patch=16, image=224, classes=1000)


def quantile_codebooks(w: torch.Tensor, entries: int, group_rows: int) -> torch.Tensor:
    """One sorted ``entries``-entry quantile codebook per ``group_rows`` rows of ``w`` (fp32, on w's device).

    Probabilities ``linspace(0, 1, entries + 2)[1:-1]`` and the post-processing of
    quant/dimq.py:132-137,175-194 (strictly increasing, mean kept); every weight of the group
    is used (no random subsample).
    """
    rows = w.shape[0]
    flat = w.reshape(rows, -1).float()
    q = torch.linspace(0.0, 1.0, entries + 2, device=w.device, dtype=torch.float32)[1:-1]
    n_groups = (rows + group_rows - 1) // group_rows
    if rows % group_rows == 0:
        samples = [flat.reshape(n_groups, -1)]                      # all groups in one batched call
    else:
        full = (rows // group_rows) * group_rows
        samples = ([flat[:full].reshape(rows // group_rows, -1)] if full else []) + [flat[full:].reshape(1, -1)]
    books = []
    for sample in samples:
        centers = torch.quantile(sample, q, dim=1).t().contiguous().sort(dim=1).values   # [g, entries]
        span = (sample.max(dim=1).values - sample.min(dim=1).values).abs()
        sigma = sample.std(dim=1, unbiased=False).abs()
        min_gap = torch.maximum(span, sigma).clamp_min(1e-6) * 1e-6
        fixed = centers.clone()
        for i in range(1, entries):
            bump = fixed[:, i] <= fixed[:, i - 1]
            fixed[:, i] = torch.where(bump, fixed[:, i - 1] + min_gap, fixed[:, i])
        fixed = fixed - (fixed.mean(dim=1, keepdim=True) - centers.mean(dim=1, keepdim=True))
        books.append(fixed.sort(dim=1).values)
    return torch.cat(books, dim=0)


def quantize_linear(weight: torch.Tensor, bias: torch.Tensor | None, bits: int, group_rows: int | None,
                    codebook_dtype: torch.dtype, name: str) -> dict[str, Any]:
    """Float weight on a CUDA device -> packed layer entry (indices assigned and packed on the GPU)."""
    out_f, in_f = weight.shape
    grp = out_f if group_rows is None else int(group_rows)
    books = quantile_codebooks(weight, 1 << bits, grp).to(codebook_dtype)
    _, packed = ops.hard_quantize(weight.float().contiguous(), books.float(), group_rows=grp, bits=bits,
                                  return_indices=False)
    return {
        "name": name, "type": "linear", "bit_w": bits, "weight_shape": [out_f, in_f], "weight_numel": out_f * in_f,
        "packed_weight": packed, "codebook": books, "group_rows": grp,
        "codebook_granularity": "per_layer" if grp == out_f else "per_row_group",
        "act_scale": None, "act_zero_point": None, "bias": bias, "layout": "linear_nk",
        "out_features": out_f, "in_features": in_f,
    }


@torch.no_grad()
def build_vit_b16_checkpoint(*, seed: int = 0, device="cuda", bits: int = 3, group_rows: int = 128,
                             codebook_dtype: torch.dtype = torch.bfloat16, layers: int | None = None,
                             dtype: torch.dtype = torch.bfloat16) -> dict[str, Any]:
    cfg = dict(VIT_B16)
    if layers is not None:
        cfg["layers"] = int(layers)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    dev = torch.device(device)

    def randn(*shape, std=0.02):
        return (torch.randn(*shape, generator=gen) * std).to(dev)

    hid, mlp = cfg["hidden"], cfg["mlp"]
    tokens = (cfg["image"] // cfg["patch"]) ** 2 + 1
    qlayers: dict[str, dict[str, Any]] = {}
    dense: dict[str, torch.Tensor] = {
        "patch_embed.weight": randn(hid, 3, cfg["patch"], cfg["patch"]).to(dtype),
        "patch_embed.bias": randn(hid).to(dtype),
        "cls_token": randn(1, 1, hid).to(dtype),
        "pos_embed": randn(1, tokens, hid).to(dtype),
        "norm.weight": (1.0 + randn(hid, std=0.05)).to(dtype),
        "norm.bias": randn(hid, std=0.05).to(dtype),
    }
    for i in range(cfg["layers"]):
        for ln in ("norm1", "norm2"):
            dense[f"blocks.{i}.{ln}.weight"] = (1.0 + randn(hid, std=0.05)).to(dtype)
            dense[f"blocks.{i}.{ln}.bias"] = randn(hid, std=0.05).to(dtype)
        for lname, (o, k) in (("attn.qkv", (3 * hid, hid)), ("attn.proj", (hid, hid)), ("mlp.fc1", (mlp, hid)),
                              ("mlp.fc2", (hid, mlp))):
            name = f"blocks.{i}.{lname}"
            qlayers[name] = quantize_linear(randn(o, k), randn(o).to(dtype), bits, group_rows, codebook_dtype, name)
    qlayers["head"] = quantize_linear(randn(cfg["classes"], hid), randn(cfg["classes"]).to(dtype), bits, group_rows,
                                      codebook_dtype, "head")
    return {"format": "dimq_packed_lut", "format_version": 2, "model_name": "vit_b16_synthetic", "config": cfg,
            "weight_encoding": "packed_bitstream_indices", "activation_quantization": "none", "layers": qlayers,
            "non_quantized_state_dict": dense}


class DIMQViT(nn.Module):
    """ViT-B/16 forward over packed DIMQ Linears (weight-only LUT GEMM), dense bf16 elsewhere."""

    def __init__(self, checkpoint: dict[str, Any], *, act_dtype: torch.dtype = torch.bfloat16,
                 fuse_epilogues: bool = True) -> None:
        super().__init__()
        self.cfg = dict(checkpoint["config"])
        self.act_dtype = act_dtype
        # By default GELU and the residual add run in the epilogue of the LUT GEMM (the residual tile
        # is prefetched with TMA); fuse_epilogues=False runs them as separate elementwise kernels, the
        # residual add fused with the following LayerNorm instead.
        self.fuse_epilogues = bool(fuse_epilogues)
        for key, value in checkpoint["non_quantized_state_dict"].items():
            self.register_buffer(key.replace(".", "__"), value.to(act_dtype))
        self.q = nn.ModuleDict()
        for name, layer in checkpoint["layers"].items():
            epi = "gelu" if (name.endswith("mlp.fc1") and self.fuse_epilogues) else None
            out_dtype = torch.float32 if name == "head" else act_dtype
            self.q[name.replace(".", "__")] = DIMQLinear.from_export_layer(layer, out_dtype=out_dtype, epilogue=epi)

    def _t(self, key: str) -> torch.Tensor:
        return getattr(self, key.replace(".", "__"))

    def _lin(self, name: str) -> DIMQLinear:
        return self.q[name.replace(".", "__")]

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        hid, heads = cfg["hidden"], cfg["heads"]
        b = images.shape[0]
        p = cfg["patch"]
        g = cfg["image"] // p
        # patch embedding (dense bf16): a stride-p conv is a GEMM over flattened (c, kh, kw) patches
        patches = images.to(self.act_dtype).view(b, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(b * g * g, 3 * p * p)
        emb = torch.addmm(self._t("patch_embed.bias"), patches, self._t("patch_embed.weight").view(hid, -1).t())
        # tokens = [cls | patches] + pos_embed, written in place (one pass instead of a cat and an add)
        t = g * g + 1
        pos = self._t("pos_embed")
        x = torch.empty(b, t, hid, dtype=self.act_dtype, device=images.device)
        x[:, :1] = self._t("cls_token") + pos[:, :1]
        torch.add(emb.view(b, g * g, hid), pos[:, 1:], out=x[:, 1:])
        if self.fuse_epilogues:
            for i in range(cfg["layers"]):
                pre = f"blocks.{i}."
                _, h = ops.add_layer_norm(x, None, self._t(pre + "norm1.weight"), self._t(pre + "norm1.bias"), 1e-6)
                a = self._attention(self._lin(pre + "attn.qkv")(h), b, t)
                x = self._lin(pre + "attn.proj")(a, residual=x)
                _, h = ops.add_layer_norm(x, None, self._t(pre + "norm2.weight"), self._t(pre + "norm2.bias"), 1e-6)
                x = self._lin(pre + "mlp.fc2")(self._lin(pre + "mlp.fc1")(h), residual=x)
            _, cls = ops.add_layer_norm(x[:, 0].contiguous(), None, self._t("norm.weight"), self._t("norm.bias"), 1e-6)
            return self._lin("head")(cls)
        # default: each residual add is fused with the LayerNorm that follows it (one pass over the
        # residual stream instead of two); GELU is a separate elementwise kernel
        delta = None
        for i in range(cfg["layers"]):
            pre = f"blocks.{i}."
            x, h = ops.add_layer_norm(x, delta, self._t(pre + "norm1.weight"), self._t(pre + "norm1.bias"), 1e-6)
            a = self._attention(self._lin(pre + "attn.qkv")(h), b, t)
            x, h = ops.add_layer_norm(x, self._lin(pre + "attn.proj")(a), self._t(pre + "norm2.weight"),
                                      self._t(pre + "norm2.bias"), 1e-6)
            delta = self._lin(pre + "mlp.fc2")(F.gelu(self._lin(pre + "mlp.fc1")(h)))
        _, cls = ops.add_layer_norm(x[:, 0].contiguous(), delta[:, 0].contiguous(), self._t("norm.weight"),
                                    self._t("norm.bias"), 1e-6)
        return self._lin("head")(cls)

    def _attention(self, qkv: torch.Tensor, b: int, t: int) -> torch.Tensor:
        hid, heads = self.cfg["hidden"], self.cfg["heads"]
        qkv = qkv.view(b, t, 3, heads, hid // heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        return a.transpose(1, 2).reshape(b, t, hid)

    def lut_gemm_flops(self, batch: int) -> float:
        """Algorithmic flops (2*M*N*K) of the quantised Linears for one forward of ``batch`` images."""
        t = (self.cfg["image"] // self.cfg["patch"]) ** 2 + 1
        total = 0.0
        for name, mod in self.q.items():
            m = batch if name == "head" else batch * t
            total += 2.0 * m * mod.out_features * mod.in_features
        return total


# ---------------------------------------------------------------------------------------------
# ResNet-18 (BN folded), every Conv2d / Linear quantised: 4-bit per-layer codebooks, except the
# first conv and the classifier at 8 bits
# ---------------------------------------------------------------------------------------------

RESNET18_STAGES = ((64, 1), (128, 2), (256, 2), (512, 2))   # (channels, stride of the first block)


def quantize_conv(weight: torch.Tensor, bias: torch.Tensor, bits: int, codebook_dtype: torch.dtype, name: str,
                  stride: int, padding: int) -> dict[str, Any]:
    """Float conv weight ``[OC, C, KH, KW]`` on a CUDA device -> packed layer entry (per-layer codebook)."""
    oc = weight.shape[0]
    books = quantile_codebooks(weight.reshape(oc, -1), 1 << bits, oc).to(codebook_dtype)
    _, packed = ops.hard_quantize(weight.float().contiguous(), books.float().reshape(-1), bits=bits,
                                  return_indices=False)
    return {"name": name, "type": "conv2d", "bit_w": bits, "weight_shape": list(weight.shape),
            "weight_numel": weight.numel(), "packed_weight": packed, "codebook": books.reshape(-1),
            "codebook_granularity": "per_layer", "act_scale": None, "act_zero_point": None, "bias": bias,
            "layout": "conv_kcrs", "out_channels": oc, "in_channels_per_group": weight.shape[1],
            "kernel_size": list(weight.shape[2:]), "stride": [stride, stride], "padding": [padding, padding],
            "dilation": [1, 1], "groups": 1}


@torch.no_grad()
def build_resnet18_checkpoint(*, seed: int = 0, device="cuda", codebook_dtype: torch.dtype = torch.bfloat16,
                              dtype: torch.dtype = torch.bfloat16, classes: int = 1000) -> dict[str, Any]:
    """Random-init ResNet-18 with BatchNorm already folded into conv weight and bias (Kaiming-normal
    weights times a random per-channel BN scale, random folded bias), quantised layer by layer."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    dev = torch.device(device)
    layers: dict[str, dict[str, Any]] = {}

    def conv(name, oc, ic, k, stride, bits=4):
        w = torch.randn(oc, ic, k, k, generator=gen) * (2.0 / (ic * k * k)) ** 0.5
        scale = 0.5 + torch.rand(oc, generator=gen)          # folded BN gamma / sqrt(var + eps)
        bias = (torch.randn(oc, generator=gen) * 0.1).to(dev).to(dtype)
        layers[name] = quantize_conv((w * scale.view(-1, 1, 1, 1)).to(dev), bias, bits, codebook_dtype, name, stride,
                                     k // 2)

    conv("conv1", 64, 3, 7, 2, bits=8)
    in_ch = 64
    for si, (ch, stride) in enumerate(RESNET18_STAGES, start=1):
        for bi in range(2):
            s = stride if bi == 0 else 1
            conv(f"layer{si}.{bi}.conv1", ch, in_ch, 3, s)
            conv(f"layer{si}.{bi}.conv2", ch, ch, 3, 1)
            if s != 1 or in_ch != ch:
                conv(f"layer{si}.{bi}.downsample", ch, in_ch, 1, s)
            in_ch = ch
    fc_w = (torch.randn(classes, 512, generator=gen) * 0.02).to(dev)
    fc_b = (torch.randn(classes, generator=gen) * 0.02).to(dev).to(dtype)
    layers["fc"] = quantize_linear(fc_w, fc_b, 8, None, codebook_dtype, "fc")
    return {"format": "dimq_packed_lut", "format_version": 2, "model_name": "resnet18_synthetic",
            "weight_encoding": "packed_bitstream_indices", "activation_quantization": "none", "layers": layers,
            "non_quantized_state_dict": {}}


class DIMQResNet18(nn.Module):
    """ResNet-18 forward over packed DIMQ layers, channels_last bf16 activations.

    3x3 / 1x1 convolutions with a multiple of 64 input channels run as tensor-core implicit GEMMs with
    bias + ReLU (+ residual) in the epilogue; the 7x7 stem (3 input channels) through the stem kernel,
    which builds its patch rows in shared memory; the max-pool is a dimq_b200 kernel, the global
    average pool a PyTorch op.
    """

    def __init__(self, checkpoint: dict[str, Any], *, act_dtype: torch.dtype = torch.bfloat16,
                 fuse_residual: bool = True) -> None:
        super().__init__()
        from .modules import DIMQConv2d

        self.act_dtype = act_dtype
        self.fuse_residual = bool(fuse_residual)
        self.convs = nn.ModuleDict()
        for name, layer in checkpoint["layers"].items():
            if name in ("conv1", "fc"):
                continue
            self.convs[name.replace(".", "__")] = DIMQConv2d.from_export_layer(layer, out_dtype=act_dtype)
        fc = checkpoint["layers"]["fc"]
        self.fc = DIMQLinear.from_export_layer(fc, out_dtype=torch.float32)
        # stem (7x7, stride 2, 3 input channels): its own tensor-core kernel builds the patches in shared
        # memory; bias + ReLU fused
        stem = checkpoint["layers"]["conv1"]
        self.stem = DIMQConv2d.from_export_layer(stem, out_dtype=act_dtype, epilogue="relu")
        oc, ic, kh, kw = stem["weight_shape"]
        self.stem_k = kh * kw * ic

    def _conv(self, name: str):
        return self.convs[name.replace(".", "__")]

    def _stem(self, images: torch.Tensor) -> torch.Tensor:
        if images.is_contiguous() and (images.shape[2] * images.shape[3]) % 8 == 0 and images.dtype in (
                torch.float32, torch.float16, torch.bfloat16):
            x = ops.images_to_nhwc(images, self.act_dtype)                                 # NCHW images -> NHWC, one pass
        else:
            x = images.to(self.act_dtype).contiguous(memory_format=torch.channels_last)
        return self.stem(x)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        x = self._stem(images)
        x = ops.max_pool_nhwc(x, 3, 2, 1)
        in_ch = 64
        for si, (ch, stride) in enumerate(RESNET18_STAGES, start=1):
            for bi in range(2):
                s = stride if bi == 0 else 1
                pre = f"layer{si}.{bi}."
                identity = x
                if s != 1 or in_ch != ch:
                    identity = self._conv(pre + "downsample")(x)
                c1 = self._conv(pre + "conv1")
                c1.epilogue = "relu"
                y = c1(x)
                c2 = self._conv(pre + "conv2")
                if self.fuse_residual:
                    c2.epilogue = "add_relu"
                    x = c2(y, residual=identity)
                else:
                    c2.epilogue = None
                    x = torch.relu_(c2(y) + identity)
                in_ch = ch
        pooled = x.mean(dim=(2, 3)).to(self.act_dtype)
        return self.fc(pooled.contiguous())

    @torch.no_grad()
    def calibrate(self, batches) -> dict[str, dict[str, Any]]:
        """Per-layer u4 activation parameters from the input ranges the 4-bit convolutions see over
        ``batches`` (keys are the checkpoint's layer names)."""
        from .calibration import calibrate_activation_qparams

        q = calibrate_activation_qparams(self, batches, select=lambda name, m: name.startswith("convs."))
        return {name[len("convs."):].replace("__", "."): v for name, v in q.items()}

    def set_activation_qparams(self, qparams: dict[str, dict[str, Any]]) -> int:
        """Switch the named 4-bit convolutions to the W4A4 mode (the stem and the classifier, 8-bit, stay
        weight-only, as the reference's default configuration leaves the first and last layer alone)."""
        from .calibration import apply_activation_qparams

        return apply_activation_qparams(self, {"convs." + k.replace(".", "__"): v for k, v in qparams.items()})

    def lut_flops(self, batch: int, image: int = 224) -> float:
        """Algorithmic flops (2 * outputs * K) of every quantised layer for one forward."""
        total = 0.0
        size = (image + 6 - 7) // 2 + 1
        total += 2.0 * batch * size * size * 64 * self.stem_k
        size = (size + 2 - 3) // 2 + 1
        for name, mod in self.convs.items():
            oc, ic, kh, kw = mod.weight_shape
            if name.endswith("__0__conv1") and mod.stride[0] == 2:
                size = (size + 2 - 3) // 2 + 1
            total += 2.0 * batch * size * size * oc * ic * kh * kw
        return total + 2.0 * batch * self.fc.out_features * self.fc.in_features
