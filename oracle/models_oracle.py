"""CPU restatement of the whole-model path: dequantise every packed layer, then run the
float model with PyTorch CPU ops — what the DIMQ reference does in its QAT-wrapper eval
forward (quant/dimq_wrapper.py:237-240: hard-quantised weight + ``F.linear``) and in
``convert_to_dequantized_model`` (quant/export_dimq.py:15-29).

TEST INFRASTRUCTURE ONLY: used by the parity tests, ``smoke()`` and the CPU-baseline /
``--impl reference`` legs of ``bench.py``.  Parity status: pinned through the layer-level
functions of ``dimq_oracle`` (checked against the reference's golden vectors); the model
wiring itself (ViT-B/16 block structure) is the synthetic workload's own definition.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from . import dimq_oracle as o


def dequantize_layer(layer: dict) -> torch.Tensor:
    """``codebook.float()[indices]`` for one packed layer (dimq_backend/reference.py:47-56)."""
    shape = [int(v) for v in layer["weight_shape"]]
    numel = int(np.prod(shape))
    idx = o.unpack_bits(layer["packed_weight"].cpu().numpy(), numel, int(layer["bit_w"])).reshape(shape[0], -1)
    books = layer["codebook"].float().cpu().numpy()
    if books.ndim == 1:
        books = books[None, :]
    w = o.dequantize(idx, books, int(layer.get("group_rows") or shape[0]))
    return torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32)).reshape(shape)


class ViTOracle:
    """fp32 CPU ViT over the dequantised weights.  ``round_dtype`` (e.g. torch.bfloat16) rounds the
    activations at the points where the GPU path stores them in that type."""

    def __init__(self, checkpoint: dict, round_dtype: torch.dtype | None = None) -> None:
        self.cfg = dict(checkpoint["config"])
        self.round_dtype = round_dtype
        self.dense = {k: v.float().cpu() for k, v in checkpoint["non_quantized_state_dict"].items()}
        self.w = {}
        self.b = {}
        for name, layer in checkpoint["layers"].items():
            self.w[name] = dequantize_layer(layer)
            self.b[name] = None if layer.get("bias") is None else layer["bias"].float().cpu()

    def _r(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.round_dtype is None else x.to(self.round_dtype).float()

    @torch.no_grad()
    def forward(self, images: torch.Tensor) -> torch.Tensor:
        cfg, d = self.cfg, self.dense
        hid, heads = cfg["hidden"], cfg["heads"]
        x = self._r(F.conv2d(self._r(images.float().cpu()), d["patch_embed.weight"], d["patch_embed.bias"],
                             stride=cfg["patch"]))
        b = x.shape[0]
        x = x.flatten(2).transpose(1, 2)
        x = self._r(torch.cat([d["cls_token"].expand(b, -1, -1), x], dim=1) + d["pos_embed"])
        t = x.shape[1]
        for i in range(cfg["layers"]):
            pre = f"blocks.{i}."
            h = self._r(F.layer_norm(x, (hid,), d[pre + "norm1.weight"], d[pre + "norm1.bias"], 1e-6))
            qkv = self._r(F.linear(h, self.w[pre + "attn.qkv"], self.b[pre + "attn.qkv"]))
            qkv = qkv.view(b, t, 3, heads, hid // heads).permute(2, 0, 3, 1, 4)
            a = self._r(F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2]))
            a = a.transpose(1, 2).reshape(b, t, hid)
            x = self._r(F.linear(a, self.w[pre + "attn.proj"], self.b[pre + "attn.proj"]) + x)
            h = self._r(F.layer_norm(x, (hid,), d[pre + "norm2.weight"], d[pre + "norm2.bias"], 1e-6))
            h = self._r(F.gelu(F.linear(h, self.w[pre + "mlp.fc1"], self.b[pre + "mlp.fc1"])))
            x = self._r(F.linear(h, self.w[pre + "mlp.fc2"], self.b[pre + "mlp.fc2"]) + x)
        cls = self._r(F.layer_norm(x[:, 0], (hid,), d["norm.weight"], d["norm.bias"], 1e-6))
        return F.linear(cls, self.w["head"], self.b["head"])


def build_vit_b16_checkpoint_cpu(*, seed: int = 0, bits: int = 3, group_rows: int = 128, layers: int = 12,
                                 codebook_round=None) -> dict:
    """A synthetic packed ViT-B/16 checkpoint made entirely on the CPU with the oracle's own
    functions (quantile codebooks per ``group_rows`` rows, nearest-codeword indices, bit-stream
    packing): N(0, 0.02) weights, the shapes of ViT-B/16.  Used by the CPU-only reference arm."""
    from . import c_oracle

    cfg = dict(layers=layers, hidden=768, heads=12, mlp=3072, patch=16, image=224, classes=1000)
    rng = np.random.default_rng(seed)
    hid, mlp = cfg["hidden"], cfg["mlp"]
    tokens = (cfg["image"] // cfg["patch"]) ** 2 + 1

    def randn(*shape, std=0.02):
        return torch.from_numpy((rng.standard_normal(shape) * std).astype(np.float32))

    def qlayer(name, out_f, in_f):
        w = randn(out_f, in_f).numpy()
        books = np.stack([o.quantile_codebook(w[g0 : g0 + group_rows], 1 << bits) for g0 in range(0, out_f, group_rows)])
        if codebook_round is not None:
            books = codebook_round(books)
        idx = c_oracle.hard_quantize(w, books, group_rows)
        return {"name": name, "type": "linear", "bit_w": bits, "weight_shape": [out_f, in_f],
                "packed_weight": torch.from_numpy(c_oracle.pack_bits(idx, bits)), "codebook": torch.from_numpy(books),
                "group_rows": group_rows, "bias": randn(out_f), "out_features": out_f, "in_features": in_f,
                "act_scale": None, "act_zero_point": None}

    dense = {"patch_embed.weight": randn(hid, 3, 16, 16), "patch_embed.bias": randn(hid),
             "cls_token": randn(1, 1, hid), "pos_embed": randn(1, tokens, hid),
             "norm.weight": 1.0 + randn(hid, std=0.05), "norm.bias": randn(hid, std=0.05)}
    qlayers = {}
    for i in range(layers):
        for ln in ("norm1", "norm2"):
            dense[f"blocks.{i}.{ln}.weight"] = 1.0 + randn(hid, std=0.05)
            dense[f"blocks.{i}.{ln}.bias"] = randn(hid, std=0.05)
        for lname, (of, k) in (("attn.qkv", (3 * hid, hid)), ("attn.proj", (hid, hid)), ("mlp.fc1", (mlp, hid)),
                               ("mlp.fc2", (hid, mlp))):
            qlayers[f"blocks.{i}.{lname}"] = qlayer(f"blocks.{i}.{lname}", of, k)
    qlayers["head"] = qlayer("head", cfg["classes"], hid)
    return {"format": "dimq_packed_lut", "format_version": 2, "config": cfg, "layers": qlayers,
            "non_quantized_state_dict": dense}


class ResNet18Oracle:
    """fp32 CPU ResNet-18 (BN folded) over the dequantised weights: ``F.conv2d`` + bias + ReLU, the
    computation of the reference's wrapper forward (quant/dimq_wrapper.py:189-197) layer by layer.
    ``round_dtype`` rounds activations where the GPU path stores them."""

    STAGES = ((64, 1), (128, 2), (256, 2), (512, 2))

    def __init__(self, checkpoint: dict, round_dtype: torch.dtype | None = None,
                 act_qparams: dict | None = None) -> None:
        self.round_dtype = round_dtype
        # W4A4 mode: layers named here see their input through the reference's uniform affine u4
        # quantiser (dimq_backend/reference.py:11-29), the contract of dimq_conv2d_reference (:113-144)
        self.act_qparams = act_qparams or {}
        self.w, self.b, self.meta = {}, {}, {}
        for name, layer in checkpoint["layers"].items():
            self.w[name] = dequantize_layer(layer)
            self.b[name] = layer["bias"].float().cpu()
            self.meta[name] = layer

    def _r(self, x):
        return x if self.round_dtype is None else x.to(self.round_dtype).float()

    def _conv(self, name, x):
        m = self.meta[name]
        if name in self.act_qparams:
            scale, zp = float(self.act_qparams[name]["scale"]), int(self.act_qparams[name]["zero_point"])
            q = torch.clamp(torch.round(x.float() / scale) + zp, 0, 15)
            x = scale * (q - zp)
        return F.conv2d(x, self.w[name], self.b[name], tuple(m["stride"]), tuple(m["padding"]))

    @torch.no_grad()
    def forward(self, images: torch.Tensor) -> torch.Tensor:
        x = self._r(torch.relu(self._conv("conv1", self._r(images.float().cpu()))))
        x = F.max_pool2d(x, 3, 2, 1)
        in_ch = 64
        for si, (ch, stride) in enumerate(self.STAGES, start=1):
            for bi in range(2):
                s = stride if bi == 0 else 1
                pre = f"layer{si}.{bi}."
                identity = x
                if s != 1 or in_ch != ch:
                    identity = self._r(self._conv(pre + "downsample", x))
                y = self._r(torch.relu(self._conv(pre + "conv1", x)))
                x = self._r(torch.relu(self._conv(pre + "conv2", y) + identity))
                in_ch = ch
        pooled = self._r(x.mean(dim=(2, 3)))
        return F.linear(pooled, self.w["fc"], self.b["fc"])


def build_resnet18_checkpoint_cpu(*, seed: int = 0, classes: int = 1000) -> dict:
    """Synthetic packed ResNet-18 (BN folded) made on the CPU with the oracle's own functions:
    4-bit per-layer quantile codebooks, 8 bits for the stem and the classifier."""
    from . import c_oracle

    rng = np.random.default_rng(seed)
    layers = {}

    def quant(name, w, bits, extra):
        flat = w.reshape(w.shape[0], -1)
        book = o.quantile_codebook(flat, 1 << bits)
        idx = c_oracle.hard_quantize(flat, book)
        layers[name] = {"name": name, "bit_w": bits, "weight_shape": list(w.shape),
                        "packed_weight": torch.from_numpy(c_oracle.pack_bits(idx, bits)),
                        "codebook": torch.from_numpy(book), "group_rows": w.shape[0],
                        "bias": torch.from_numpy((rng.standard_normal(w.shape[0]) * 0.1).astype(np.float32)), **extra}

    def conv(name, oc, ic, k, stride, bits=4):
        w = (rng.standard_normal((oc, ic, k, k)) * (2.0 / (ic * k * k)) ** 0.5).astype(np.float32)
        w *= (0.5 + rng.random(oc)).astype(np.float32).reshape(-1, 1, 1, 1)
        quant(name, w, bits, {"type": "conv2d", "stride": [stride, stride], "padding": [k // 2, k // 2]})

    conv("conv1", 64, 3, 7, 2, bits=8)
    in_ch = 64
    for si, (ch, stride) in enumerate(ResNet18Oracle.STAGES, start=1):
        for bi in range(2):
            s = stride if bi == 0 else 1
            conv(f"layer{si}.{bi}.conv1", ch, in_ch, 3, s)
            conv(f"layer{si}.{bi}.conv2", ch, ch, 3, 1)
            if s != 1 or in_ch != ch:
                conv(f"layer{si}.{bi}.downsample", ch, in_ch, 1, s)
            in_ch = ch
    quant("fc", (rng.standard_normal((classes, 512)) * 0.02).astype(np.float32), 8,
          {"type": "linear", "out_features": classes, "in_features": 512})
    return {"format": "dimq_packed_lut", "format_version": 2, "layers": layers, "non_quantized_state_dict": {}}
