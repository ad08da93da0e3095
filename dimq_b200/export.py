"""Checkpoint formats and export helpers, with the index work done on the GPU.

Mirrors the names, arguments and dictionaries of

* quant/dimq.py:197-221            ``hard_quantize_weight``
* quant/export_dimq.py:55-112      ``export_compact_checkpoint`` / ``load_compact_checkpoint``
* dimq_backend/export.py:24-260    ``assign_weight_indices``, ``pack_u4_indices``, ``unpack_u4_indices``,
                                   activation-qparam helpers, ``infer_module_hparams``,
                                   ``export_packed_dimq_checkpoint``

The nearest-codeword assignment and the bit packing run in the CUDA library on
``cuda:<current>``; tensors are moved there and results come back on the
caller's device.  Dictionary layouts are unchanged (``dimq_compact`` and
``dimq_packed_lut`` version 1); layers that are not 4-bit / per-layer are written
with ``format_version`` 2 and the extra keys ``bit_w``, ``group_rows`` and
``codebook_granularity``.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch
import torch.nn as nn

from . import ops

QMIN_U4 = 0
QMAX_U4 = 15


def _cuda_device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("dimq_b200 export helpers need a CUDA device (there is no CPU path)")
    return torch.device("cuda", torch.cuda.current_device())


def _to_cuda(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_cuda else t.to(_cuda_device())


# ---- quant/dimq.py --------------------------------------------------------------

def hard_quantize_weight(w: torch.Tensor, centers: torch.Tensor, chunk_size: int | None = 262144):
    """``(values like w, idx int64 like w)`` — nearest centre, ties to the lowest index.

    ``chunk_size`` is accepted for signature compatibility; the kernel needs no
    chunking and the result does not depend on it.  At most 256 centres (indices of one
    byte): the reference (quant/dimq.py:197-221) also takes larger codebooks and stores
    int16 indices for them; this backend raises ``RuntimeError`` there.
    """
    if centers.numel() == 0:
        raise ValueError("centers must be non-empty")
    wc = _to_cuda(w.detach())
    wc = wc if wc.is_floating_point() else wc.float()
    if wc.dtype == torch.float64:
        wc = wc.float()
    cc = _to_cuda(centers.detach()).float().reshape(-1)
    idx, _ = ops.hard_quantize(wc, cc)
    idx = idx.to(device=w.device, dtype=torch.int64).reshape(w.shape)
    values = centers.reshape(-1)[idx.to(centers.device)].to(dtype=w.dtype, device=w.device)
    return values, idx


# ---- dimq_backend/export.py -------------------------------------------------------

def assign_weight_indices(weight: torch.Tensor, codebook: torch.Tensor) -> torch.Tensor:
    centers = codebook.detach().float().reshape(-1)
    if centers.numel() > 16:
        raise ValueError(f"packed u4 export supports at most 16 centers, got {centers.numel()}")
    if centers.numel() == 0:
        raise ValueError("codebook must not be empty")
    idx, _ = ops.hard_quantize(_to_cuda(weight.detach()).float(), _to_cuda(centers))
    return idx.to(weight.device).reshape(weight.shape)


def pack_indices(indices: torch.Tensor, bits: int) -> torch.Tensor:
    flat = indices.detach().contiguous().reshape(-1).to(torch.uint8)
    if flat.numel() == 0:
        return flat.new_empty((0,), dtype=torch.uint8)
    if int(flat.max().item()) >= (1 << bits):
        raise ValueError(f"indices must be in [0, {(1 << bits) - 1}]")
    return ops.pack_bits(_to_cuda(flat), bits).to(indices.device)


def unpack_indices(packed: torch.Tensor, numel: int, bits: int, *, shape=None) -> torch.Tensor:
    flat = packed.detach().contiguous().reshape(-1).to(torch.uint8)
    if numel < 0:
        raise ValueError("numel must be non-negative")
    needed = (numel * bits + 7) // 8
    if flat.numel() < needed:
        raise ValueError(f"packed tensor has {flat.numel()} bytes, expected at least {needed}")
    out = ops.unpack_bits(_to_cuda(flat), numel, bits).to(packed.device)
    return out.reshape(tuple(shape)) if shape is not None else out


def pack_u4_indices(indices: torch.Tensor) -> torch.Tensor:
    flat = indices.detach().reshape(-1)
    if flat.numel() and (int(flat.max().item()) > 15 or int(flat.min().item()) < 0):
        raise ValueError("u4 indices must be in [0, 15]")
    return pack_indices(indices, 4)


def unpack_u4_indices(packed: torch.Tensor, numel: int, *, shape=None) -> torch.Tensor:
    return unpack_indices(packed, numel, 4, shape=shape)


def activation_qparams_from_minmax(min_val: float, max_val: float, *, qmin: int = QMIN_U4, qmax: int = QMAX_U4,
                                   eps: float = 1e-8) -> dict[str, Any]:
    min_val, max_val = float(min_val), float(max_val)
    if not (min_val == min_val and max_val == max_val) or abs(min_val) == float("inf") or abs(max_val) == float("inf"):
        raise ValueError("activation min/max must be finite")
    if min_val > max_val:
        min_val, max_val = max_val, min_val
    if max_val - min_val < eps:
        scale, zero_point = 1.0, 0
    else:
        scale = max((max_val - min_val) / float(qmax - qmin), eps)
        zero_point = max(qmin, min(qmax, int(round(qmin - min_val / scale))))
    return {"bit_a": 4, "scale": float(scale), "zero_point": int(zero_point), "qmin": int(qmin), "qmax": int(qmax),
            "granularity": "per_tensor"}


def default_activation_qparams() -> dict[str, Any]:
    return {"bit_a": 4, "scale": 1.0, "zero_point": 8, "qmin": QMIN_U4, "qmax": QMAX_U4,
            "granularity": "per_tensor", "source": "default_uncalibrated"}


def _normalize_act_qparams(value: Mapping[str, Any]) -> dict[str, Any]:
    if "scale" not in value or "zero_point" not in value:
        raise ValueError("activation qparams must include scale and zero_point")
    scale = float(value["scale"])
    if scale <= 0.0:
        raise ValueError("activation scale must be positive")
    zero_point = int(value["zero_point"])
    qmin, qmax = int(value.get("qmin", QMIN_U4)), int(value.get("qmax", QMAX_U4))
    if qmin != QMIN_U4 or qmax != QMAX_U4:
        raise ValueError("this backend currently supports only u4 activation range [0, 15]")
    if zero_point < qmin or zero_point > qmax:
        raise ValueError("activation zero_point must be in [0, 15]")
    out = dict(value)
    out.update({"bit_a": 4, "scale": scale, "zero_point": zero_point, "qmin": qmin, "qmax": qmax,
                "granularity": value.get("granularity", "per_tensor")})
    return out


def load_activation_qparams(path: str | Path) -> dict[str, dict[str, Any]]:
    data = json.loads(Path(path).read_text())
    if not isinstance(data, dict):
        raise ValueError("activation qparams JSON must contain a mapping")
    return {str(k): _normalize_act_qparams(v) for k, v in data.items()}


def _pair(value: Any) -> tuple[int, int]:
    if isinstance(value, int):
        return int(value), int(value)
    if isinstance(value, (tuple, list, torch.Size)) and len(value) == 2:
        return int(value[0]), int(value[1])
    raise ValueError(f"expected an int or pair, got {value!r}")


def infer_module_hparams(model: nn.Module) -> dict[str, dict[str, Any]]:
    hparams: dict[str, dict[str, Any]] = {}
    for name, module in model.named_modules():
        if isinstance(module, nn.Conv2d):
            hparams[name] = {"type": "conv2d", "stride": list(_pair(module.stride)),
                             "padding": list(_pair(module.padding)), "dilation": list(_pair(module.dilation)),
                             "groups": int(module.groups),
                             "bias": module.bias.detach().cpu() if module.bias is not None else None}
        elif isinstance(module, nn.Linear):
            hparams[name] = {"type": "linear",
                             "bias": module.bias.detach().cpu() if module.bias is not None else None}
    return hparams


@torch.no_grad()
def export_packed_dimq_checkpoint(compact_checkpoint, output_path, *, act_qparams=None, layer_hparams=None,
                                  model_name: str = "dimq_packed_lut", codebook_dtype: torch.dtype = torch.float16,
                                  weight_only: bool = False) -> dict[str, Any]:
    """Compact checkpoint -> packed runtime checkpoint (dimq_backend/export.py:159-260).

    4-bit, 16-centre, per-layer inputs give the reference's version-1 dictionary
    byte for byte.  Other bit widths (``bits`` of the compact layer in {2, 3, 8})
    and grouped codebooks (``centers`` of shape ``[G, K]`` with a ``group_rows``
    entry) are written as version 2.  ``weight_only=True`` stores
    ``act_scale=None`` so that the runtime layers skip the activation quantiser.
    """
    if isinstance(compact_checkpoint, Mapping):
        compact, source_path = dict(compact_checkpoint), None
    else:
        source_path = str(compact_checkpoint)
        compact = torch.load(Path(compact_checkpoint), map_location="cpu")
    if compact.get("format") != "dimq_compact":
        raise ValueError(f"expected a dimq_compact checkpoint, got {compact.get('format')!r}")

    if act_qparams is None:
        qmap = {"__default__": default_activation_qparams()}
    elif isinstance(act_qparams, (str, Path)):
        qmap = load_activation_qparams(act_qparams)
    else:
        qmap = {str(k): _normalize_act_qparams(v) for k, v in act_qparams.items()}
    hmap = {str(k): dict(v) for k, v in (layer_hparams or {}).items()}
    non_quantized = compact.get("non_quantized_state_dict", {})

    layers: dict[str, dict[str, Any]] = {}
    version = 1
    for name, layer in compact["layers"].items():
        centers = layer["centers"].detach().float()
        bits = int(layer.get("bits", 4))
        grouped = centers.dim() == 2 and centers.shape[0] > 1
        extended = weight_only or grouped or bits != 4
        if not extended and centers.numel() != 16:
            raise ValueError(f"{name} has {centers.numel()} centers; this W4A4 backend expects 16 learned centers")
        if bits not in (2, 3, 4, 8) or centers.shape[-1] > (1 << bits):
            raise ValueError(f"{name}: {centers.shape[-1]} centres cannot be stored with {bits}-bit indices")
        indices = layer["indices"].detach().to(torch.uint8)
        if indices.numel() and int(indices.max().item()) >= (1 << bits):
            raise ValueError(f"{name} contains indices outside [0, {(1 << bits) - 1}]")
        shape = [int(d) for d in layer["shape"]]
        hp = hmap.get(name)
        if hp and hp.get("type") in {"conv2d", "linear"}:
            layer_type = str(hp["type"])
        elif len(shape) == 2:
            layer_type = "linear"
        elif len(shape) == 4:
            layer_type = "conv2d"
        else:
            raise ValueError(f"cannot infer layer type from weight shape {shape}")
        bias = hp["bias"] if hp and hp.get("bias") is not None else non_quantized.get(f"{name}.bias")
        if name in qmap:
            aq = _normalize_act_qparams(qmap[name])
        elif "__default__" in qmap:
            aq = _normalize_act_qparams(qmap["__default__"])
        else:
            raise KeyError(f"missing activation qparams for layer {name!r}")
        packed = pack_indices(indices, bits).cpu()
        entry: dict[str, Any] = {
            "name": name, "type": layer_type, "bit_w": bits, "bit_a": 4, "weight_shape": shape,
            "weight_numel": int(indices.numel()), "packed_weight": packed, "packed_indices": packed,
            "codebook": (centers if grouped else centers.reshape(-1)).to(dtype=codebook_dtype).cpu(),
            "codebook_granularity": "per_row_group" if grouped else "per_layer",
            "act_scale": None if weight_only else float(aq["scale"]),
            "act_zero_point": None if weight_only else int(aq["zero_point"]),
            "act_qmin": int(aq.get("qmin", QMIN_U4)), "act_qmax": int(aq.get("qmax", QMAX_U4)),
            "activation_qparams": aq,
            "bias": bias.detach().cpu().to(dtype=codebook_dtype) if bias is not None else None,
        }
        if grouped:
            entry["group_rows"] = int(layer["group_rows"])
        if extended:
            version = 2
        if layer_type == "linear":
            entry.update(layout="linear_nk", out_features=shape[0], in_features=shape[1])
        else:
            hp = hp or {}
            default_pad = (shape[2] // 2, shape[3] // 2) if len(shape) == 4 else (0, 0)
            entry.update(layout="conv_kcrs", out_channels=shape[0], in_channels_per_group=shape[1],
                         kernel_size=shape[2:4], stride=list(_pair(hp.get("stride", (1, 1)))),
                         padding=list(_pair(hp.get("padding", default_pad))),
                         dilation=list(_pair(hp.get("dilation", (1, 1)))), groups=int(hp.get("groups", 1)))
        layers[name] = entry

    state = {
        "format": "dimq_packed_lut", "format_version": version, "model_name": model_name,
        "source_checkpoint": source_path, "source_format": compact.get("format"),
        "source_extra": compact.get("extra", {}), "model_meta": compact.get("model_meta", {}),
        "quant_cfg": compact.get("quant_cfg", {}),
        "weight_encoding": "packed_u4_indices" if version == 1 else "packed_bitstream_indices",
        "activation_quantization": "uniform_affine_u4" if not weight_only else "none",
        "layers": layers, "non_quantized_state_dict": non_quantized,
    }
    output_path = Path(output_path)
    output_path.parent.mkdir(parents=True, exist_ok=True)
    torch.save(state, output_path)
    return state


# ---- quant/export_dimq.py -----------------------------------------------------------

def get_dimq_modules(model: nn.Module) -> list[tuple[str, nn.Module]]:
    """Modules that look like the reference's QAT wrappers (quant/dimq_wrapper.py:172-260):
    a ``weight`` and a ``centers`` parameter plus a ``cfg`` with ``w_bits``."""
    found = []
    for name, module in model.named_modules():
        if hasattr(module, "centers") and hasattr(module, "weight") and hasattr(getattr(module, "cfg", None), "w_bits"):
            found.append((name, module))
    return found


@torch.no_grad()
def export_compact_checkpoint(model: nn.Module, path, *, extra=None, include_model_state: bool = False):
    """Same dictionary as quant/export_dimq.py:55-108, with the assignment done on the GPU."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    modules = get_dimq_modules(model)
    layers: dict[str, dict[str, Any]] = {}
    for name, module in modules:
        centers = module.centers.detach().float().sort().values
        weight, indices = hard_quantize_weight(module.weight, centers.to(module.centers.dtype),
                                               getattr(module.cfg, "chunk_size", None))
        index_dtype = torch.uint8 if centers.numel() <= 256 else torch.int16
        layers[name] = {
            "shape": list(module.weight.shape), "bits": int(module.cfg.w_bits), "centers": centers.cpu(),
            "indices": indices.detach().cpu().to(index_dtype),
            "dequantized_weight_dtype": str(weight.dtype).replace("torch.", ""),
        }
        if getattr(module.cfg, "a_bits", None) is not None:
            layers[name]["activation_bits"] = int(module.cfg.a_bits)
            layers[name]["activation_centers"] = module.activation_centers.detach().float().cpu()
            layers[name]["activation_centers_initialized"] = bool(
                module.activation_centers_initialized.detach().cpu().item())
    skip = set()
    for name, _ in modules:
        skip.update({f"{name}.weight", f"{name}.centers", f"{name}.activation_centers",
                     f"{name}.activation_centers_initialized"})
    first_cfg = modules[0][1].cfg.to_dict() if modules and hasattr(modules[0][1].cfg, "to_dict") else None
    state: dict[str, Any] = {
        "format": "dimq_compact",
        "model_meta": {"num_quantized_layers": len(modules), "quantized_layer_names": [n for n, _ in modules]},
        "quant_cfg": first_cfg,
        "layers": layers,
        "non_quantized_state_dict": {k: v.detach().cpu() for k, v in model.state_dict().items() if k not in skip},
    }
    if include_model_state:
        state["model_state_dict"] = model.state_dict()
    if extra:
        state["extra"] = extra
    torch.save(state, path)
    return state


def load_compact_checkpoint(path, map_location="cpu"):
    return torch.load(Path(path), map_location=map_location)
