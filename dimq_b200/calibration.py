"""Activation calibration for the W4A4 mode: collect per-layer input ranges over a few batches and turn
them into the per-tensor affine u4 parameters the packed checkpoint stores.

The reference has the formula (``activation_qparams_from_minmax``, dimq_backend/export.py:81-111) and
the place the result goes (``act_qparams`` of ``export_packed_dimq_checkpoint``, :159-260), but nothing
that produces the min/max; without them its export falls back to scale 1.0 / zero point 8
(``default_activation_qparams``, :114-125).  This module is that missing pass.
"""

from __future__ import annotations

from typing import Any, Callable, Iterable

import torch
import torch.nn as nn

from .export import activation_qparams_from_minmax
from .modules import DIMQConv2d, DIMQLinear


class ActivationRangeCollector:
    """Forward pre-hooks that keep the running min / max of the first input of every selected module.

    The reductions run on the input's device and stay there (two scalars per module); ``ranges()``
    moves them to the host once.
    """

    def __init__(self, model: nn.Module, select: Callable[[str, nn.Module], bool] | None = None) -> None:
        if select is None:
            select = lambda name, module: isinstance(module, (DIMQLinear, DIMQConv2d, nn.Linear, nn.Conv2d))
        self._stats: dict[str, list[torch.Tensor]] = {}
        self._handles = []
        for name, module in model.named_modules():
            if name and select(name, module):
                self._handles.append(module.register_forward_pre_hook(self._hook(name)))

    def _hook(self, name: str):
        def record(module, args):
            x = args[0].detach()
            if x.numel() == 0:
                return
            lo, hi = torch.aminmax(x.float())
            if name in self._stats:
                cur = self._stats[name]
                cur[0] = torch.minimum(cur[0], lo)
                cur[1] = torch.maximum(cur[1], hi)
            else:
                self._stats[name] = [lo, hi]
        return record

    def ranges(self) -> dict[str, tuple[float, float]]:
        return {name: (float(lo.item()), float(hi.item())) for name, (lo, hi) in self._stats.items()}

    def remove(self) -> None:
        for handle in self._handles:
            handle.remove()
        self._handles.clear()

    def __enter__(self) -> "ActivationRangeCollector":
        return self

    def __exit__(self, *exc) -> None:
        self.remove()


@torch.no_grad()
def calibrate_activation_qparams(model: nn.Module, batches: Iterable[Any], *,
                                 select: Callable[[str, nn.Module], bool] | None = None,
                                 forward: Callable[[nn.Module, Any], Any] | None = None) -> dict[str, dict[str, Any]]:
    """Run ``model`` over ``batches`` and return ``{module name: u4 activation qparams}`` — the mapping
    ``export_packed_dimq_checkpoint(act_qparams=...)`` and :func:`apply_activation_qparams` take."""
    with ActivationRangeCollector(model, select) as collector:
        for batch in batches:
            if forward is not None:
                forward(model, batch)
            elif isinstance(batch, (tuple, list)):
                model(*batch)
            else:
                model(batch)
        ranges = collector.ranges()
    out = {}
    for name, (lo, hi) in ranges.items():
        q = activation_qparams_from_minmax(lo, hi)
        q["source"] = "calibrated_minmax"
        q["observed_min"], q["observed_max"] = lo, hi
        out[name] = q
    return out


def apply_activation_qparams(model: nn.Module, qparams: dict[str, dict[str, Any]]) -> int:
    """Switch the packed 4-bit layers named in ``qparams`` to the W4A4 mode with those parameters
    (layers with other bit widths or grouped codebooks stay weight-only).  Returns how many were set."""
    count = 0
    for name, module in model.named_modules():
        if name in qparams and isinstance(module, (DIMQLinear, DIMQConv2d)):
            if module.bits != 4 or module.codebook.numel() != 16:
                continue
            module.act_scale = float(qparams[name]["scale"])
            module.act_zero_point = int(qparams[name]["zero_point"])
            count += 1
    return count
