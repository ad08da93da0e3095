"""QAT-side use of the nearest-codeword kernel: the straight-through fake quantisation that the
reference's wrappers evaluate on every training step.

``fake_quant_weight`` (quant/dimq_wrapper.py:72-75, ``forward_mode == "hard_ste"``) computes
``weight + (hard_quantize_weight(weight, centers)[0] - weight).detach()``: forward value = the
hard-quantised weight (up to the rounding of the two additions), gradient = identity on the weight,
none on the centres (they learn through the DIMQ losses, quant/dimq.py:244-296).  The reference
builds a ``[chunk, K]`` distance matrix per chunk for that; here it is one pass over the weight in
the CUDA library.  The trainer, the losses and the wrapper classes themselves are outside this
backend's scope; this module is the drop-in for that one call.
"""

from __future__ import annotations

import torch

from . import ops


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight: torch.Tensor, centers: torch.Tensor, group_rows):
        return ops.fake_quantize_ste(weight.detach(), centers.detach(), group_rows=group_rows)

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        return grad_out, None, None


def fake_quant_weight(weight: torch.Tensor, centers: torch.Tensor, chunk_size: int | None = None, *,
                      group_rows: int | None = None) -> torch.Tensor:
    """Straight-through hard quantisation of ``weight`` to its nearest centre.

    Same value and gradients as the reference expression
    ``weight + (hard_quantize_weight(weight, centers, chunk_size)[0] - weight).detach()``.
    ``chunk_size`` is accepted for signature compatibility (the kernel needs no chunking);
    ``centers`` may be ``[G, K]`` with ``group_rows`` rows of ``weight`` per codebook (additive).
    CUDA tensors only: there is no CPU path.
    """
    if centers.numel() == 0:
        raise ValueError("centers must be non-empty")
    return _FakeQuantSTE.apply(weight, centers, group_rows)


def fake_quant_activation(x: torch.Tensor, activation_centers: torch.Tensor, chunk_size: int | None = None) -> torch.Tensor:
    """``x + (q - x).detach()`` with ``q`` the nearest activation centre (quant/dimq_wrapper.py:80-85,
    without the running update of the centres, which belongs to the trainer)."""
    return _FakeQuantSTE.apply(x, activation_centers, None)
