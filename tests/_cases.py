"""Seeded synthetic workloads shared by the parity tests (numpy, CPU)."""

from __future__ import annotations

import numpy as np

from oracle import c_oracle
from oracle import dimq_oracle as o


def make_weight(n_out: int, k_in: int, bits: int, seed: int, *, group_rows: int | None = None, std: float = 0.02,
                cb_dtype=np.float16):
    """N(0, std) weight -> quantile codebooks (per layer or per `group_rows` rows) -> indices -> packed stream.

    The codebook is rounded to `cb_dtype` first (a numpy dtype, or "bf16"; the packed export stores
    fp16) and the SAME rounded codebook is what both the oracle and the kernel see.
    """
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n_out, k_in)) * std).astype(np.float32)
    entries = 1 << bits
    if group_rows is None:
        cbs = o.quantile_codebook(w, entries)[None, :]
        grp = n_out
    else:
        grp = group_rows
        cbs = np.stack([o.quantile_codebook(w[g0 : g0 + grp], entries) for g0 in range(0, n_out, grp)])
    cbs = bf16_round(cbs) if cb_dtype == "bf16" else cbs.astype(cb_dtype).astype(np.float32)
    idx = c_oracle.hard_quantize(w, cbs, grp)
    packed = c_oracle.pack_bits(idx, bits)
    return {"w": w, "codebooks": cbs, "idx": idx, "packed": packed, "group_rows": grp, "bits": bits}


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to bf16 (nearest even) and return as fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)
