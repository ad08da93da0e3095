"""Generate the golden vectors under tests/golden/ from the DIMQ reference.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/DIMQ

It imports the reference's own Python functions (``quant.dimq``,
``dimq_backend.export``, ``dimq_backend.reference``) on CPU, feeds them seeded
inputs — the shapes of the reference's tests plus edge cases — and stores
inputs and outputs as ``.npz``.  The files are committed; the tests never need
the reference checkout again.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ref / "dimq_cuda_backend"))
    from quant.dimq import hard_quantize_weight, init_centers_1d
    from dimq_backend.export import (
        assign_weight_indices,
        export_packed_dimq_checkpoint,
        pack_u4_indices,
        unpack_u4_indices,
    )
    from dimq_backend.reference import (
        build_product_table,
        dequantize_packed_weight,
        dimq_conv2d_lut_reference,
        dimq_conv2d_reference,
        dimq_linear_dequant_reference,
        dimq_linear_reference,
        quantize_activation_u4,
    )
    import torch.nn.functional as F

    torch.set_num_threads(1)
    out: dict[str, np.ndarray] = {}

    # ---- pack / unpack (u4) -------------------------------------------------
    g = torch.Generator().manual_seed(0)
    pack_cases = {
        "arange17": torch.arange(17, dtype=torch.uint8) % 16,
        "arange257x7": (torch.arange(257, dtype=torch.uint8) * 7) % 16,
        "n1": torch.tensor([13], dtype=torch.uint8),
        "n2": torch.tensor([1, 15], dtype=torch.uint8),
        "allmax9": torch.full((9,), 15, dtype=torch.uint8),
        "rand4099": torch.randint(0, 16, (4099,), generator=g, dtype=torch.uint8),
        "rand2d": torch.randint(0, 16, (6, 11), generator=g, dtype=torch.uint8),
    }
    for name, idx in pack_cases.items():
        packed = pack_u4_indices(idx)
        restored = unpack_u4_indices(packed, idx.numel())
        assert torch.equal(restored, idx.reshape(-1))
        out[f"pack_{name}_idx"] = idx.numpy()
        out[f"pack_{name}_packed"] = packed.numpy()

    # ---- hard quantisation --------------------------------------------------
    torch.manual_seed(0)
    w = torch.randn(20000) * 0.02
    for k in (4, 8, 16, 256):
        centers = init_centers_1d(w, k, "quantile")
        vals, idx = hard_quantize_weight(w, centers)
        out[f"hq_k{k}_w"] = w.numpy()
        out[f"hq_k{k}_centers"] = centers.numpy()
        out[f"hq_k{k}_idx"] = idx.to(torch.uint8).numpy()
        out[f"hq_k{k}_vals"] = vals.numpy()
        if k <= 16:
            assert torch.equal(assign_weight_indices(w, centers), idx.to(torch.uint8))
    # the reference's own unit-test input (tests/test_dimq_math.py:35-43)
    w_lin = torch.linspace(-2.0, 2.0, 101)
    c3 = torch.tensor([-1.0, 0.0, 1.0])
    _, idx = hard_quantize_weight(w_lin, c3, chunk_size=17)
    out["hq_lin_w"] = w_lin.numpy()
    out["hq_lin_centers"] = c3.numpy()
    out["hq_lin_idx"] = idx.to(torch.uint8).numpy()
    # adversarial values: exact midpoints, duplicates, infinities, NaN, denormals
    w_adv = torch.tensor(
        [0.5, 1.5, 2.5, -0.5, 0.0, 1.0, float("inf"), float("-inf"), float("nan"), 1e-40, -1e-40,
         3.4e38, -3.4e38, 1.0000001, 0.9999999, 2.0, 1.25, 1.75],
        dtype=torch.float32,
    )
    adv_books = {
        "sorted": torch.tensor([0.0, 1.0, 2.0, 3.0]),
        "dups": torch.tensor([0.0, 1.0, 1.0, 2.0]),
        "unsorted": torch.tensor([2.0, -1.0, 1.0, 0.0]),
        "withnan": torch.tensor([0.0, 1.0, float("nan"), 2.0]),
        "withinf": torch.tensor([float("-inf"), 0.0, 1.0, float("inf")]),
        "tiny": torch.tensor([-1e-40, 0.0, 1e-40, 1e-39]),
    }
    out["hq_adv_w"] = w_adv.numpy()
    for name, cb in adv_books.items():
        _, idx = hard_quantize_weight(w_adv, cb)
        out[f"hq_adv_{name}_centers"] = cb.numpy()
        out[f"hq_adv_{name}_idx"] = idx.to(torch.uint8).numpy()

    # quantile codebooks on slices (the grouped-codebook extension is the
    # reference function applied slice by slice)
    torch.manual_seed(1)
    w2 = torch.randn(24, 40) * 0.02
    out["grp_w"] = w2.numpy()
    cbs, idxs = [], []
    for g0 in range(0, 24, 8):
        c = init_centers_1d(w2[g0 : g0 + 8], 8, "quantile")
        _, i = hard_quantize_weight(w2[g0 : g0 + 8], c)
        cbs.append(c.numpy())
        idxs.append(i.to(torch.uint8).numpy())
    out["grp_codebooks"] = np.stack(cbs)
    out["grp_idx"] = np.concatenate(idxs, axis=0)

    # ---- activation quantiser / product table -------------------------------
    torch.manual_seed(2)
    xq = torch.cat([
        torch.randn(300) * 2.0,
        torch.arange(-20, 21, dtype=torch.float32) * 0.125 * 0.5,   # exact .5 boundaries at scale .125
        torch.tensor([1e30, -1e30, float("inf"), float("-inf"), 0.0, -0.0, 1e-30]),
    ])
    out["aq_x"] = xq.numpy()
    aq_grid = [(0.125, 8), (0.2, 7), (1.0, 0), (0.25, 15), (3.0, 3)]
    out["aq_grid"] = np.array(aq_grid, dtype=np.float64)
    for i, (s, z) in enumerate(aq_grid):
        out[f"aq_q{i}"] = quantize_activation_u4(xq, s, int(z)).numpy()
    cb16_h = torch.linspace(-1.0, 1.0, 16, dtype=torch.float16)
    cb16_f = torch.linspace(-0.5, 0.5, 16)
    out["pt_cb_f16_as_f32"] = cb16_h.float().numpy()
    out["pt_table_f16"] = build_product_table(cb16_h, 0.125, 8).numpy()
    out["pt_cb_f32"] = cb16_f.numpy()
    out["pt_table_f32"] = build_product_table(cb16_f, 0.2, 7).numpy()

    # ---- W4A4 linear (shapes of dimq_cuda_backend/tests/test_cuda_ops.py:51-64) ----
    torch.manual_seed(3)
    x = torch.randn(4, 11)
    cb = torch.linspace(-0.5, 0.5, 16)
    widx = torch.randint(0, 16, (6, 11), dtype=torch.uint8)
    packed = pack_u4_indices(widx)
    bias = torch.randn(6)
    out["lin_x"] = x.numpy()
    out["lin_cb"] = cb.numpy()
    out["lin_widx"] = widx.numpy()
    out["lin_packed"] = packed.numpy()
    out["lin_bias"] = bias.numpy()
    out["lin_y_lut"] = dimq_linear_reference(x, packed, cb, 0.2, 7, 6, 11, bias).numpy()
    out["lin_y_deq"] = dimq_linear_dequant_reference(x, packed, cb, 0.2, 7, 6, 11, bias).numpy()
    out["lin_y_nobias"] = dimq_linear_reference(x, packed, cb, 0.2, 7, 6, 11, None).numpy()
    # batched leading dims, bigger K
    torch.manual_seed(5)
    xb = torch.randn(2, 5, 64)
    widx_b = torch.randint(0, 16, (24, 64), dtype=torch.uint8)
    packed_b = pack_u4_indices(widx_b)
    cbb = (torch.randn(16) * 0.05).sort().values
    out["linb_x"] = xb.numpy()
    out["linb_cb"] = cbb.numpy()
    out["linb_packed"] = packed_b.numpy()
    out["linb_y_lut"] = dimq_linear_reference(xb, packed_b, cbb, 0.3, 8, 24, 64, None).numpy()

    # ---- W4A4 conv (shapes of test_cuda_ops.py:67-93) -----------------------
    torch.manual_seed(4)
    xc = torch.randn(2, 3, 6, 7)
    cbc = torch.linspace(-0.75, 0.75, 16)
    cidx = torch.randint(0, 16, (5, 3, 3, 3), dtype=torch.uint8)
    cpacked = pack_u4_indices(cidx)
    cbias = torch.randn(5)
    kw = dict(stride=(2, 1), padding=(1, 1), dilation=(1, 1), groups=1)
    out["conv_x"] = xc.numpy()
    out["conv_cb"] = cbc.numpy()
    out["conv_widx"] = cidx.numpy()
    out["conv_packed"] = cpacked.numpy()
    out["conv_bias"] = cbias.numpy()
    out["conv_y_deq"] = dimq_conv2d_reference(xc, cpacked, cbc, 0.25, 7, cidx.shape, cbias, **kw).numpy()
    out["conv_y_lut"] = dimq_conv2d_lut_reference(xc, cpacked, cbc, 0.25, 7, cidx.shape, cbias, **kw).numpy()
    # groups and dilation
    torch.manual_seed(6)
    xg = torch.randn(2, 4, 9, 8)
    gidx = torch.randint(0, 16, (6, 2, 3, 2), dtype=torch.uint8)
    gpacked = pack_u4_indices(gidx)
    kwg = dict(stride=(1, 2), padding=(2, 1), dilation=(2, 1), groups=2)
    out["convg_x"] = xg.numpy()
    out["convg_widx"] = gidx.numpy()
    out["convg_packed"] = gpacked.numpy()
    out["convg_y_deq"] = dimq_conv2d_reference(xg, gpacked, cbc, 0.25, 7, gidx.shape, None, **kwg).numpy()

    # ---- weight-only path: dequantize_packed_weight + F.linear / F.conv2d ---
    torch.manual_seed(7)
    ww = torch.randn(48, 96) * 0.02
    cbw = init_centers_1d(ww, 16, "quantile")
    _, wi = hard_quantize_weight(ww, cbw)
    wpacked = pack_u4_indices(wi.to(torch.uint8))
    xw = torch.randn(10, 96)
    bw = torch.randn(48) * 0.1
    w_hat = dequantize_packed_weight(wpacked, cbw, (48, 96))
    out["wq_lin_w"] = ww.numpy()
    out["wq_lin_cb"] = cbw.numpy()
    out["wq_lin_packed"] = wpacked.numpy()
    out["wq_lin_x"] = xw.numpy()
    out["wq_lin_bias"] = bw.numpy()
    out["wq_lin_what"] = w_hat.numpy()
    out["wq_lin_y"] = F.linear(xw, w_hat, bw).numpy()
    torch.manual_seed(8)
    wc = torch.randn(8, 4, 3, 3) * (2.0 / 36) ** 0.5
    cbwc = init_centers_1d(wc, 16, "quantile")
    _, wci = hard_quantize_weight(wc, cbwc)
    wcpacked = pack_u4_indices(wci.to(torch.uint8))
    xwc = torch.relu(torch.randn(2, 4, 10, 9))
    w_hat_c = dequantize_packed_weight(wcpacked, cbwc, (8, 4, 3, 3))
    out["wq_conv_cb"] = cbwc.numpy()
    out["wq_conv_packed"] = wcpacked.numpy()
    out["wq_conv_x"] = xwc.numpy()
    out["wq_conv_y"] = F.conv2d(xwc, w_hat_c, None, 1, 1).numpy()
    out["wq_conv_y_s2"] = F.conv2d(xwc, w_hat_c, None, 2, 1).numpy()

    np.savez_compressed(HERE / "reference_vectors.npz", **out)

    # ---- packed checkpoint layout (dimq_backend/export.py:159-260) ----------
    compact = {
        "format": "dimq_compact",
        "model_meta": {"num_quantized_layers": 2, "quantized_layer_names": ["fc", "conv"]},
        "quant_cfg": {"w_bits": 4},
        "layers": {
            "fc": {"shape": [48, 96], "bits": 4, "centers": cbw, "indices": wi.to(torch.uint8),
                   "dequantized_weight_dtype": "float32"},
            "conv": {"shape": [8, 4, 3, 3], "bits": 4, "centers": cbwc, "indices": wci.to(torch.uint8),
                     "dequantized_weight_dtype": "float32"},
        },
        "non_quantized_state_dict": {"fc.bias": bw},
    }
    state = export_packed_dimq_checkpoint(
        compact, HERE / "_tmp_packed.pt",
        layer_hparams={"conv": {"type": "conv2d", "stride": [2, 2], "padding": [1, 1], "dilation": [1, 1], "groups": 1}},
    )
    (HERE / "_tmp_packed.pt").unlink()
    tensors: dict[str, np.ndarray] = {}
    meta: dict[str, object] = {k: v for k, v in state.items() if k not in ("layers", "non_quantized_state_dict")}
    meta["layers"] = {}
    for lname, layer in state["layers"].items():
        entry = {}
        for key, val in layer.items():
            if isinstance(val, torch.Tensor):
                tensors[f"{lname}.{key}"] = val.float().numpy() if val.is_floating_point() else val.numpy()
                entry[key] = {"tensor": f"{lname}.{key}", "dtype": str(val.dtype)}
            else:
                entry[key] = val
        meta["layers"][lname] = entry
    np.savez_compressed(HERE / "packed_checkpoint_tensors.npz", **tensors)
    (HERE / "packed_checkpoint_meta.json").write_text(json.dumps(meta, indent=1, sort_keys=True, default=str))
    print("wrote", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/DIMQ")
    main(sys.argv[1])
