"""Checkpoint dictionaries and the module swap, end to end.

* ``export_packed_dimq_checkpoint`` must reproduce, key for key and byte for byte, the version-1
  dictionary the reference wrote for the same compact input
  (dimq_cuda_backend/dimq_backend/export.py:208-255; fixture made by tests/golden/make_golden.py).
* ``export_compact_checkpoint`` must write the dictionary of quant/export_dimq.py:74-105.
* A packed file goes through ``torch.save`` -> ``torch.load`` -> ``replace_modules_with_packed_dimq``
  (dimq_cuda_backend/dimq_backend/modules.py:161-172) -> GPU forward and is compared with the oracle,
  for a version-1 (W4A4) file, for the file the reference itself wrote, and for a version-2 file
  (3-bit indices, one codebook per 128 output rows, weight-only).
"""

from __future__ import annotations

import json
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import c_oracle
from oracle import dimq_oracle as o
from tests._cases import bf16_round, make_weight

GOLDEN = Path(__file__).resolve().parent / "golden"


def reference_packed_state() -> dict:
    """The packed checkpoint dictionary the reference exported, rebuilt from the fixture files."""
    meta = json.loads((GOLDEN / "packed_checkpoint_meta.json").read_text())
    with np.load(GOLDEN / "packed_checkpoint_tensors.npz") as z:
        tensors = {k: z[k] for k in z.files}
    state = {k: v for k, v in meta.items() if k != "layers"}
    state["layers"] = {}
    for lname, layer in meta["layers"].items():
        entry = {}
        for key, val in layer.items():
            if isinstance(val, dict) and "tensor" in val:
                dtype = getattr(torch, val["dtype"].replace("torch.", ""))
                entry[key] = torch.from_numpy(tensors[val["tensor"]]).to(dtype)
            else:
                entry[key] = val
        state["layers"][lname] = entry
    return state


def compact_input(golden) -> dict:
    """The compact checkpoint make_golden.py fed to the reference's exporter."""
    fc_idx = o.unpack_u4(golden["wq_lin_packed"], 48 * 96).reshape(48, 96)
    conv_idx = o.unpack_u4(golden["wq_conv_packed"], 8 * 4 * 3 * 3).reshape(8, 4, 3, 3)
    return {
        "format": "dimq_compact",
        "model_meta": {"num_quantized_layers": 2, "quantized_layer_names": ["fc", "conv"]},
        "quant_cfg": {"w_bits": 4},
        "layers": {
            "fc": {"shape": [48, 96], "bits": 4, "centers": torch.from_numpy(golden["wq_lin_cb"]),
                   "indices": torch.from_numpy(fc_idx), "dequantized_weight_dtype": "float32"},
            "conv": {"shape": [8, 4, 3, 3], "bits": 4, "centers": torch.from_numpy(golden["wq_conv_cb"]),
                     "indices": torch.from_numpy(conv_idx), "dequantized_weight_dtype": "float32"},
        },
        "non_quantized_state_dict": {"fc.bias": torch.from_numpy(golden["wq_lin_bias"])},
    }


CONV_HPARAMS = {"conv": {"type": "conv2d", "stride": [2, 2], "padding": [1, 1], "dilation": [1, 1], "groups": 1}}


def assert_same_tree(got, want, where="state"):
    """Same keys in the same order, same python values, same tensor dtypes and bytes."""
    if isinstance(want, dict):
        assert isinstance(got, dict), where
        assert list(got.keys()) == list(want.keys()), f"{where}: keys {list(got.keys())} != {list(want.keys())}"
        for k in want:
            assert_same_tree(got[k], want[k], f"{where}[{k!r}]")
    elif isinstance(want, torch.Tensor):
        assert isinstance(got, torch.Tensor), where
        assert got.dtype == want.dtype and got.shape == want.shape, f"{where}: {got.dtype}{tuple(got.shape)}"
        assert got.device.type == "cpu", where
        assert torch.equal(got, want), where
    elif isinstance(want, (list, tuple)):
        assert list(got) == list(want), f"{where}: {got!r} != {want!r}"
    else:
        assert got == want and type(got) is type(want), f"{where}: {got!r} != {want!r}"


def test_reference_fixture_agrees_with_oracle(golden):
    """CPU: the stored reference export is what the oracle's packing rule gives for the same indices."""
    state = reference_packed_state()
    assert state["format"] == "dimq_packed_lut" and state["format_version"] == 1
    for name, packed_key, cb_key, numel in (("fc", "wq_lin_packed", "wq_lin_cb", 48 * 96),
                                            ("conv", "wq_conv_packed", "wq_conv_cb", 288)):
        layer = state["layers"][name]
        idx = o.unpack_u4(golden[packed_key], numel)
        assert np.array_equal(layer["packed_weight"].numpy(), o.pack_u4(idx))
        assert np.array_equal(layer["packed_weight"].numpy(), c_oracle.pack_bits(idx, 4))
        assert torch.equal(layer["packed_weight"], layer["packed_indices"])
        assert torch.equal(layer["codebook"], torch.from_numpy(golden[cb_key]).to(torch.float16))
        assert layer["weight_numel"] == numel


@pytest.mark.gpu
def test_export_packed_v1_equals_reference_dictionary(golden, cuda_device, tmp_path):
    from dimq_b200 import export_packed_dimq_checkpoint

    want = reference_packed_state()
    out = tmp_path / "sub" / "packed.pt"
    got = export_packed_dimq_checkpoint(compact_input(golden), out, layer_hparams=CONV_HPARAMS)
    # make_golden.py stringified nothing but None-valued fields; tuples come back as lists from JSON
    for layer in got["layers"].values():
        if "kernel_size" in layer:
            layer["kernel_size"] = list(layer["kernel_size"])
    want["non_quantized_state_dict"] = {"fc.bias": torch.from_numpy(golden["wq_lin_bias"])}
    # the fixture went through JSON with sorted keys: compare in its order (the written order is
    # checked by test_export_packed_key_order_follows_reference)
    def reorder(g, w):
        if isinstance(w, dict):
            assert isinstance(g, dict) and sorted(g.keys()) == sorted(w.keys()), (sorted(g.keys()), sorted(w.keys()))
            return {k: reorder(g[k], w[k]) for k in w}
        return g

    got_cmp = reorder(got, want)
    assert_same_tree(got_cmp, want)
    # and the file on disk holds the same dictionary
    loaded = torch.load(out, map_location="cpu")
    assert list(loaded.keys()) == list(got.keys())
    assert torch.equal(loaded["layers"]["fc"]["packed_weight"], want["layers"]["fc"]["packed_weight"])


@pytest.mark.gpu
def test_export_packed_key_order_follows_reference(golden, cuda_device, tmp_path):
    """Key order of the written dictionaries (dimq_backend/export.py:208-255, read as text)."""
    from dimq_b200 import export_packed_dimq_checkpoint

    got = export_packed_dimq_checkpoint(compact_input(golden), tmp_path / "p.pt", layer_hparams=CONV_HPARAMS)
    assert list(got.keys()) == ["format", "format_version", "model_name", "source_checkpoint", "source_format",
                                "source_extra", "model_meta", "quant_cfg", "weight_encoding",
                                "activation_quantization", "layers", "non_quantized_state_dict"]
    common = ["name", "type", "bit_w", "bit_a", "weight_shape", "weight_numel", "packed_weight", "packed_indices",
              "codebook", "codebook_granularity", "act_scale", "act_zero_point", "act_qmin", "act_qmax",
              "activation_qparams", "bias"]
    assert list(got["layers"]["fc"].keys()) == common + ["layout", "out_features", "in_features"]
    assert list(got["layers"]["conv"].keys()) == common + ["layout", "out_channels", "in_channels_per_group",
                                                           "kernel_size", "stride", "padding", "dilation", "groups"]
    assert got["weight_encoding"] == "packed_u4_indices" and got["model_name"] == "dimq_packed_lut"


class _Wrapper(nn.Module):
    """Stand-in for the reference's QAT wrapper (quant/dimq_wrapper.py:172-260): a ``weight`` shared with
    the wrapped layer, a ``centers`` parameter, a ``cfg`` with ``w_bits`` / ``to_dict``."""

    def __init__(self, inner: nn.Module, centers: torch.Tensor, w_bits: int) -> None:
        super().__init__()
        self.weight = inner.weight
        self.bias = inner.bias
        self.centers = nn.Parameter(centers.clone())
        fields = {"w_bits": w_bits, "a_bits": None, "chunk_size": 262144}
        self.cfg = SimpleNamespace(**fields, to_dict=lambda: dict(fields))


@pytest.mark.gpu
def test_export_compact_checkpoint_dictionary(cuda_device, tmp_path):
    from dimq_b200 import export_compact_checkpoint, load_compact_checkpoint

    torch.manual_seed(5)
    model = nn.Sequential()
    lin, conv = nn.Linear(96, 48), nn.Conv2d(4, 8, 3, bias=False)
    # unsorted centres: the exporter sorts them (quant/export_dimq.py:71)
    c_lin = torch.from_numpy(o.quantile_codebook(lin.weight.detach().numpy(), 16))[torch.randperm(16)]
    c_conv = torch.from_numpy(o.quantile_codebook(conv.weight.detach().numpy(), 8))
    model.add_module("fc", _Wrapper(lin, c_lin, 4))
    model.add_module("conv", _Wrapper(conv, c_conv, 3))
    model.add_module("norm", nn.BatchNorm2d(8))
    path = tmp_path / "deep" / "compact.pt"
    state = export_compact_checkpoint(model, path, extra={"note": "x"})
    loaded = load_compact_checkpoint(path)
    for s in (state, loaded):
        assert list(s.keys()) == ["format", "model_meta", "quant_cfg", "layers", "non_quantized_state_dict", "extra"]
        assert s["format"] == "dimq_compact"
        assert s["model_meta"] == {"num_quantized_layers": 2, "quantized_layer_names": ["fc", "conv"]}
        assert s["quant_cfg"] == {"w_bits": 4, "a_bits": None, "chunk_size": 262144}
        assert s["extra"] == {"note": "x"}
        for name, mod, bits in (("fc", lin, 4), ("conv", conv, 3)):
            layer = s["layers"][name]
            assert list(layer.keys()) == ["shape", "bits", "centers", "indices", "dequantized_weight_dtype"]
            assert layer["shape"] == list(mod.weight.shape) and layer["bits"] == bits
            centers = layer["centers"]
            assert centers.dtype == torch.float32 and centers.device.type == "cpu"
            assert torch.equal(centers, centers.sort().values)
            assert layer["indices"].dtype == torch.uint8 and layer["indices"].shape == mod.weight.shape
            want = o.hard_quantize(mod.weight.detach().numpy(), centers.numpy())
            assert np.array_equal(layer["indices"].numpy(), want.reshape(mod.weight.shape))
            assert layer["dequantized_weight_dtype"] == "float32"
        keys = set(s["non_quantized_state_dict"].keys())
        assert "fc.bias" in keys and "norm.running_mean" in keys
        assert not keys & {"fc.weight", "fc.centers", "conv.weight", "conv.centers"}
    with_state = export_compact_checkpoint(model, tmp_path / "c2.pt", include_model_state=True)
    assert "model_state_dict" in with_state and "extra" not in with_state


class _Net(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.stem = nn.Sequential()
        self.stem.add_module("conv", nn.Conv2d(4, 8, 3, stride=2, padding=1, bias=False))
        self.fc = nn.Linear(96, 48)


@pytest.mark.gpu
@pytest.mark.parametrize("source", ["own_export", "reference_file"])
def test_v1_file_round_trip_through_module_swap(golden, cuda_device, tmp_path, source):
    """A version-1 file (ours, or the one the reference wrote) -> load -> swap -> W4A4 forward."""
    from dimq_b200 import DIMQConv2d, DIMQLinear, export_packed_dimq_checkpoint, replace_modules_with_packed_dimq

    path = tmp_path / "packed_v1.pt"
    if source == "own_export":
        export_packed_dimq_checkpoint(compact_input(golden), path, layer_hparams=CONV_HPARAMS)
    else:
        torch.save(reference_packed_state(), path)
    state = torch.load(path, map_location="cpu")
    state["layers"] = {"fc": state["layers"]["fc"], "stem.conv": state["layers"]["conv"]}
    model = replace_modules_with_packed_dimq(_Net(), state).to(cuda_device)
    assert isinstance(model.fc, DIMQLinear) and isinstance(model.stem.conv, DIMQConv2d)
    assert model.stem.conv.stride == (2, 2) and model.stem.conv.padding == (1, 1)
    cb_fc = state["layers"]["fc"]["codebook"].float().numpy()
    cb_conv = state["layers"]["stem.conv"]["codebook"].float().numpy()
    bias = state["layers"]["fc"]["bias"].float().numpy()
    x = golden["wq_lin_x"]
    got = model.fc(torch.from_numpy(x).to(cuda_device)).cpu().numpy()
    want = o.linear_lut_a4(x, golden["wq_lin_packed"], cb_fc, 1.0, 8, 48, 96, bias)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
    xc = golden["wq_conv_x"]
    got = model.stem.conv(torch.from_numpy(xc).to(cuda_device)).cpu().numpy()
    want = o.conv2d_lut_a4(xc, golden["wq_conv_packed"], cb_conv, 1.0, 8, (8, 4, 3, 3), None, stride=(2, 2),
                           padding=(1, 1))
    assert got.shape == want.shape and np.allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
def test_v2_file_round_trip_through_module_swap(cuda_device, tmp_path):
    """3-bit indices, one codebook per 128 rows, weight-only: export -> save -> load -> swap -> forward."""
    from dimq_b200 import DIMQLinear, export_packed_dimq_checkpoint, replace_modules_with_packed_dimq

    n, k = 320, 256            # last group is short (64 rows)
    case = make_weight(n, k, 3, seed=11, group_rows=128)
    rng = np.random.default_rng(2)
    bias = rng.standard_normal(n).astype(np.float32) * 0.1
    compact = {
        "format": "dimq_compact", "model_meta": {"num_quantized_layers": 1, "quantized_layer_names": ["fc"]},
        "quant_cfg": None,
        "layers": {"fc": {"shape": [n, k], "bits": 3, "centers": torch.from_numpy(case["codebooks"]),
                          "indices": torch.from_numpy(case["idx"]), "group_rows": 128,
                          "dequantized_weight_dtype": "float32"}},
        "non_quantized_state_dict": {"fc.bias": torch.from_numpy(bias)},
    }
    path = tmp_path / "packed_v2.pt"
    written = export_packed_dimq_checkpoint(compact, path, weight_only=True)
    assert written["format_version"] == 2 and written["weight_encoding"] == "packed_bitstream_indices"
    state = torch.load(path, map_location="cpu")
    layer = state["layers"]["fc"]
    assert layer["bit_w"] == 3 and layer["group_rows"] == 128 and layer["codebook_granularity"] == "per_row_group"
    assert layer["act_scale"] is None and tuple(layer["codebook"].shape) == (3, 8)
    assert np.array_equal(layer["packed_weight"].numpy(), case["packed"])

    class Net(nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.fc = nn.Linear(k, n)

    model = replace_modules_with_packed_dimq(Net(), state, out_dtype=torch.float32).to(cuda_device)
    assert isinstance(model.fc, DIMQLinear) and model.fc.bits == 3 and model.fc.group_rows == 128
    books = layer["codebook"].float().numpy()            # the stored (fp16-rounded) codebooks
    bias16 = layer["bias"].float().numpy()
    for m in (5, 700):                                   # index-streaming and tensor-core regimes
        x = bf16_round(rng.standard_normal((m, k)).astype(np.float32))
        got = model.fc(torch.from_numpy(x).to(cuda_device, torch.bfloat16)).float().cpu().numpy()
        want = o.linear_wq(x, case["packed"], books, 3, n, k, bias16, 128)
        max_abs, rel = o.parity_metrics(got, want)
        assert max_abs <= 1e-2 and rel <= 1e-3, (m, max_abs, rel)


@pytest.mark.gpu
def test_conv_module_sees_reloaded_weights(cuda_device):
    """The re-ordered index copy of the tensor-core convolution follows ``load_state_dict``."""
    from dimq_b200 import DIMQConv2d

    rng = np.random.default_rng(4)
    shape = (64, 64, 3, 3)
    cb = np.sort(rng.standard_normal(16).astype(np.float16)).astype(np.float32)
    x = bf16_round(np.maximum(rng.standard_normal((2, 64, 12, 12)), 0).astype(np.float32))
    xt = torch.from_numpy(x).to(cuda_device, torch.bfloat16).contiguous(memory_format=torch.channels_last)

    def packed_for(seed):
        idx = np.random.default_rng(seed).integers(0, 16, size=shape, dtype=np.uint8)
        return c_oracle.pack_bits(idx.reshape(-1), 4)

    p0, p1 = packed_for(0), packed_for(1)
    mod = DIMQConv2d(torch.from_numpy(p0), torch.from_numpy(cb).half(), None, None, shape, None, stride=1,
                     padding=1, out_dtype=torch.float32).to(cuda_device)
    for packed in (p0, p1):
        sd = mod.state_dict()
        sd["packed_weight"] = torch.from_numpy(packed)
        mod.load_state_dict(sd)
        got = mod(xt).float().cpu().numpy()
        want = o.conv2d_wq(x, packed, cb[None, :], 4, shape, None, stride=(1, 1), padding=(1, 1))
        max_abs, rel = o.parity_metrics(got, want)
        assert max_abs <= 1e-2 and rel <= 1e-3, (max_abs, rel)
