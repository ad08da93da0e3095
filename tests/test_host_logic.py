"""CPU-only checks: the C ABI loads and exports what the header declares, argument validation
happens on the host before any launch, and the batch-sharding logic works across 2 gloo ranks."""

from __future__ import annotations

import ctypes as C
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from dimq_b200 import _lib
    from dimq_b200.build import build

    build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(lib):
    from dimq_b200 import _lib

    header = (ROOT / "include" / "dimq_b200.h").read_text()
    declared = set(re.findall(r"DIMQ_API\s+[\w\s\*]+?\b(dimq_\w+)\s*\(", header))
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.dimq_version() >= 100
    assert lib.dimq_status_string(0).decode() == "ok"
    assert "bit width" in lib.dimq_status_string(-4).decode()


def test_argument_errors_are_reported_without_a_gpu(lib):
    null = C.c_void_p(0)
    one = C.c_void_p(16)
    assert lib.dimq_pack_bits(one, C.c_int64(8), 5, one, null) == -4          # bad bit width
    assert lib.dimq_pack_bits(one, C.c_int64(-1), 4, one, null) == -2         # bad size
    assert lib.dimq_pack_bits(null, C.c_int64(8), 4, one, null) == -1         # null pointer
    assert lib.dimq_pack_bits(null, C.c_int64(0), 4, null, null) == 0         # empty input: nothing to do
    assert lib.dimq_quantize_activation_u4(one, 0, C.c_int64(4), C.c_float(0.0), 3, one, null) == -5
    assert lib.dimq_quantize_activation_u4(one, 0, C.c_int64(4), C.c_float(1.0), 16, one, null) == -5
    assert lib.dimq_quantize_activation_u4(one, 7, C.c_int64(4), C.c_float(1.0), 3, one, null) == -3
    assert lib.dimq_build_product_table(one, 0, C.c_int64(1), 300, C.c_float(1.0), 3, one, null) == -2
    assert lib.dimq_hard_quantize(one, 0, C.c_int64(2), C.c_int64(2), one, 16, C.c_int64(1), null, one, 2, null) == -4
    assert lib.dimq_linear_lut(one, 0, one, one, 0, C.c_float(1.0), 3, null, 0, one, C.c_int64(1), C.c_int64(0),
                               C.c_int64(4), null) == -2


def test_linear_module_builds_tiled_indices_only_where_the_small_m_kernel_takes_them():
    """DIMQLinear's lazy second copy of the indices: no copy for many rows, a short K, a small weight or fp32
    activations; where one is due, building it needs the GPU (no CPU fallback: it raises)."""
    from dimq_b200.modules import DIMQLinear

    def layer(n, k, bits=4):
        return DIMQLinear(torch.zeros(n * k * bits // 8, dtype=torch.uint8), torch.zeros(1 << bits), None, None, n, k,
                          bits=bits)

    big = layer(1024, 4096)                                  # 2 MB of indices
    x16 = torch.zeros(4, 4096, dtype=torch.bfloat16)
    assert big._prepacked(64, x16) is None                   # more than 16 rows
    assert big._prepacked(4, x16.float()) is None            # fp32 activations
    assert layer(4096, 1024)._prepacked(4, x16[:, :1024]) is None   # K below 2048
    assert layer(256, 4096)._prepacked(4, x16) is None       # 0.5 MB of indices
    assert layer(1024, 4096, bits=8)._prepacked(4, x16) is None
    with pytest.raises(RuntimeError):
        big._prepacked(4, x16)                               # due, but these are CPU tensors


def test_linear_prepack_argument_errors(lib):
    buf = (C.c_uint8 * 64)()
    assert lib.dimq_linear_prepack(None, 4, C.c_int64(16), C.c_int64(128), buf, None) == -1   # null pointer
    for bits, n, k in ((8, 16, 128), (4, 24, 128), (4, 16, 192), (4, 0, 128)):
        assert lib.dimq_linear_prepack(buf, bits, C.c_int64(n), C.c_int64(k), buf, None) < 0, (bits, n, k)


def test_small_m_kernel_plan_through_the_workspace_queries(lib):
    """How the register-resident small-M kernel cuts K into slices of 2048, read off the scratch it asks for
    (slices worked on at a time x M x N floats; nothing with one slice).  Host logic only: no launch."""
    from dimq_b200 import _lib

    fake = 1 << 20                                   # an aligned address that is never dereferenced
    need = C.c_int64(-1)

    def query(fn, m, n, k, bits=4, x_dtype=_lib.BF16, x=fake):
        w = _lib.WqWeight(fake, bits, fake, _lib.F16, 1 << bits, 1, n, None)
        rc = fn(C.c_void_p(x), x_dtype, C.byref(w), C.c_int64(m), C.c_int64(n), C.c_int64(k), C.byref(need))
        return rc, need.value

    forced = lib.dimq_linear_wq_regs_workspace_bytes
    assert query(forced, 8, 4096, 8192) == (0, 4 * 8 * 4096 * 4)        # four slices at a time
    assert query(forced, 1, 4096, 4096) == (0, 2 * 1 * 4096 * 4)
    assert query(forced, 16, 4096, 2048) == (0, 0)                      # one slice: no scratch
    assert query(forced, 3, 4096, 11008) == (0, 3 * 3 * 4096 * 4)       # 5.4 -> 6 slices, three at a time, two passes
    assert query(forced, 3, 64, 22528) == (0, 0)                        # 11 slices: a prime, one at a time
    assert query(forced, 3, 64, 16384) == (0, 4 * 3 * 64 * 4)           # 8 slices: four at a time, two passes
    for m, n, k, kw in ((17, 64, 2048, {}), (4, 72, 2048, {}), (4, 64, 1024, {}), (4, 64, 2112, {}),
                        (4, 64, 2048, {"bits": 8}), (4, 64, 2048, {"x_dtype": _lib.F32}), (4, 64, 2048, {"x": fake + 8})):
        assert query(forced, m, n, k, **kw)[0] < 0, (m, n, k, kw)       # rows, N % 16, K, bits, dtype, alignment
    # the automatic choice takes it from 2 MB of indices on; below that the call needs no scratch
    auto = lib.dimq_linear_wq_workspace_bytes
    assert query(auto, 4, 1024, 4096) == (0, 2 * 4 * 1024 * 4)
    assert query(auto, 4, 512, 4096) == (0, 0)
    assert query(auto, 4, 4096, 1024) == (0, 0)                         # K below 2048: the index-streaming kernel


def test_conv_geometry(lib):
    from dimq_b200._lib import ConvGeom

    g = ConvGeom()
    g.batch, g.in_channels, g.in_h, g.in_w = 2, 3, 6, 7
    g.out_channels, g.in_channels_per_group, g.kernel_h, g.kernel_w = 5, 3, 3, 3
    g.stride_h, g.stride_w, g.pad_h, g.pad_w, g.dilation_h, g.dilation_w, g.groups = 2, 1, 1, 1, 1, 1, 1
    assert lib.dimq_conv_out_size(C.byref(g)) == 0
    assert (g.out_h, g.out_w) == (3, 7)      # dimq_cuda_backend/csrc/dimq_conv2d_lut.cu:129-130
    g.in_channels = 4
    assert lib.dimq_conv_out_size(C.byref(g)) == -6
    g.in_channels, g.kernel_h = 3, 9
    assert lib.dimq_conv_out_size(C.byref(g)) == -6


def test_ops_module_registers_reference_schemas():
    import dimq_b200  # noqa: F401

    for name in ("pack_u4", "unpack_u4", "quantize_activation_u4", "build_product_table", "linear_lut", "conv2d_lut"):
        assert hasattr(torch.ops.dimq, name)
    with pytest.raises(NotImplementedError):
        torch.ops.dimq.pack_u4(torch.zeros(4, dtype=torch.uint8))  # CUDA dispatch key only, as in the reference
    from dimq_b200.modules import DIMQLinear

    layer = DIMQLinear(torch.zeros(8, dtype=torch.uint8), torch.zeros(16), 1.0, 8, 4, 4)
    with pytest.raises(RuntimeError):
        layer(torch.zeros(1, 4))  # no CPU fallback
    with pytest.raises(ValueError):
        DIMQLinear(torch.zeros(8, dtype=torch.uint8), torch.zeros(8), 1.0, 8, 4, 4, bits=3)


def test_activation_qparams_helpers():
    from dimq_b200 import export

    q = export.activation_qparams_from_minmax(-1.0, 2.0)
    assert q["scale"] == pytest.approx(0.2) and q["zero_point"] == 5 and q["qmax"] == 15
    assert export.activation_qparams_from_minmax(3.0, 3.0)["scale"] == 1.0
    assert export.default_activation_qparams()["zero_point"] == 8
    with pytest.raises(ValueError):
        export.activation_qparams_from_minmax(float("nan"), 1.0)


def test_shard_bounds():
    from dimq_b200.dist import shard_bounds

    assert [shard_bounds(256, r, 8) for r in (0, 7)] == [(0, 32), (224, 256)]
    spans = [shard_bounds(10, r, 4) for r in range(4)]
    assert spans == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(ValueError):
        shard_bounds(4, 4, 4)


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from dimq_b200.dist import shard_bounds, gather_logits
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
for total in (8, 7):
    full = torch.arange(total * 3, dtype=torch.float32).reshape(total, 3)
    b, e = shard_bounds(total, rank, 2)
    out = gather_logits(full[b:e] * 1.0, total)
    assert torch.equal(out, full), (rank, total)
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_gather_logits_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT), port, str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("ok" in o for o in outs)


def test_default_build_has_no_diagnostics(lib):
    """The shipped library neither reads diagnostic switches from the environment nor takes a device
    pointer from it: the counters and role-skipping switches exist only in the -DDIMQ_B200_DIAG build."""
    from dimq_b200 import _lib

    assert not hasattr(lib, "dimq_diag_configure")
    blob = _lib.LIB_PATH.read_bytes()
    for name in (b"DIMQ_B200_PROFILE_PTR", b"DIMQ_B200_TC_DEBUG", b"DIMQ_B200_TC_REP"):
        assert name not in blob, name
    sources = "".join(p.read_text() for p in (ROOT / "dimq_b200" / "csrc").iterdir())
    assert sources.count("getenv(") == 1 and 'getenv("DIMQ_B200_TC_EPI")' in sources
