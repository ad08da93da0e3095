"""GPU parity of the large-M form of the weight-only ops — index stream expanded once to a 16-bit
weight, then the dense TMA + tcgen05 GEMM / implicit-GEMM convolution — against the CPU oracle.

Through the C ABI (``dimq_linear_wq_expand`` / ``dimq_conv2d_wq_expand`` when forced,
``dimq_linear_wq_ws`` / ``dimq_conv2d_wq_ws`` for the automatic choice).  fp32 outputs are held to
max-abs 1e-2 / relative L2 1e-3 against dequantise-then-fp32 ``F.linear`` / ``F.conv2d`` on the same
16-bit-rounded inputs; 16-bit outputs add their own rounding (2^-9 relative).
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import dimq_oracle as o
from tests._cases import bf16_round, make_weight

pytestmark = pytest.mark.gpu

MAX_ABS, REL_L2 = 1e-2, 1e-3
MAX_ABS_16, REL_L2_16 = 3e-2, 4e-3      # 16-bit output: rounding of y included


@pytest.fixture(scope="module")
def ops(cuda_device):
    from dimq_b200 import ops as _ops

    _ops.require_extension()
    return _ops


def _cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _round_to(x: np.ndarray, dtype: torch.dtype) -> np.ndarray:
    return bf16_round(x) if dtype == torch.bfloat16 else x.astype(np.float16).astype(np.float32)


LINEAR_CASES = [
    # m, k, n, bits, group_rows
    (128, 64, 64, 4, None),        # one tile, the 64-row weight tile
    (129, 64, 8, 2, None),         # one row past a tile; 8 features
    (300, 192, 320, 3, 128),       # short last codebook group, short last feature tile
    (1000, 768, 1000, 3, 128),     # the ViT head's width at many rows
    (777, 1024, 136, 2, None),
    (2048, 512, 264, 8, None),
    (1536, 256, 768, 4, 1),        # one codebook per row
]


@pytest.mark.parametrize("case", LINEAR_CASES)
@pytest.mark.parametrize("mode", ["bf16_x_bf16_cb", "bf16_x_fp16_cb", "fp16_x_fp16_cb"])
def test_linear_expand_fp32_out(ops, case, mode):
    m, k, n, bits, grp = case
    x_t = torch.float16 if mode.startswith("fp16") else torch.bfloat16
    cb_t = torch.bfloat16 if mode.endswith("bf16_cb") else torch.float16
    cw = make_weight(n, k, bits, seed=m + n, group_rows=grp, cb_dtype="bf16" if cb_t == torch.bfloat16 else np.float16)
    rng = np.random.default_rng(k)
    x = _round_to(rng.standard_normal((m, k)).astype(np.float32), x_t)
    bias = rng.standard_normal(n).astype(np.float32)
    want = o.linear_wq(x, cw["packed"], cw["codebooks"], bits, n, k, bias, cw["group_rows"])
    got = ops.dimq_linear_wq(_cuda(x, x_t), _cuda(cw["packed"]), _cuda(cw["codebooks"], cb_t), _cuda(bias), n, k,
                             bits=bits, group_rows=grp, algo="expand")
    assert ops.last_device_status() == 0
    assert got.dtype == torch.float32 and tuple(got.shape) == (m, n)
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= MAX_ABS and rel <= REL_L2, (case, mode, max_abs, rel)


@pytest.mark.parametrize("y_t", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("epi", [None, "relu", "gelu", "add_relu"])
@pytest.mark.parametrize("with_res", [False, True])
def test_linear_expand_epilogues(ops, y_t, epi, with_res):
    if epi == "add_relu" and not with_res:
        pytest.skip("add_relu without a residual is relu")
    m, k, n = 700, 256, 392
    cw = make_weight(n, k, 4, seed=3, cb_dtype="bf16")
    rng = np.random.default_rng(9)
    x = bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    bias = bf16_round(rng.standard_normal(n).astype(np.float32))
    res = _round_to(rng.standard_normal((m, n)).astype(np.float32), y_t) if with_res else None
    lin = o.linear_wq(x, cw["packed"], cw["codebooks"], 4, n, k, bias)
    if epi == "add_relu":
        want = np.maximum(lin + res, 0)
    else:
        act = {None: lambda v: v, "relu": lambda v: np.maximum(v, 0),
               "gelu": lambda v: F.gelu(torch.from_numpy(v)).numpy()}[epi](lin)
        want = act + res if with_res else act
    got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16),
                             _cuda(bias, torch.bfloat16), n, k, bits=4, algo="expand", out_dtype=y_t, epilogue=epi,
                             residual=None if res is None else _cuda(res, y_t))
    assert got.dtype == y_t and ops.last_device_status() == 0
    max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
    tol = (MAX_ABS, REL_L2) if y_t == torch.float32 else (MAX_ABS_16, REL_L2_16)
    assert max_abs <= tol[0] and rel <= tol[1], (y_t, epi, with_res, max_abs, rel)


def test_linear_auto_takes_the_expanded_form_at_many_rows(ops):
    from dimq_b200 import _lib

    k, n = 512, 768
    cw = make_weight(n, k, 3, seed=21, group_rows=128, cb_dtype="bf16")
    packed, cb = _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16)
    rng = np.random.default_rng(1)
    for m, launches in ((1024, 2), (600, 1)):      # 1024 rows: expansion + GEMM; 600: the in-pipeline kernel
        x = bf16_round(rng.standard_normal((m, k)).astype(np.float32))
        before = _lib.LAUNCH_COUNT[0]
        got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), packed, cb, None, n, k, bits=3, group_rows=128)
        assert _lib.LAUNCH_COUNT[0] - before == launches, m
        want = o.linear_wq(x, cw["packed"], cw["codebooks"], 3, n, k, None, 128)
        max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
        assert max_abs <= MAX_ABS and rel <= REL_L2, (m, max_abs, rel)
    assert ops.last_device_status() == 0


def test_linear_expand_rejects_what_it_cannot_take(ops):
    cw = make_weight(40, 96, 4, seed=2, cb_dtype="bf16")
    x = torch.randn(64, 96, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):        # K is not a multiple of 64
        ops.dimq_linear_wq(x, _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16), None, 40, 96, bits=4,
                           algo="expand")
    cw = make_weight(42, 128, 4, seed=2, cb_dtype="bf16")
    x = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):        # bf16 rows of 42 features are not 16-byte multiples
        ops.dimq_linear_wq(x, _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16), None, 42, 128, bits=4,
                           algo="expand", out_dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):        # fp32 activations
        ops.dimq_linear_wq(x.float(), _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16), None, 42, 128,
                           bits=4, algo="expand")


def test_expand_workspace_is_checked_by_the_c_abi(ops):
    from dimq_b200 import _lib

    n, k, m = 64, 128, 256
    cw = make_weight(n, k, 4, seed=4, cb_dtype="bf16")
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    packed, cb = _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16)
    y = torch.empty(m, n, device="cuda", dtype=torch.float32)
    w = _lib.WqWeight(packed.data_ptr(), 4, cb.data_ptr(), _lib.BF16, 16, 1, n, 0)
    need = C.c_int64(0)
    lib = _lib.lib()
    assert lib.dimq_expand_workspace_bytes(_lib.BF16, C.byref(w), C.c_int64(n), C.c_int64(k), C.byref(need)) == 0
    assert need.value == n * k * 2
    w16 = _lib.WqWeight(packed.data_ptr(), 4, cb.data_ptr(), _lib.F16, 16, 1, n, 0)    # hi + lo pairs
    lib.dimq_expand_workspace_bytes(_lib.BF16, C.byref(w16), C.c_int64(n), C.c_int64(k), C.byref(need))
    assert need.value == 2 * n * k * 2
    ws = torch.empty(n * k * 2 - 16, dtype=torch.uint8, device="cuda")
    args = (_lib.ptr(x), _lib.BF16, C.byref(w), None, 0, None, _lib.ptr(y), _lib.F32, C.c_int64(m), C.c_int64(n),
            C.c_int64(k), 0)
    st = lib.dimq_linear_wq_expand(*args, _lib.ptr(ws), C.c_int64(ws.numel()), _lib.stream_ptr(x.device))
    assert st == -12 and b"scratch" in lib.dimq_status_string(st)      # DIMQ_ERR_SCRATCH_TOO_SMALL, nothing launched
    st = lib.dimq_linear_wq_expand(*args, None, C.c_int64(1 << 20), _lib.stream_ptr(x.device))
    assert st == -12
    torch.cuda.synchronize()


# ---- implicit-GEMM convolution ----------------------------------------------------------------------

CONV_CASES = [
    # batch, C, H, W, OC, k, stride, pad, dilation
    (4, 64, 56, 56, 64, 3, 1, 1, 1),     # config 2 geometry at a small batch
    (3, 64, 56, 56, 128, 3, 2, 1, 1),    # stride-2 3x3
    (3, 64, 56, 56, 128, 1, 2, 0, 1),    # 1x1 stride-2 downsample
    (2, 128, 28, 28, 128, 3, 1, 1, 1),
    (5, 128, 14, 14, 192, 3, 1, 1, 1),
    (6, 128, 7, 7, 136, 3, 1, 1, 1),     # OC not a multiple of the weight tile
    (2, 64, 13, 9, 64, 3, 2, 1, 1),      # odd sizes with stride 2
    (2, 64, 12, 10, 64, 3, 1, 2, 2),     # dilation 2
    (1, 64, 3, 5, 8, 3, 1, 1, 1),        # fewer output pixels than one tile
]


def _conv_oracle(x, cw, bits, wshape, bias, s, pad, dil):
    """dequantise (oracle) + fp32 F.conv2d on the CPU: the reference's weight-only contract."""
    idx = o.unpack_bits(cw["packed"], int(np.prod(wshape)), bits).reshape(wshape[0], -1)
    w_hat = o.dequantize(idx, cw["codebooks"], cw["group_rows"]).reshape(wshape)
    b = None if bias is None else torch.from_numpy(bias)
    return F.conv2d(torch.from_numpy(x), torch.from_numpy(w_hat), b, s, pad, dil).numpy()


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("mode", ["per_channel_fp16cb", "per_layer_bf16cb"])
def test_conv_expand_fp32_out(ops, case, mode):
    b, c, h, w, oc, k, s, pad, dil = case
    rng = np.random.default_rng(sum(case))
    std = (2.0 / (c * k * k)) ** 0.5
    if mode == "per_channel_fp16cb":
        cw, grp, cb_t = make_weight(oc, c * k * k, 4, seed=7, group_rows=1, std=std), 1, torch.float16
    else:
        cw, grp, cb_t = make_weight(oc, c * k * k, 4, seed=8, std=std, cb_dtype="bf16"), None, torch.bfloat16
    x = bf16_round(np.maximum(rng.standard_normal((b, c, h, w)).astype(np.float32), 0))
    bias = rng.standard_normal(oc).astype(np.float32)
    wshape = (oc, c, k, k)
    want = _conv_oracle(x, cw, 4, wshape, bias, s, pad, dil)
    packed = _cuda(cw["packed"])
    khwc = ops.conv_prepack(packed, wshape, 4)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    got = ops.dimq_conv2d_wq(x_cl, packed, _cuda(cw["codebooks"], cb_t), _cuda(bias), wshape, (s, s), (pad, pad),
                             (dil, dil), 1, bits=4, group_rows=grp, packed_khwc=khwc, algo="expand")
    assert ops.last_device_status() == 0
    assert got.is_contiguous(memory_format=torch.channels_last) and got.dtype == torch.float32
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= MAX_ABS and rel <= REL_L2, (case, mode, max_abs, rel)


def test_conv_expand_residual_relu_bf16_out(ops):
    b, c, h, w, oc = 4, 64, 28, 28, 64
    rng = np.random.default_rng(3)
    cw = make_weight(oc, c * 9, 4, seed=5, std=(2.0 / (c * 9)) ** 0.5, cb_dtype="bf16")
    x = bf16_round(np.maximum(rng.standard_normal((b, c, h, w)).astype(np.float32), 0))
    res = bf16_round(rng.standard_normal((b, oc, h, w)).astype(np.float32))
    bias = rng.standard_normal(oc).astype(np.float32)
    lin = _conv_oracle(x, cw, 4, (oc, c, 3, 3), bias, 1, 1, 1)
    packed = _cuda(cw["packed"])
    khwc = ops.conv_prepack(packed, (oc, c, 3, 3), 4)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    r_cl = _cuda(res, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    for epi, want in (("add_relu", np.maximum(lin + res, 0)), ("relu", np.maximum(lin, 0) + res)):
        got = ops.dimq_conv2d_wq(x_cl, packed, _cuda(cw["codebooks"], torch.bfloat16), _cuda(bias), (oc, c, 3, 3),
                                 (1, 1), (1, 1), (1, 1), 1, bits=4, out_dtype=torch.bfloat16, epilogue=epi,
                                 residual=r_cl, packed_khwc=khwc, algo="expand")
        assert got.dtype == torch.bfloat16
        max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
        assert max_abs <= MAX_ABS_16 and rel <= REL_L2_16, (epi, max_abs, rel)
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("h,w", [(1, 1), (1, 6), (5, 1)])
def test_conv_stride2_on_one_pixel_wide_maps_falls_back(ops, h, w):
    """A 3x3 stride-2 pad-1 convolution over a map with a single row or column: the tensor-core paths
    address stride 2 through parity planes, one of which is empty here, so the automatic choice must
    take the direct kernel — and the pixel right of / below the map must count as zero."""
    b, c, oc = 2, 64, 64
    rng = np.random.default_rng(h * 10 + w)
    cw = make_weight(oc, c * 9, 4, seed=13, std=0.05, cb_dtype="bf16")
    x = bf16_round(rng.standard_normal((b, c, h, w)).astype(np.float32))
    want = _conv_oracle(x, cw, 4, (oc, c, 3, 3), None, 2, 1, 1)
    packed = _cuda(cw["packed"])
    khwc = ops.conv_prepack(packed, (oc, c, 3, 3), 4)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    cb = _cuda(cw["codebooks"], torch.bfloat16)
    got = ops.dimq_conv2d_wq(x_cl, packed, cb, None, (oc, c, 3, 3), (2, 2), (1, 1), (1, 1), 1, bits=4, packed_khwc=khwc)
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= MAX_ABS and rel <= REL_L2, (max_abs, rel)
    for algo in ("tcgen05", "expand"):
        with pytest.raises(RuntimeError):
            ops.dimq_conv2d_wq(x_cl, packed, cb, None, (oc, c, 3, 3), (2, 2), (1, 1), (1, 1), 1, bits=4,
                               packed_khwc=khwc, algo=algo)
    assert ops.last_device_status() == 0


# ---- the configurations at their stated sizes --------------------------------------------------------

def test_config2_conv_at_batch_64(ops):
    """3x3, stride 1, pad 1, 64 -> 64 channels on 56 x 56, batch 64, per-output-channel 16-entry codebooks,
    bf16 NHWC activations = ReLU of N(0, 1): the tile plan of the full batch, automatic kernel choice."""
    b, c, hw, oc = 64, 64, 56, 64
    rng = np.random.default_rng(0)
    cw = make_weight(oc, c * 9, 4, seed=0, group_rows=1, std=(2.0 / (c * 9)) ** 0.5)
    x = bf16_round(np.maximum(rng.standard_normal((b, c, hw, hw)).astype(np.float32), 0))
    want = _conv_oracle(x, cw, 4, (oc, c, 3, 3), None, 1, 1, 1)
    packed = _cuda(cw["packed"])
    khwc = ops.conv_prepack(packed, (oc, c, 3, 3), 4)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    got = ops.dimq_conv2d_wq(x_cl, packed, _cuda(cw["codebooks"], torch.float16), None, (oc, c, 3, 3), (1, 1), (1, 1),
                             (1, 1), 1, bits=4, group_rows=1, packed_khwc=khwc)
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    print(f"config 2 at batch 64: max_abs={max_abs:.3e} rel_l2={rel:.3e}")
    assert max_abs <= MAX_ABS and rel <= REL_L2 and ops.last_device_status() == 0


@pytest.mark.parametrize("k,n", [(768, 2304), (768, 768), (768, 3072), (3072, 768)])
def test_vit_layer_shapes_at_batch_128(ops, k, n):
    """The four Linear shapes of ViT-B/16 at the full 128 x 197 = 25 216 token rows (3-bit, one bf16
    codebook per 128 rows), fp32 output, automatic kernel choice, against fp32 F.linear on the CPU."""
    m = 128 * 197
    cw = make_weight(n, k, 3, seed=k + n, group_rows=128, cb_dtype="bf16")
    gen = torch.Generator().manual_seed(n)
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    bias = torch.randn(n, generator=gen).to(torch.bfloat16)
    idx = o.unpack_bits(cw["packed"], n * k, 3).reshape(n, k)
    w_hat = torch.from_numpy(o.dequantize(idx, cw["codebooks"], 128))
    want = F.linear(x.float(), w_hat, bias.float())
    got = ops.dimq_linear_wq(x.cuda(), _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16), bias.cuda(), n, k,
                             bits=3, group_rows=128).cpu()
    diff = got - want
    max_abs, rel = float(diff.abs().max()), float(diff.norm() / want.norm())
    print(f"ViT layer {k}->{n} at M={m}: max_abs={max_abs:.3e} rel_l2={rel:.3e}")
    assert max_abs <= MAX_ABS and rel <= REL_L2 and ops.last_device_status() == 0


@pytest.mark.parametrize("mode", ["bf16_cb_fp32_out", "fp16_cb_two_terms_fp32_out", "bf16_cb_residual_gelu_bf16_out"])
def test_linear_shapes_of_the_cta_pair_tiling(ops, mode):
    """75 activation blocks (the last one ragged) x 5 weight tiles of 256 rows: the tile count at which the
    large-M path forms CTA pairs (256 x 256 tiles, cta_group::2); the last pair has a single block.  Codebooks in
    the activations' format and not (hi + lo terms), and the fused epilogue with a 16-bit output."""
    m, k, n = 9500, 512, 1280
    two = mode.startswith("fp16")
    cw = make_weight(n, k, 4, seed=21, group_rows=128, cb_dtype=np.float16 if two else "bf16")
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    bias = torch.randn(n, generator=gen).to(torch.bfloat16)
    idx = o.unpack_bits(cw["packed"], n * k, 4).reshape(n, k)
    w_hat = torch.from_numpy(o.dequantize(idx, cw["codebooks"], 128))
    lin = F.linear(x.float(), w_hat, bias.float())
    cb = _cuda(cw["codebooks"], torch.float16 if two else torch.bfloat16)
    if mode.endswith("bf16_out"):
        res = torch.randn(m, n, generator=gen).to(torch.bfloat16)
        want = F.gelu(lin) + res.float()
        got = ops.dimq_linear_wq(x.cuda(), _cuda(cw["packed"]), cb, bias.cuda(), n, k, bits=4, group_rows=128,
                                 out_dtype=torch.bfloat16, epilogue="gelu", residual=res.cuda()).float().cpu()
        tol_abs, tol_rel = MAX_ABS_16, REL_L2_16
    else:
        want = lin
        got = ops.dimq_linear_wq(x.cuda(), _cuda(cw["packed"]), cb, bias.cuda(), n, k, bits=4, group_rows=128).cpu()
        tol_abs, tol_rel = MAX_ABS, REL_L2
    diff = got - want
    max_abs, rel = float(diff.abs().max()), float(diff.norm() / want.norm())
    print(f"pair tiling {mode}: max_abs={max_abs:.3e} rel_l2={rel:.3e}")
    assert max_abs <= tol_abs and rel <= tol_rel and ops.last_device_status() == 0


RESNET_LAYERS = [
    # C, H, OC, k, stride (ResNet-18's distinct quantised 4-bit convolutions with >= 64 input channels)
    (64, 56, 64, 3, 1), (64, 56, 128, 3, 2), (64, 56, 128, 1, 2), (128, 28, 128, 3, 1), (128, 28, 256, 3, 2),
    (128, 28, 256, 1, 2), (256, 14, 256, 3, 1), (256, 14, 512, 3, 2), (256, 14, 512, 1, 2), (512, 7, 512, 3, 1),
]


@pytest.mark.parametrize("layer", RESNET_LAYERS)
def test_resnet_layer_geometries_at_batch_256(ops, layer):
    """Every distinct convolution geometry of ResNet-18 at the batch-256 tile plan (4-bit per-layer bf16
    codebook, fused bias + ReLU, fp32 output, automatic kernel choice)."""
    c, hw, oc, k, s = layer
    b, pad = 256, k // 2
    cw = make_weight(oc, c * k * k, 4, seed=c + oc + k, std=(2.0 / (c * k * k)) ** 0.5, cb_dtype="bf16")
    gen = torch.Generator().manual_seed(oc + s)
    x = torch.relu(torch.randn(b, c, hw, hw, generator=gen)).to(torch.bfloat16)
    bias = torch.randn(oc, generator=gen)
    idx = o.unpack_bits(cw["packed"], oc * c * k * k, 4).reshape(oc, -1)
    w_hat = torch.from_numpy(o.dequantize(idx, cw["codebooks"], None).reshape(oc, c, k, k))
    want = torch.relu(F.conv2d(x.float(), w_hat, bias, s, pad))
    packed = _cuda(cw["packed"])
    khwc = ops.conv_prepack(packed, (oc, c, k, k), 4)
    x_cl = x.cuda().contiguous(memory_format=torch.channels_last)
    got = ops.dimq_conv2d_wq(x_cl, packed, _cuda(cw["codebooks"], torch.bfloat16), bias.cuda(), (oc, c, k, k), (s, s),
                             (pad, pad), (1, 1), 1, bits=4, epilogue="relu", packed_khwc=khwc).cpu()
    diff = got - want
    max_abs, rel = float(diff.abs().max()), float(diff.norm() / want.norm())
    print(f"ResNet layer {layer} at batch {b}: max_abs={max_abs:.3e} rel_l2={rel:.3e}")
    assert max_abs <= MAX_ABS and rel <= REL_L2 and ops.last_device_status() == 0


# ---- stem convolution (3 input channels, stride 2) -----------------------------------------------------

STEM_CASES = [
    # batch, H, W, OC, k, pad, bits
    (2, 224, 224, 64, 7, 3, 8),      # the ResNet stem
    (3, 37, 40, 64, 7, 3, 8),        # odd height, 20 output columns: ragged tiles on every side
    (2, 64, 48, 32, 3, 1, 4),        # 3x3, 32 channels
    (1, 30, 56, 128, 5, 2, 4),       # 5x5, 128 channels
    (2, 9, 24, 16, 7, 0, 3),         # no padding, 16 channels, map smaller than a tile
]


@pytest.mark.parametrize("case", STEM_CASES)
@pytest.mark.parametrize("mode", ["bf16_cb", "fp16_cb_two_terms"])
def test_stem_conv_fp32_out(ops, case, mode):
    b, h, w, oc, k, pad, bits = case
    rng = np.random.default_rng(sum(case))
    cw = make_weight(oc, 3 * k * k, bits, seed=oc + k, std=(2.0 / (3 * k * k)) ** 0.5,
                     cb_dtype="bf16" if mode == "bf16_cb" else np.float16)
    cb_t = torch.bfloat16 if mode == "bf16_cb" else torch.float16
    x = bf16_round(rng.standard_normal((b, 3, h, w)).astype(np.float32))
    bias = rng.standard_normal(oc).astype(np.float32)
    wshape = (oc, 3, k, k)
    want = _conv_oracle(x, cw, bits, wshape, bias, 2, pad, 1)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    got = ops.dimq_conv2d_wq(x_cl, _cuda(cw["packed"]), _cuda(cw["codebooks"], cb_t), _cuda(bias), wshape, (2, 2),
                             (pad, pad), (1, 1), 1, bits=bits, algo="expand")
    assert ops.last_device_status() == 0
    assert got.is_contiguous(memory_format=torch.channels_last) and got.dtype == torch.float32
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= MAX_ABS and rel <= REL_L2, (case, mode, max_abs, rel)


def test_stem_conv_needs_16_byte_rows_else_the_direct_kernel_runs(ops):
    """The stem kernel fetches its input windows with TMA, which wants 16-byte aligned image rows
    (W * 6 bytes): other widths are refused when forced and take the direct kernel automatically."""
    b, h, w, oc = 5, 37, 45, 64
    rng = np.random.default_rng(8)
    cw = make_weight(oc, 147, 8, seed=3, std=(2.0 / 147) ** 0.5, cb_dtype="bf16")
    x = bf16_round(rng.standard_normal((b, 3, h, w)).astype(np.float32))
    want = _conv_oracle(x, cw, 8, (oc, 3, 7, 7), None, 2, 3, 1)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    args = (_cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16), None, (oc, 3, 7, 7), (2, 2), (3, 3), (1, 1), 1)
    with pytest.raises(RuntimeError):
        ops.dimq_conv2d_wq(x_cl, *args, bits=8, algo="expand")
    got = ops.dimq_conv2d_wq(x_cl, *args, bits=8)
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= MAX_ABS and rel <= REL_L2 and ops.last_device_status() == 0


def test_stem_conv_auto_relu_bf16_out_and_nonfinite_neighbours(ops):
    """Automatic choice at the ResNet stem's size with bias + ReLU and bf16 output; and an infinite pixel
    must poison only the outputs whose 7x7 window contains it (the patch rows carry one extra pixel per
    kernel row, which is cleared)."""
    from dimq_b200 import _lib

    b, h, w, oc = 4, 224, 224, 64
    rng = np.random.default_rng(5)
    cw = make_weight(oc, 147, 8, seed=1, std=(2.0 / 147) ** 0.5, cb_dtype="bf16")
    x = bf16_round(rng.standard_normal((b, 3, h, w)).astype(np.float32))
    bias = rng.standard_normal(oc).astype(np.float32)
    want = np.maximum(_conv_oracle(x, cw, 8, (oc, 3, 7, 7), bias, 2, 3, 1), 0)
    x_cl = _cuda(x, torch.bfloat16).contiguous(memory_format=torch.channels_last)
    args = (_cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16), _cuda(bias), (oc, 3, 7, 7), (2, 2), (3, 3), (1, 1), 1)
    before = _lib.LAUNCH_COUNT[0]
    got = ops.dimq_conv2d_wq(x_cl, *args, bits=8, out_dtype=torch.bfloat16, epilogue="relu")
    assert _lib.LAUNCH_COUNT[0] - before == 2          # weight expansion + stem kernel
    max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
    assert max_abs <= MAX_ABS_16 and rel <= REL_L2_16, (max_abs, rel)
    x_inf = x_cl.clone()
    x_inf[1, 0, 100, 101] = float("inf")                # input pixel (100, 101) of image 1
    got_inf = ops.dimq_conv2d_wq(x_inf, *args, bits=8).cpu()
    bad = ~torch.isfinite(got_inf)
    rows = [oh for oh in range(112) if 0 <= 100 - (2 * oh - 3) < 7]
    cols = [ow for ow in range(112) if 0 <= 101 - (2 * ow - 3) < 7]
    expect = torch.zeros_like(bad)
    expect[1, :, rows[0]:rows[-1] + 1, cols[0]:cols[-1] + 1] = True
    assert not (bad & ~expect).any()                    # nothing outside the windows that contain the pixel
    assert ops.last_device_status() == 0
