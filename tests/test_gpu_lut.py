"""GPU parity of the LUT GEMM / conv kernels against the CPU oracle, through the C ABI.

Tolerances: the W4A4 (product-table) ops are checked at the reference's own
1e-5; the weight-only ops at max-abs 1e-2 and relative L2 1e-3 against the
dequantise-then-fp32-linear/conv oracle on the same (bf16/fp16-rounded) inputs.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import dimq_oracle as o
from tests._cases import bf16_round, make_weight

pytestmark = pytest.mark.gpu

MAX_ABS = 1e-2
REL_L2 = 1e-3


@pytest.fixture(scope="module")
def ops(cuda_device):
    from dimq_b200 import ops as _ops

    _ops.require_extension()
    return _ops


def _cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _assert_close(y: torch.Tensor, y_ref: np.ndarray, what: str = ""):
    assert tuple(y.shape) == tuple(y_ref.shape), (y.shape, y_ref.shape)
    max_abs, rel = o.parity_metrics(y.float().cpu().numpy(), y_ref)
    assert max_abs <= MAX_ABS and rel <= REL_L2, f"{what}: max_abs={max_abs:.3e} rel_l2={rel:.3e}"


# ---- W4A4 product-table ops (the reference's own CUDA tests) ---------------------

def test_linear_lut_reference_case(ops, golden):
    # dimq_cuda_backend/tests/test_cuda_ops.py:51-64
    y = ops.dimq_linear_lut(_cuda(golden["lin_x"]), _cuda(golden["lin_packed"]), _cuda(golden["lin_cb"]), 0.2, 7,
                            _cuda(golden["lin_bias"]), 6, 11)
    assert y.dtype == torch.float32
    np.testing.assert_allclose(y.cpu().numpy(), golden["lin_y_lut"], rtol=1e-5, atol=1e-5)
    y = ops.dimq_linear_lut(_cuda(golden["lin_x"]), _cuda(golden["lin_packed"]), _cuda(golden["lin_cb"]), 0.2, 7,
                            None, 6, 11)
    np.testing.assert_allclose(y.cpu().numpy(), golden["lin_y_nobias"], rtol=1e-5, atol=1e-5)
    y = ops.dimq_linear_lut(_cuda(golden["linb_x"]), _cuda(golden["linb_packed"]), _cuda(golden["linb_cb"]), 0.3, 8,
                            None, 24, 64)
    assert y.shape == (2, 5, 24)
    np.testing.assert_allclose(y.cpu().numpy(), golden["linb_y_lut"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (5, 33, 17), (70, 129, 45), (256, 768, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_linear_lut_matches_c_oracle(ops, m, k, n, dtype):
    rng = np.random.default_rng(m * 31 + k)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
    widx = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    packed = o.pack_u4(widx)
    cb = np.sort(rng.standard_normal(16).astype(np.float32) * 0.1)
    bias = rng.standard_normal(n).astype(np.float32)
    want = c_oracle.linear_lut_a4(x.float().numpy(), packed, cb, 0.25, 6, n, k, bias)
    got = ops.dimq_linear_lut(x.cuda(), _cuda(packed), _cuda(cb), 0.25, 6, _cuda(bias, torch.float16), n, k)
    want_h = c_oracle.linear_lut_a4(x.float().numpy(), packed, cb, 0.25, 6, n, k, bias.astype(np.float16).astype(np.float32))
    np.testing.assert_allclose(got.cpu().numpy(), want_h, rtol=1e-5, atol=2e-5)
    del want


def test_linear_lut_argument_checks(ops, golden):
    x, pw, cb = _cuda(golden["lin_x"]), _cuda(golden["lin_packed"]), _cuda(golden["lin_cb"])
    with pytest.raises(RuntimeError):
        ops.dimq_linear_lut(x, pw, cb, 0.0, 7, None, 6, 11)
    with pytest.raises(RuntimeError):
        ops.dimq_linear_lut(x, pw, cb, 0.2, 16, None, 6, 11)
    with pytest.raises(RuntimeError):
        ops.dimq_linear_lut(x, pw, cb[:8], 0.2, 7, None, 6, 11)
    with pytest.raises(RuntimeError):
        ops.dimq_linear_lut(x, pw, cb, 0.2, 7, None, 60, 11)  # packed too small
    with pytest.raises(RuntimeError):
        ops.dimq_linear_lut(x, pw, cb, 0.2, 7, None, 6, 12)   # last dim mismatch
    with pytest.raises(RuntimeError):
        ops.dimq_linear_lut(x, pw.to(torch.int32), cb, 0.2, 7, None, 6, 11)
    with pytest.raises(NotImplementedError):
        torch.ops.dimq.linear_lut(x.cpu(), pw.cpu(), cb.cpu(), 0.2, 7, None, 6, 11)


def test_conv2d_lut_reference_case(ops, golden):
    # dimq_cuda_backend/tests/test_cuda_ops.py:67-93
    y = ops.dimq_conv2d_lut(_cuda(golden["conv_x"]), _cuda(golden["conv_packed"]), _cuda(golden["conv_cb"]), 0.25, 7,
                            _cuda(golden["conv_bias"]), (5, 3, 3, 3), (2, 1), (1, 1), (1, 1), 1)
    assert y.dtype == torch.float32
    np.testing.assert_allclose(y.cpu().numpy(), golden["conv_y_deq"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(y.cpu().numpy(), golden["conv_y_lut"], rtol=1e-5, atol=1e-5)
    y = ops.dimq_conv2d_lut(_cuda(golden["convg_x"]), _cuda(golden["convg_packed"]), _cuda(golden["conv_cb"]), 0.25,
                            7, None, (6, 2, 3, 2), (1, 2), (2, 1), (2, 1), 2)
    np.testing.assert_allclose(y.cpu().numpy(), golden["convg_y_deq"], rtol=1e-5, atol=1e-5)
    # channels_last storage is read in place and the result comes back channels_last
    x_cl = _cuda(golden["conv_x"]).contiguous(memory_format=torch.channels_last)
    y_cl = ops.dimq_conv2d_lut(x_cl, _cuda(golden["conv_packed"]), _cuda(golden["conv_cb"]), 0.25, 7,
                               _cuda(golden["conv_bias"]), (5, 3, 3, 3), (2, 1), (1, 1), (1, 1), 1)
    assert y_cl.is_contiguous(memory_format=torch.channels_last)
    np.testing.assert_allclose(y_cl.cpu().numpy(), golden["conv_y_deq"], rtol=1e-5, atol=1e-5)
    with pytest.raises(RuntimeError):
        ops.dimq_conv2d_lut(_cuda(golden["conv_x"]), _cuda(golden["conv_packed"]), _cuda(golden["conv_cb"]), 0.25, 7,
                            None, (5, 4, 3, 3), (2, 1), (1, 1), (1, 1), 1)
    empty = ops.dimq_conv2d_lut(_cuda(golden["conv_x"])[:0], _cuda(golden["conv_packed"]), _cuda(golden["conv_cb"]),
                                0.25, 7, None, (5, 3, 3, 3), (2, 1), (1, 1), (1, 1), 1)
    assert empty.shape == (0, 5, 3, 7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv2d_lut_matches_c_oracle(ops, dtype):
    rng = np.random.default_rng(21)
    x = torch.from_numpy(rng.standard_normal((3, 8, 13, 11)).astype(np.float32)).to(dtype)
    widx = rng.integers(0, 16, size=(12, 4, 3, 5), dtype=np.uint8)
    packed = o.pack_u4(widx)
    cb = np.sort(rng.standard_normal(16).astype(np.float32) * 0.2)
    bias = rng.standard_normal(12).astype(np.float32)
    kw = dict(stride=(2, 1), padding=(1, 2), dilation=(1, 2), groups=2)
    want = c_oracle.conv2d_lut_a4(x.float().numpy(), packed, cb, 0.3, 5, widx.shape, bias, **kw)
    got = ops.dimq_conv2d_lut(x.cuda(), _cuda(packed), _cuda(cb), 0.3, 5, _cuda(bias), widx.shape, kw["stride"],
                              kw["padding"], kw["dilation"], kw["groups"])
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-5, atol=2e-5)


# ---- W4A4 on the tensor cores (large problems) -------------------------------------
# Same op, computed as sum (s*C[w]) * (a - z) with the scaled codewords rounded to a hi + lo bf16 pair:
# checked against the exact table-lookup oracle at the weight-only tolerance, and observed far inside it.

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k,n", [(1024, 768, 384), (777, 128, 130)])
def test_linear_lut_tensor_core_path(ops, m, k, n, dtype):
    from dimq_b200 import _lib

    assert m >= ops.A4_TC_MIN_ROWS
    rng = np.random.default_rng(m + k)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32) * 1.5).to(dtype)
    widx = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    packed = o.pack_u4(widx)
    cb = np.sort(rng.standard_normal(16).astype(np.float32) * 0.1)
    bias = rng.standard_normal(n).astype(np.float32)
    want = c_oracle.linear_lut_a4(x.float().numpy(), packed, cb, 0.25, 6, n, k, bias)
    before = _lib.LAUNCH_COUNT[0]
    got = ops.dimq_linear_lut(x.cuda(), _cuda(packed), _cuda(cb), 0.25, 6, _cuda(bias), n, k)
    assert _lib.LAUNCH_COUNT[0] - before == 2, "expected the quantiser + tensor-core GEMM pair"
    assert got.dtype == torch.float32
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= 1e-3 and rel <= 1e-4, (max_abs, rel)
    assert ops.last_device_status() == 0


@pytest.mark.parametrize("stride,pad,ksize", [(1, 1, 3), (2, 1, 3), (2, 0, 1)])
def test_conv2d_lut_tensor_core_path(ops, stride, pad, ksize):
    from dimq_b200 import _lib

    rng = np.random.default_rng(5 + stride + ksize)
    x = torch.from_numpy(rng.standard_normal((4, 64, 28, 28)).astype(np.float32)).to(torch.float16)
    widx = rng.integers(0, 16, size=(96, 64, ksize, ksize), dtype=np.uint8)
    packed = o.pack_u4(widx)
    cb = np.sort(rng.standard_normal(16).astype(np.float32) * 0.2)
    bias = rng.standard_normal(96).astype(np.float32)
    kw = dict(stride=(stride, stride), padding=(pad, pad), dilation=(1, 1), groups=1)
    want = c_oracle.conv2d_lut_a4(x.float().numpy(), packed, cb, 0.3, 5, widx.shape, bias, **kw)
    x_cl = x.cuda().contiguous(memory_format=torch.channels_last)
    before = _lib.LAUNCH_COUNT[0]
    got = ops.dimq_conv2d_lut(x_cl, _cuda(packed), _cuda(cb), 0.3, 5, _cuda(bias), widx.shape, kw["stride"],
                              kw["padding"], kw["dilation"], 1)
    assert _lib.LAUNCH_COUNT[0] - before == 3, "expected re-order + quantiser + tensor-core convolution"
    assert got.is_contiguous(memory_format=torch.channels_last)
    max_abs, rel = o.parity_metrics(got.cpu().numpy(), want)
    assert max_abs <= 1e-3 and rel <= 1e-4, (max_abs, rel)
    # NCHW-contiguous input keeps the exact direct kernel
    exact = ops.dimq_conv2d_lut(x.cuda(), _cuda(packed), _cuda(cb), 0.3, 5, _cuda(bias), widx.shape, kw["stride"],
                                kw["padding"], kw["dilation"], 1)
    np.testing.assert_allclose(exact.cpu().numpy(), want, rtol=1e-5, atol=1e-4)
    assert ops.last_device_status() == 0


def test_a4_tensor_core_workspace_checks(ops):
    import ctypes as C

    from dimq_b200 import _lib

    need = C.c_int64(0)
    assert _lib.lib().dimq_a4_workspace_bytes(C.c_int64(1024 * 64), C.c_int64(0), C.byref(need)) == 0
    assert need.value == 256 + 1024 * 64 * 2
    x = torch.zeros(1024, 64, device="cuda")
    pw = torch.zeros(64 * 64 // 2, dtype=torch.uint8, device="cuda")
    cb = torch.linspace(-1, 1, 16, device="cuda")
    y = torch.empty(1024, 64, device="cuda")
    ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    args = lambda nbytes, k=64: (_lib.ptr(x), 0, _lib.ptr(pw), _lib.ptr(cb), 0, C.c_float(0.1), 8, None, 0, _lib.ptr(y),
                                 C.c_int64(1024), C.c_int64(64), C.c_int64(k), _lib.ptr(ws), C.c_int64(nbytes), None)
    assert _lib.lib().dimq_linear_lut_tc(*args(need.value - 1)) == -12
    assert _lib.lib().dimq_linear_lut_tc(*args(need.value, 32)) == -7  # K not a multiple of 64: nothing launched
    assert _lib.lib().dimq_linear_lut_tc(*args(need.value)) == 0
    torch.cuda.synchronize()
    # zero activations quantise to code 8 = the zero point: every product is zero
    assert float(y.abs().max()) == 0.0


# ---- weight-only GEMM --------------------------------------------------------------

def test_linear_wq_golden(ops, golden):
    for algo in ("generic", None):
        y = ops.dimq_linear_wq(_cuda(golden["wq_lin_x"]), _cuda(golden["wq_lin_packed"]), _cuda(golden["wq_lin_cb"]),
                               _cuda(golden["wq_lin_bias"]), 48, 96, bits=4, algo=algo)
        np.testing.assert_allclose(y.cpu().numpy(), golden["wq_lin_y"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("m,k,n,grp", [(3, 37, 29, None), (40, 100, 70, 16), (1, 64, 8, 1)])
def test_linear_wq_generic_odd_shapes(ops, bits, m, k, n, grp):
    case = make_weight(n, k, bits, seed=bits * 100 + m, group_rows=grp, cb_dtype=np.float32)
    rng = np.random.default_rng(m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    want = o.linear_wq(x, case["packed"], case["codebooks"], bits, n, k, bias, case["group_rows"])
    got = ops.dimq_linear_wq(_cuda(x), _cuda(case["packed"]), _cuda(case["codebooks"]), _cuda(bias), n, k, bits=bits,
                             group_rows=case["group_rows"], algo="generic")
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-5, atol=1e-5)


def test_linear_wq_config1_fp32(ops):
    """Single DIMQ Linear 768 -> 3072, fp32 activations [8*197, 768], 4-bit per-layer quantile codebook."""
    case = make_weight(3072, 768, 4, seed=0, cb_dtype=np.float32)
    x = np.random.default_rng(0).standard_normal((8 * 197, 768)).astype(np.float32)
    want = o.linear_wq(x, case["packed"], case["codebooks"], 4, 3072, 768)
    got = ops.dimq_linear_wq(_cuda(x).view(8, 197, 768), _cuda(case["packed"]), _cuda(case["codebooks"]), None, 3072,
                             768, bits=4)
    assert got.shape == (8, 197, 3072)
    _assert_close(got.view(-1, 3072), want, "config 1")


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8])
def test_linear_wq_stream_small_m(ops, bits, m):
    n, k = 520, 1024
    case = make_weight(n, k, bits, seed=bits + 10 * m, group_rows=128)
    x = bf16_round(np.random.default_rng(m).standard_normal((m, k)).astype(np.float32))
    bias = np.random.default_rng(m + 1).standard_normal(n).astype(np.float32)
    want = o.linear_wq(x, case["packed"], case["codebooks"], bits, n, k, bias, 128)
    got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), _cuda(case["packed"]), _cuda(case["codebooks"], torch.float16),
                             _cuda(bias), n, k, bits=bits, group_rows=128, algo="stream")
    _assert_close(got, want, f"stream bits={bits} m={m}")
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=2e-4, atol=2e-4)
    # K = 768: a row is 24 units, fewer than one per lane
    case = make_weight(n, 768, bits, seed=bits, group_rows=None)
    x = bf16_round(np.random.default_rng(m).standard_normal((m, 768)).astype(np.float32))
    want = o.linear_wq(x, case["packed"], case["codebooks"], bits, n, 768)
    got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), _cuda(case["packed"]), _cuda(case["codebooks"]), None, n, 768,
                             bits=bits, algo="stream")
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=2e-4, atol=2e-4)


# ---- small-M index-streaming kernel for 16-bit activations (pair tables + warp MMA) ---------

# (activation dtype, codebook rounding, codebook dtype); the last one is the reference export's default
# (fp16 codebook) under bf16 activations: the kernel converts the activations to fp16 while staging them
MS_MODES = [(torch.bfloat16, "bf16", torch.bfloat16), (torch.float16, np.float16, torch.float16),
            (torch.float16, np.float32, torch.float32), (torch.bfloat16, np.float16, torch.float16)]


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("m,k,n,grp", [(1, 128, 16, None), (3, 768, 100, None), (8, 1024, 520, 128), (9, 1024, 4096, None),
                                       (16, 4096, 1024, None), (17, 256, 33, 16), (32, 2048, 300, 32),
                                       (5, 8192, 64, None), (2, 384, 2304, 128)])
def test_linear_wq_mma_stream(ops, bits, m, k, n, grp, mode):
    x_dtype, cb_np, cb_torch = MS_MODES[mode]
    case = make_weight(n, k, bits, seed=bits * 7 + m, group_rows=grp, cb_dtype=cb_np)
    rng = np.random.default_rng(m + k + n)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(x_dtype)
    bias = rng.standard_normal(n).astype(np.float32)
    # fp16 operands: the codewords the kernel multiplies are the fp16 roundings of the codebook
    cbs = case["codebooks"].astype(np.float16).astype(np.float32) if x_dtype == torch.float16 else case["codebooks"]
    want = o.linear_wq(x.float().numpy(), case["packed"], cbs, bits, n, k, bias, case["group_rows"])
    args = (x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], cb_torch), _cuda(bias), n, k)
    # the two widest cases may not fit beside the lookup table (activation rows, per-warp partial sums
    # and index rings share 227 KB): the kernel then refuses and the automatic choice takes another one
    may_refuse = (m, k) in ((16, 4096), (32, 2048))
    try:
        got = ops.dimq_linear_wq(*args, bits=bits, group_rows=grp, algo="mma_stream")
    except RuntimeError as err:
        assert may_refuse and "does not support" in str(err), err
        got = ops.dimq_linear_wq(*args, bits=bits, group_rows=grp)
        _assert_close(got, want, "auto dispatch after refusal")
        return
    assert ops.last_device_status() == 0
    _assert_close(got, want, f"mma_stream bits={bits} {m}x{k}x{n} mode={mode}")
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
def test_linear_wq_mma_stream_epilogues(ops, y_dtype):
    m, k, n = 12, 512, 200
    case = make_weight(n, k, 4, seed=3, cb_dtype="bf16")
    rng = np.random.default_rng(8)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
    bias = rng.standard_normal(n).astype(np.float32)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(y_dtype)
    lin = o.linear_wq(x.float().numpy(), case["packed"], case["codebooks"], 4, n, k, bias)
    for epi, fn in (("relu", lambda v: np.maximum(v, 0)), ("gelu", None), (None, lambda v: v)):
        want = torch.nn.functional.gelu(torch.from_numpy(lin)).numpy() if fn is None else fn(lin)
        want = want + res.float().numpy()
        got = ops.dimq_linear_wq(x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], torch.bfloat16), _cuda(bias),
                                 n, k, bits=4, out_dtype=y_dtype, epilogue=epi, residual=res.cuda(), algo="mma_stream")
        assert got.dtype == y_dtype
        max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
        assert max_abs <= (3e-2 if y_dtype == torch.bfloat16 else 1e-3) and rel <= (5e-3 if y_dtype == torch.bfloat16 else 1e-4), (epi, max_abs, rel)
    want = np.maximum(lin + res.float().numpy(), 0)
    got = ops.dimq_linear_wq(x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], torch.bfloat16), _cuda(bias), n, k,
                             bits=4, out_dtype=y_dtype, epilogue="add_relu", residual=res.cuda(), algo="mma_stream")
    max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
    assert rel <= (5e-3 if y_dtype == torch.bfloat16 else 1e-4), (max_abs, rel)


def test_linear_wq_mma_stream_rejects_what_it_cannot_take(ops):
    case = make_weight(64, 256, 4, seed=1)
    x = torch.zeros(4, 256, device="cuda")
    pw, cb = _cuda(case["packed"]), _cuda(case["codebooks"])
    with pytest.raises(RuntimeError):  # fp32 activations
        ops.dimq_linear_wq(x, pw, cb, None, 64, 256, bits=4, algo="mma_stream")
    with pytest.raises(RuntimeError):  # more than 32 rows
        ops.dimq_linear_wq(torch.zeros(33, 256, device="cuda", dtype=torch.float16), pw, cb, None, 64, 256, bits=4,
                           algo="mma_stream")


def test_linear_wq_mma_stream_converts_bf16_activations_of_any_magnitude(ops):
    """bf16 activations with an fp16 codebook run as fp16 MMAs.  Rows whose largest magnitude lies
    outside the exactly convertible range are scaled by a power of two on the way in and back on the
    way out, so huge, tiny, zero and mixed rows all keep the weight-only tolerance (relative here: the
    rows span 40 orders of magnitude)."""
    m, k, n = 7, 512, 96
    case = make_weight(n, k, 4, seed=5)                      # fp16-rounded codebook
    rng = np.random.default_rng(2)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[1] *= 1.0e6            # beyond fp16's 65504
    x[2] *= 1.0e-9           # below fp16's subnormals
    x[3] = 0.0               # all zero
    x[4, :5] *= 3.0e37       # a few huge values among ordinary ones
    x[5] *= 1.0e-20
    x[6] *= 3.0e30
    x = bf16_round(x)
    want = o.linear_wq(x, case["packed"], case["codebooks"], 4, n, k).astype(np.float64)
    got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), _cuda(case["packed"]), _cuda(case["codebooks"], torch.float16),
                             None, n, k, bits=4, algo="mma_stream").cpu().numpy().astype(np.float64)
    assert ops.last_device_status() == 0 and np.isfinite(got).all()
    for row in range(m):
        scale = np.linalg.norm(want[row])
        err = np.linalg.norm(got[row] - want[row])
        assert err <= 1e-3 * scale + (0.0 if scale > 0 else 1e-30), (row, err, scale)


# ---- small-M kernel for large weights: activations and indices in registers, k split over a cluster ----

# (m, k, n, group rows): 1 / 2 / 3 / 4 / 5 CTAs per cluster, several passes (k / 2048 = 11 is prime; 16384 = 2 x 4
# slices), codebook groups, fewer row blocks than clusters
MR_SHAPES = [(1, 2048, 64, None), (8, 4096, 256, 128), (9, 8192, 304, None), (3, 6144, 160, 16), (5, 10240, 48, None),
             (16, 22528, 32, None), (2, 16384, 96, 32),
             # K that does not fill its last 2048-k slice: 17, 24 and 86 ranges of 128
             (3, 2176, 64, None), (7, 3072, 320, 16), (16, 11008, 48, None)]
# enough row blocks that every cluster walks more of them than it keeps in flight (and crosses codebook groups)
MR_LONG_SHAPES = [(16, 2048, 9616, 32), (4, 8192, 2400, 128), (7, 14336, 1360, 16), (2, 16384, 2384, None)]


@pytest.mark.parametrize("mode", [0, 3])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("m,k,n,grp", MR_LONG_SHAPES)
def test_linear_wq_mma_regs_many_row_blocks(ops, bits, m, k, n, grp, mode):
    """~20 M weights per case: random index bytes against the exact fp32 kernel of this library (itself checked
    against the oracle above), and one case against the oracle."""
    x_dtype, _, cb_torch = MS_MODES[mode]
    gen = torch.Generator(device="cuda").manual_seed(bits * 100 + m)
    packed = torch.randint(0, 256, (n, k * bits // 8), dtype=torch.uint8, device="cuda", generator=gen)
    groups = 1 if grp is None else -(-n // grp)
    cb = (torch.randn(groups, 1 << bits, device="cuda", generator=gen) * 0.02).to(cb_torch)
    x = torch.randn(m, k, device="cuda", generator=gen).to(x_dtype)
    bias = torch.randn(n, device="cuda", generator=gen)
    got = ops.dimq_linear_wq(x, packed, cb, bias, n, k, bits=bits, group_rows=grp, algo="mma_regs")
    assert ops.last_device_status() == 0
    cb_used = cb.to(x_dtype) if x_dtype == torch.float16 else cb      # fp16 MMAs round the codewords to fp16
    want = ops.dimq_linear_wq(x, packed, cb_used, bias, n, k, bits=bits, group_rows=grp, algo="generic")
    _assert_close(got, want.cpu().numpy(), f"mma_regs long bits={bits} {m}x{k}x{n} mode={mode}")
    np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=2e-4, atol=2e-4 * np.sqrt(k / 1024))
    if (bits, mode, k) == (4, 3, 8192):
        ref = o.linear_wq(x.float().cpu().numpy(), packed.cpu().numpy(), cb.float().cpu().numpy(), bits, n, k,
                          bias.cpu().numpy(), grp)
        _assert_close(got, ref, "mma_regs long against the oracle")


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("m,k,n,grp", MR_SHAPES)
def test_linear_wq_mma_regs(ops, bits, m, k, n, grp, mode):
    x_dtype, cb_np, cb_torch = MS_MODES[mode]
    case = make_weight(n, k, bits, seed=bits * 5 + m, group_rows=grp, cb_dtype=cb_np)
    rng = np.random.default_rng(m + k + n)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(x_dtype)
    bias = rng.standard_normal(n).astype(np.float32)
    cbs = case["codebooks"].astype(np.float16).astype(np.float32) if x_dtype == torch.float16 else case["codebooks"]
    want = o.linear_wq(x.float().numpy(), case["packed"], cbs, bits, n, k, bias, case["group_rows"])
    got = ops.dimq_linear_wq(x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], cb_torch), _cuda(bias), n, k,
                             bits=bits, group_rows=grp, algo="mma_regs")
    assert ops.last_device_status() == 0
    _assert_close(got, want, f"mma_regs bits={bits} {m}x{k}x{n} mode={mode}")
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=2e-4, atol=2e-4 * np.sqrt(k / 1024))


@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
def test_linear_wq_mma_regs_epilogues(ops, y_dtype):
    m, k, n = 12, 4096, 208
    case = make_weight(n, k, 4, seed=3, cb_dtype="bf16")
    rng = np.random.default_rng(8)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
    bias = rng.standard_normal(n).astype(np.float32)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(y_dtype)
    lin = o.linear_wq(x.float().numpy(), case["packed"], case["codebooks"], 4, n, k, bias)
    args = (x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], torch.bfloat16), _cuda(bias), n, k)
    for epi, fn in (("relu", lambda v: np.maximum(v, 0)), ("gelu", None), (None, lambda v: v),
                    ("add_relu", lambda v: np.maximum(v + res.float().numpy(), 0))):
        want = torch.nn.functional.gelu(torch.from_numpy(lin)).numpy() if fn is None else fn(lin)
        if epi != "add_relu":
            want = want + res.float().numpy()
        got = ops.dimq_linear_wq(*args, bits=4, out_dtype=y_dtype, epilogue=epi, residual=res.cuda(), algo="mma_regs")
        assert got.dtype == y_dtype
        max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
        assert rel <= (5e-3 if y_dtype == torch.bfloat16 else 1e-4), (epi, max_abs, rel)


def test_linear_wq_mma_regs_rejects_and_auto_dispatch(ops):
    case = make_weight(64, 2048, 4, seed=1)
    pw, cb = _cuda(case["packed"]), _cuda(case["codebooks"])
    with pytest.raises(RuntimeError):  # fp32 activations
        ops.dimq_linear_wq(torch.zeros(4, 2048, device="cuda"), pw, cb, None, 64, 2048, bits=4, algo="mma_regs")
    with pytest.raises(RuntimeError):  # more than 16 rows
        ops.dimq_linear_wq(torch.zeros(17, 2048, device="cuda", dtype=torch.float16), pw, cb, None, 64, 2048, bits=4,
                           algo="mma_regs")
    case = make_weight(64, 1024, 4, seed=1)
    with pytest.raises(RuntimeError):  # k below 2048
        ops.dimq_linear_wq(torch.zeros(4, 1024, device="cuda", dtype=torch.float16), _cuda(case["packed"]),
                           _cuda(case["codebooks"]), None, 64, 1024, bits=4, algo="mma_regs")
    # 2 MB of indices and more: the automatic choice is this kernel (same bits as the forced call)
    n, k = 4096, 4096
    case = make_weight(n, k, 4, seed=9)
    x = torch.from_numpy(np.random.default_rng(3).standard_normal((6, k)).astype(np.float32)).to(torch.bfloat16).cuda()
    args = (x, _cuda(case["packed"]), _cuda(case["codebooks"], torch.float16), None, n, k)
    assert torch.equal(ops.dimq_linear_wq(*args, bits=4), ops.dimq_linear_wq(*args, bits=4, algo="mma_regs"))
    assert not torch.equal(ops.dimq_linear_wq(*args, bits=4), ops.dimq_linear_wq(*args, bits=4, algo="mma_stream"))


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_linear_prepack_and_tiled_small_m_kernel(ops, bits):
    """dimq_linear_prepack is the byte permutation it says it is, and the small-M kernel gives the same bits
    from the tiled indices as from the canonical ones (same arithmetic, another load pattern)."""
    n, k = 1040, 4224     # 65 row blocks; 33 ranges of 128 k: three slices, the last with one live warp
    gen = torch.Generator(device="cuda").manual_seed(bits)
    packed = torch.randint(0, 256, (n, k * bits // 8), dtype=torch.uint8, device="cuda", generator=gen)
    tiled = ops.linear_prepack(packed, n, k, bits)
    piece = 16 * bits     # bytes of one row of a 128-k range
    want = packed.view(n // 16, 16, k // 128, piece).permute(0, 2, 1, 3).contiguous().view(-1)
    assert torch.equal(tiled, want)
    assert np.array_equal(tiled.cpu().numpy(), o.linear_prepack(packed.cpu().numpy(), n, k, bits))
    cb = (torch.randn(n // 16, 1 << bits, device="cuda", generator=gen) * 0.02).to(torch.float16)
    bias = torch.randn(n, device="cuda", generator=gen)
    for m, x_dtype in ((1, torch.bfloat16), (5, torch.float16), (16, torch.bfloat16)):
        x = torch.randn(m, k, device="cuda", generator=gen).to(x_dtype)
        args = (x, packed, cb, bias, n, k)
        plain = ops.dimq_linear_wq(*args, bits=bits, group_rows=16, algo="mma_regs")
        fast = ops.dimq_linear_wq(*args, bits=bits, group_rows=16, algo="mma_regs", packed_tiled=tiled)
        assert ops.last_device_status() == 0
        assert torch.equal(plain, fast), (bits, m)
        auto = ops.dimq_linear_wq(*args, bits=bits, group_rows=16, packed_tiled=tiled)   # 2 MB of indices and more at 4 bits
        exact = ops.dimq_linear_wq(*args, bits=bits, group_rows=16, algo="generic")
        _assert_close(auto, exact.cpu().numpy(), f"tiled auto bits={bits} m={m}")
    with pytest.raises(RuntimeError):
        ops.linear_prepack(packed, n + 8, k, bits)      # N not a multiple of 16 (and a short buffer)
    # the module builds the tiled copy by itself the first time a small batch meets a large enough weight
    from dimq_b200.modules import DIMQLinear
    layer = DIMQLinear(packed, cb, None, None, n, k, bias, bits=bits, group_rows=16)
    x = torch.randn(3, k, device="cuda", generator=gen).to(torch.bfloat16)
    y = layer(x)
    assert (layer._tiled is not None) == (n * k * bits >= 1 << 24)
    assert torch.equal(y, ops.dimq_linear_wq(x, packed, cb, bias, n, k, bits=bits, group_rows=16))
    layer(torch.randn(64, k, device="cuda", generator=gen).to(torch.bfloat16))    # many rows: other kernels, same module


def test_linear_wq_mma_regs_converts_bf16_activations_of_any_magnitude(ops):
    """bf16 activations with an fp16 codebook run as fp16 MMAs; a (row, 128-k range) whose largest magnitude
    lies outside the exactly convertible range is scaled by a power of two on the way in and its partial sums
    back on the way out: huge, tiny, zero and mixed rows keep the weight-only tolerance."""
    m, k, n = 7, 4096, 96
    case = make_weight(n, k, 4, seed=5)                      # fp16-rounded codebook
    rng = np.random.default_rng(2)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[1] *= 1.0e6            # beyond fp16's 65504
    x[2] *= 1.0e-9           # below fp16's subnormals
    x[3] = 0.0               # all zero
    x[4, :5] *= 3.0e37       # a few huge values among ordinary ones
    x[5] *= 1.0e-20
    x[6] *= 3.0e30
    x = bf16_round(x)
    want = o.linear_wq(x, case["packed"], case["codebooks"], 4, n, k).astype(np.float64)
    got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), _cuda(case["packed"]), _cuda(case["codebooks"], torch.float16),
                             None, n, k, bits=4, algo="mma_regs").cpu().numpy().astype(np.float64)
    assert ops.last_device_status() == 0 and np.isfinite(got).all()
    for row in range(m):
        scale = np.linalg.norm(want[row])
        err = np.linalg.norm(got[row] - want[row])
        assert err <= 1e-3 * scale + (0.0 if scale > 0 else 1e-30), (row, err, scale)


TC_SHAPES = [(192, 64, 128), (200, 128, 130), (577, 768, 384), (64, 1024, 256), (16, 256, 128)]


# operand precision modes of the tensor-core kernel: (activation dtype, codebook dtype)
#   bf16 x, fp16 codebook -> bf16 operands, every codeword split into hi + lo (two MMAs per k-step)
#   bf16 x, bf16 codebook -> bf16 operands, exact in one term
#   fp16 x, fp16 codebook -> fp16 operands, exact in one term
TC_MODES = [(torch.bfloat16, np.float16, torch.float16), (torch.bfloat16, "bf16", torch.bfloat16),
            (torch.float16, np.float16, torch.float16)]


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("m,k,n", TC_SHAPES)
def test_linear_wq_tcgen05(ops, bits, m, k, n, mode):
    x_dtype, cb_np, cb_torch = TC_MODES[mode]
    grp = None if bits == 8 else 128
    case = make_weight(n, k, bits, seed=bits * 13 + m, group_rows=grp, cb_dtype=cb_np)
    rng = np.random.default_rng(m + k)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(x_dtype)
    bias = rng.standard_normal(n).astype(np.float32)
    want = o.linear_wq(x.float().numpy(), case["packed"], case["codebooks"], bits, n, k, bias, case["group_rows"])
    got = ops.dimq_linear_wq(x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], cb_torch),
                             _cuda(bias), n, k, bits=bits, group_rows=grp, algo="tcgen05")
    assert ops.last_device_status() == 0
    _assert_close(got, want, f"tcgen05 bits={bits} {m}x{k}x{n} mode={mode}")


def test_linear_wq_tcgen05_per_channel_codebooks(ops):
    """One codebook per output row: the lookup tables hold single codewords instead of pairs."""
    m, k, n = 250, 576, 64
    case = make_weight(n, k, 4, seed=9, group_rows=1, std=(2.0 / 576) ** 0.5)
    x = torch.relu(torch.from_numpy(np.random.default_rng(2).standard_normal((m, k)).astype(np.float32))).to(torch.bfloat16)
    want = o.linear_wq(x.float().numpy(), case["packed"], case["codebooks"], 4, n, k, None, 1)
    for cb_torch in (torch.float16, torch.float32):
        got = ops.dimq_linear_wq(x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], cb_torch), None, n, k,
                                 bits=4, group_rows=1, algo="tcgen05")
        assert ops.last_device_status() == 0
        _assert_close(got, want, "per-channel")


@pytest.mark.parametrize("x_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
def test_linear_wq_tcgen05_dtypes_epilogues(ops, x_dtype, y_dtype):
    m, k, n = 300, 256, 200
    case = make_weight(n, k, 4, seed=3)
    rng = np.random.default_rng(8)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(x_dtype)
    bias = rng.standard_normal(n).astype(np.float32)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(y_dtype)
    lin = o.linear_wq(x.float().numpy(), case["packed"], case["codebooks"], 4, n, k, bias)
    for epi, fn in (("relu", lambda v: np.maximum(v, 0)), ("gelu", None), (None, lambda v: v)):
        if fn is None:
            want = torch.nn.functional.gelu(torch.from_numpy(lin)).numpy()
        else:
            want = fn(lin)
        want = want + res.float().numpy()
        got = ops.dimq_linear_wq(x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], torch.float16), _cuda(bias),
                                 n, k, bits=4, out_dtype=y_dtype, epilogue=epi, residual=res.cuda(), algo="tcgen05")
        assert got.dtype == y_dtype
        tol = 2e-2 if y_dtype == torch.bfloat16 else 1e-2
        max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
        assert max_abs <= tol * 3 and rel <= (5e-3 if y_dtype == torch.bfloat16 else REL_L2), (epi, max_abs, rel)


@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,k,n,bits,grp", [(64, 4096, 1024, 4, None), (256, 4096, 1024, 3, 128), (100, 2048, 384, 2, None),
                                            (200, 1024, 130, 4, None)])
def test_linear_wq_split_k(ops, m, k, n, bits, grp, y_dtype):
    """Few output tiles and a long K: the automatic choice hands the tcgen05 kernel a workspace and it
    splits K; bias, epilogue and residual are applied by the finishing kernel."""
    import ctypes as C

    from dimq_b200 import _lib

    case = make_weight(n, k, bits, seed=bits + m, group_rows=grp, cb_dtype="bf16")
    rng = np.random.default_rng(m + n)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
    bias = rng.standard_normal(n).astype(np.float32)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(y_dtype)
    lin = o.linear_wq(x.float().numpy(), case["packed"], case["codebooks"], bits, n, k, bias, case["group_rows"])
    xc, pw, cb = x.cuda(), _cuda(case["packed"]), _cuda(case["codebooks"], torch.bfloat16)
    w, keep = ops._wq_weight(pw, cb, bits, n, n * k, grp)
    need = C.c_int64(0)
    assert _lib.lib().dimq_linear_wq_workspace_bytes(_lib.ptr(xc), 2, C.byref(w), C.c_int64(m), C.c_int64(n),
                                                     C.c_int64(k), C.byref(need)) == 0
    assert need.value == m * n * 4, "this shape is expected to take the split-K path"
    before = _lib.LAUNCH_COUNT[0]
    got = ops.dimq_linear_wq(xc, pw, cb, _cuda(bias), n, k, bits=bits, group_rows=grp, out_dtype=y_dtype)
    assert _lib.LAUNCH_COUNT[0] - before == 2
    assert ops.last_device_status() == 0
    max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), lin)
    assert max_abs <= (3e-2 if y_dtype == torch.bfloat16 else MAX_ABS) and rel <= (5e-3 if y_dtype == torch.bfloat16 else REL_L2), (max_abs, rel)
    # the same numbers as the unsplit kernel up to the order of the fp32 additions
    ref = ops.dimq_linear_wq(xc, pw, cb, _cuda(bias), n, k, bits=bits, group_rows=grp, out_dtype=torch.float32,
                             algo="tcgen05")
    got32 = ops.dimq_linear_wq(xc, pw, cb, _cuda(bias), n, k, bits=bits, group_rows=grp, out_dtype=torch.float32)
    assert float((got32 - ref).abs().max()) <= 1e-3
    # epilogue and residual in the finishing kernel
    want = np.maximum(lin + res.float().numpy(), 0)
    got = ops.dimq_linear_wq(xc, pw, cb, _cuda(bias), n, k, bits=bits, group_rows=grp, out_dtype=y_dtype,
                             epilogue="add_relu", residual=res.cuda())
    max_abs, rel = o.parity_metrics(got.float().cpu().numpy(), want)
    assert rel <= (5e-3 if y_dtype == torch.bfloat16 else REL_L2), (max_abs, rel)
    del keep


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("k,n", [(1024, 4096), (4096, 1024)])
@pytest.mark.parametrize("m", [1, 4, 16, 64, 256, 4096])
def test_linear_wq_m_sweep_auto_dispatch(ops, bits, k, n, m):
    """The M-sweep of the regime dispatch on ViT-L shapes, bf16 activations, per-layer codebooks."""
    case = _sweep_case(bits, k, n)
    x = bf16_round(np.random.default_rng(m).standard_normal((m, k)).astype(np.float32))
    want = o.linear_wq(x, case["packed"], case["codebooks"], bits, n, k)
    got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), case["packed_cuda"], case["cb_cuda"], None, n, k, bits=bits)
    assert ops.last_device_status() == 0
    _assert_close(got, want, f"sweep bits={bits} m={m} {k}->{n}")
    if m <= 32:
        # what the automatic choice runs here (fp16 codebook, bf16 activations: the reference export's default)
        # is a small-M kernel - the register-resident one from 2 MB of indices on when M <= 16 and K is a
        # multiple of 128 and at least 2048, else the index-streaming one: the two results are the same bits
        small = "mma_regs" if (m <= 16 and k >= 2048 and k % 128 == 0 and n * k * bits // 8 >= 2 << 20) else "mma_stream"
        try:
            forced = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), case["packed_cuda"], case["cb_cuda"], None, n, k,
                                        bits=bits, algo=small)
        except RuntimeError as err:
            # 16 rows of 4096 activations do not fit beside the 64 KB table of the 2-bit form
            assert (m, k, bits, small) == (16, 4096, 2, "mma_stream") and "does not support" in str(err), err
        else:
            assert torch.equal(got, forced)


_SWEEP_CACHE: dict = {}


def _sweep_case(bits, k, n):
    key = (bits, k, n)
    if key not in _SWEEP_CACHE:
        case = make_weight(n, k, bits, seed=bits)
        case["packed_cuda"] = _cuda(case["packed"])
        case["cb_cuda"] = _cuda(case["codebooks"], torch.float16)
        _SWEEP_CACHE[key] = case
    return _SWEEP_CACHE[key]


def test_linear_wq_linearity_at_full_size(ops):
    """Size-independent property at M = 4096: y(a*x1 + x2) = a*y(x1) + y(x2) up to rounding."""
    case = _sweep_case(4, 1024, 4096)
    rng = np.random.default_rng(77)
    x1 = torch.from_numpy(rng.standard_normal((4096, 1024)).astype(np.float32)).cuda()
    x2 = torch.from_numpy(rng.standard_normal((4096, 1024)).astype(np.float32)).cuda()
    f = lambda t: ops.dimq_linear_wq(t.to(torch.float16), case["packed_cuda"], case["cb_cuda"], None, 4096, 1024, bits=4)
    y1, y2, y12 = f(x1), f(x2), f(2.0 * x1 + x2)
    max_abs, rel = o.parity_metrics(y12.cpu().numpy(), (2.0 * y1 + y2).cpu().numpy())
    assert rel <= 2e-3, (max_abs, rel)


# ---- weight-only conv ------------------------------------------------------------------

def test_conv2d_wq_golden(ops, golden):
    x = _cuda(golden["wq_conv_x"])
    for stride, key in (((1, 1), "wq_conv_y"), ((2, 2), "wq_conv_y_s2")):
        y = ops.dimq_conv2d_wq(x, _cuda(golden["wq_conv_packed"]), _cuda(golden["wq_conv_cb"]), None, (8, 4, 3, 3),
                               stride, (1, 1), (1, 1), 1, bits=4)
        np.testing.assert_allclose(y.cpu().numpy(), golden[key], rtol=1e-5, atol=1e-5)
        y = ops.dimq_conv2d_wq(x.contiguous(memory_format=torch.channels_last), _cuda(golden["wq_conv_packed"]),
                               _cuda(golden["wq_conv_cb"]), None, (8, 4, 3, 3), stride, (1, 1), (1, 1), 1, bits=4)
        assert y.is_contiguous(memory_format=torch.channels_last)
        np.testing.assert_allclose(y.cpu().numpy(), golden[key], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_conv2d_wq_generic_per_channel_codebooks(ops, bits):
    rng = np.random.default_rng(bits)
    oc, icg, kh, kw = 16, 6, 3, 3
    case = make_weight(oc, icg * kh * kw, bits, seed=bits, group_rows=1, std=(2.0 / (icg * 9)) ** 0.5,
                       cb_dtype=np.float32)
    x = np.maximum(rng.standard_normal((2, 12, 9, 10)).astype(np.float32), 0)
    bias = rng.standard_normal(oc).astype(np.float32)
    kwargs = dict(stride=(1, 2), padding=(1, 0), dilation=(1, 1), groups=2)
    want = o.conv2d_wq(x, case["packed"], case["codebooks"], bits, (oc, icg, kh, kw), bias, group_rows=1, **kwargs)
    got = ops.dimq_conv2d_wq(_cuda(x), _cuda(case["packed"]), _cuda(case["codebooks"]), _cuda(bias),
                             (oc, icg, kh, kw), kwargs["stride"], kwargs["padding"], kwargs["dilation"], 2, bits=bits,
                             group_rows=1, epilogue="relu")
    np.testing.assert_allclose(got.cpu().numpy(), np.maximum(want, 0), rtol=1e-4, atol=1e-4)


def test_bounded_wait_expires_and_the_context_stays_usable(ops):
    """A wait with a short poll limit on a barrier nobody arrives at must give up, set the CTA abort
    flag and the status word, and return; the status reads once and clears; a GEMM right after runs."""
    import ctypes as C

    from dimq_b200 import _lib

    assert ops.last_device_status() == 0
    result = torch.zeros(2, dtype=torch.int32, device="cuda")
    st = _lib.lib().dimq_selftest_bounded_wait(C.c_uint32(16), _lib.ptr(result), _lib.stream_ptr(result.device))
    assert st == 0
    torch.cuda.synchronize()
    assert result.tolist() == [1, 1]
    assert ops.last_device_status() == 0x80007E57
    assert ops.last_device_status() == 0                      # reading cleared it
    assert _lib.lib().dimq_selftest_bounded_wait(C.c_uint32(0), _lib.ptr(result), None) == -2   # argument check
    cw = make_weight(256, 512, 3, seed=1, group_rows=128, cb_dtype="bf16")
    rng = np.random.default_rng(0)
    for m in (400, 1500):       # the in-pipeline kernel and the expanded form, right after the expiry
        x = bf16_round(rng.standard_normal((m, 512)).astype(np.float32))
        got = ops.dimq_linear_wq(_cuda(x, torch.bfloat16), _cuda(cw["packed"]), _cuda(cw["codebooks"], torch.bfloat16),
                                 None, 256, 512, bits=3, group_rows=128)
        _assert_close(got, o.linear_wq(x, cw["packed"], cw["codebooks"], 3, 256, 512, None, 128), f"m={m}")
    assert ops.last_device_status() == 0
