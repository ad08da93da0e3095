"""ctypes binding of ``libdimq_b200.so`` (the C ABI declared in include/dimq_b200.h).

There is no CPU or PyTorch fallback behind this module: if the shared library is
missing or an entry point reports an error, a ``RuntimeError`` is raised.
"""

from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

import torch

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libdimq_b200.so"

F32, F16, BF16 = 0, 1, 2
ALGO_AUTO, ALGO_GENERIC, ALGO_STREAM, ALGO_TCGEN05 = 0, 1, 2, 3
EPI_NONE, EPI_RELU, EPI_GELU, EPI_ADD_RELU = 0, 1, 2, 3

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

# every symbol include/dimq_b200.h declares
EXPORTED_SYMBOLS = (
    "dimq_version", "dimq_status_string", "dimq_pack_u4", "dimq_unpack_u4", "dimq_pack_bits",
    "dimq_unpack_bits", "dimq_quantize_activation_u4", "dimq_build_product_table", "dimq_linear_lut",
    "dimq_conv_out_size", "dimq_conv2d_lut", "dimq_hard_quantize", "dimq_linear_wq", "dimq_conv2d_wq",
    "dimq_last_device_status", "dimq_add_layer_norm", "dimq_conv_prepack", "dimq_conv2d_wq_static", "dimq_im2col", "dimq_max_pool_nhwc", "dimq_images_to_nhwc",
    "dimq_a4_workspace_bytes", "dimq_linear_lut_tc", "dimq_conv2d_lut_tc",
    "dimq_linear_wq_workspace_bytes", "dimq_linear_wq_ws", "dimq_expand_workspace_bytes", "dimq_linear_wq_expand",
    "dimq_linear_wq_regs_workspace_bytes", "dimq_linear_wq_regs", "dimq_linear_prepack",
    "dimq_conv2d_wq_workspace_bytes", "dimq_conv2d_wq_ws", "dimq_conv2d_wq_expand", "dimq_selftest_bounded_wait", "dimq_fake_quantize_ste", "dimq_centre_quantize_u4",
)


class ConvGeom(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "batch", "in_channels", "in_h", "in_w", "out_channels", "in_channels_per_group", "kernel_h", "kernel_w",
        "stride_h", "stride_w", "pad_h", "pad_w", "dilation_h", "dilation_w", "groups", "out_h", "out_w")] + [
        ("x_stride", C.c_int64 * 4), ("y_stride", C.c_int64 * 4)]


class WqWeight(C.Structure):
    _fields_ = [("packed", C.c_void_p), ("bits", C.c_int32), ("codebooks", C.c_void_p), ("cb_dtype", C.c_int32),
                ("entries", C.c_int32), ("groups", C.c_int64), ("group_rows", C.c_int64), ("packed_khwc", C.c_void_p)]


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    """Load the shared library (built by ``dimq_b200.build``); raise if it is absent."""
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build the sm_100a kernels with `python -m dimq_b200.build` "
            "(needs nvcc).  dimq_b200 has no CPU fallback."
        )
    handle = C.CDLL(str(LIB_PATH))
    handle.dimq_status_string.restype = C.c_char_p
    handle.dimq_status_string.argtypes = [C.c_int]
    for name in EXPORTED_SYMBOLS:
        if name != "dimq_status_string":
            getattr(handle, name).restype = C.c_int
    return handle


def is_available() -> bool:
    try:
        lib()
    except (RuntimeError, OSError):
        return False
    return True


# number of kernels this process has launched through the C ABI (one per successful entry-point call)
LAUNCH_COUNT = [0]


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().dimq_status_string(int(status)).decode()
        raise RuntimeError(f"dimq_b200.{what} failed: {msg} (status {status})")
    if what != "last_device_status":
        LAUNCH_COUNT[0] += 1


def dtype_code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"{what} must be float32, float16 or bfloat16, got {t.dtype}") from None


def ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr(device: torch.device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
