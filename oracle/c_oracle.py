"""ctypes front end of oracle/dimq_oracle.c (test infrastructure only)."""

from __future__ import annotations

import ctypes as C

import numpy as np

from .build_oracle import build

_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(str(build()))
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def pack_bits(idx: np.ndarray, bits: int) -> np.ndarray:
    flat = np.ascontiguousarray(idx, dtype=np.uint8).reshape(-1)
    out = np.zeros(((flat.size * bits + 7) // 8,), dtype=np.uint8)
    lib().dimq_oracle_pack_bits(_p(flat), C.c_int64(flat.size), C.c_int(bits), _p(out))
    return out


def unpack_bits(packed: np.ndarray, n: int, bits: int) -> np.ndarray:
    flat = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    out = np.zeros((n,), dtype=np.uint8)
    lib().dimq_oracle_unpack_bits(_p(flat), C.c_int64(n), C.c_int(bits), _p(out))
    return out


def hard_quantize(w: np.ndarray, codebooks: np.ndarray, group_rows: int | None = None) -> np.ndarray:
    wf = np.ascontiguousarray(w, dtype=np.float32)
    cb = np.ascontiguousarray(codebooks, dtype=np.float32)
    if cb.ndim == 1:
        rows, cols, grp = 1, wf.size, 1
    else:
        rows = wf.shape[0]
        cols = wf.size // max(rows, 1)
        grp = int(group_rows) if group_rows else rows
    out = np.zeros(wf.shape, dtype=np.uint8)
    lib().dimq_oracle_hard_quantize(_p(wf), C.c_int64(rows), C.c_int64(cols), _p(cb), C.c_int(cb.shape[-1]),
                                    C.c_int64(grp), _p(out))
    return out


def quantize_activation_u4(x: np.ndarray, s: float, z: int) -> np.ndarray:
    xf = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(xf.shape, dtype=np.uint8)
    lib().dimq_oracle_quantize_activation_u4(_p(xf), C.c_int64(xf.size), C.c_float(s), C.c_int(z), _p(out))
    return out


def product_table(cb: np.ndarray, s: float, z: int) -> np.ndarray:
    c = np.ascontiguousarray(cb, dtype=np.float32).reshape(-1)
    out = np.zeros((c.size, 16), dtype=np.float32)
    lib().dimq_oracle_product_table(_p(c), C.c_int(c.size), C.c_float(s), C.c_int(z), _p(out))
    return out


def linear_lut_a4(x, packed_w, cb, s, z, n_out, k_in, bias=None) -> np.ndarray:
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k_in)
    pw = np.ascontiguousarray(packed_w, dtype=np.uint8)
    c = np.ascontiguousarray(cb, dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    y = np.zeros((x2.shape[0], n_out), dtype=np.float32)
    lib().dimq_oracle_linear_lut_a4(_p(x2), _p(pw), _p(c), C.c_float(s), C.c_int(z),
                                    None if b is None else _p(b), _p(y), C.c_int64(x2.shape[0]),
                                    C.c_int64(n_out), C.c_int64(k_in))
    return y.reshape(*np.shape(x)[:-1], n_out)


def conv2d_lut_a4(x, packed_w, cb, s, z, weight_shape, bias=None, stride=(1, 1), padding=(0, 0),
                  dilation=(1, 1), groups=1) -> np.ndarray:
    xf = np.ascontiguousarray(x, dtype=np.float32)
    pw = np.ascontiguousarray(packed_w, dtype=np.uint8)
    c = np.ascontiguousarray(cb, dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    oc, icg, kh, kw = (int(v) for v in weight_shape)
    bsz, ch, h, w = xf.shape
    oh = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (w + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    y = np.zeros((bsz, oc, oh, ow), dtype=np.float32)
    ints = [bsz, ch, h, w, oc, icg, kh, kw, stride[0], stride[1], padding[0], padding[1], dilation[0],
            dilation[1], groups]
    lib().dimq_oracle_conv2d_lut_a4(_p(xf), _p(pw), _p(c), C.c_float(s), C.c_int(z),
                                    None if b is None else _p(b), _p(y), *[C.c_int(int(v)) for v in ints])
    return y


def linear_wq(x, packed_w, bits, codebooks, n_out, k_in, bias=None, group_rows=None) -> np.ndarray:
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k_in)
    pw = np.ascontiguousarray(packed_w, dtype=np.uint8)
    cb = np.ascontiguousarray(codebooks, dtype=np.float32)
    grp = int(group_rows) if (group_rows and cb.ndim == 2 and cb.shape[0] > 1) else n_out
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    y = np.zeros((x2.shape[0], n_out), dtype=np.float32)
    lib().dimq_oracle_linear_wq(_p(x2), _p(pw), C.c_int(bits), _p(cb), C.c_int(cb.shape[-1]), C.c_int64(grp),
                                None if b is None else _p(b), _p(y), C.c_int64(x2.shape[0]), C.c_int64(n_out),
                                C.c_int64(k_in))
    return y.reshape(*np.shape(x)[:-1], n_out)
