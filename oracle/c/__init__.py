"""ctypes front-end of the plain-C restatement (oracle/c/oracle.c). Test infrastructure only."""

import ctypes as C

import numpy as np

from .build import build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def reduce(partials):
    p = np.ascontiguousarray(partials, dtype=np.uint16)
    world, rows, n = p.shape
    out = np.empty((rows, n), dtype=np.uint16)
    lib().orc_reduce(_p(p), world, rows, n, _p(out))
    return out


def reduce_norm(partials, weight, eps, scale=1.0, h=None):
    p = np.ascontiguousarray(partials, dtype=np.uint16)
    world, rows, n = p.shape
    w = np.ascontiguousarray(weight, dtype=np.uint16)
    out = np.empty((rows, n), dtype=np.uint16)
    h_after = None if h is None else np.ascontiguousarray(h, dtype=np.uint16).copy()
    lib().orc_reduce_norm(_p(p), _p(h_after) if h_after is not None else None, _p(w), C.c_float(eps), C.c_float(scale),
                          world, rows, n, _p(out))
    return out, h_after


def gemm_bf16(x, w, splits=1):
    x, w = np.ascontiguousarray(x, dtype=np.uint16), np.ascontiguousarray(w, dtype=np.uint16)
    m, k = x.shape
    n = w.shape[0]
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_gemm_bf16(_p(x), _p(w), m, n, k, splits, _p(out))
    return out


def round_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_round_bf16(_p(x), C.c_size_t(x.size), _p(out))
    return out


def nvfp4_dequant(codes, scales, scale2):
    codes, scales = np.ascontiguousarray(codes, dtype=np.uint8), np.ascontiguousarray(scales, dtype=np.uint8)
    rows, k = codes.shape[0], codes.shape[1] * 2
    out = np.empty((rows, k), dtype=np.uint16)
    lib().orc_nvfp4_dequant(_p(codes), _p(scales), C.c_float(scale2), rows, k, _p(out))
    return out


def nvfp4_down(a_codes, a_scales, w_codes, w_scales, g2):
    a_codes, a_scales = np.ascontiguousarray(a_codes, dtype=np.uint8), np.ascontiguousarray(a_scales, dtype=np.uint8)
    w_codes, w_scales = np.ascontiguousarray(w_codes, dtype=np.uint8), np.ascontiguousarray(w_scales, dtype=np.uint8)
    m, f = a_codes.shape[0], a_codes.shape[1] * 2
    n = w_codes.shape[0]
    y = np.empty((m, n), dtype=np.uint16)
    lib().orc_nvfp4_down(_p(a_codes), _p(a_scales), _p(w_codes), _p(w_scales), C.c_float(g2), m, n, f, _p(y))
    return y


def moe_combine(y, ids, weights, lo, local, shared=None):
    y = np.ascontiguousarray(y, dtype=np.uint16)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    rows, top_k = ids.shape
    n = y.shape[-1]
    out = np.empty((rows, n), dtype=np.uint16)
    sh = None if shared is None else np.ascontiguousarray(shared, dtype=np.uint16)
    lib().orc_moe_combine(_p(y), _p(ids), _p(weights), _p(sh) if sh is not None else None, lo, local, rows, top_k, n,
                          _p(out))
    return out
