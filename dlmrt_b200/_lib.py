"""ctypes binding of libdlmrt_b200.so (include/dlmrt_b200.h). There is no fallback: a missing or unbuildable
library is an ImportError, and a non-zero return code is an exception."""

import ctypes as C
from pathlib import Path

MAX_WORLD = 8
EPOCH_SLOTS = 256
STATUS_WORDS = 4
FUSED_MAX_N = 3072
NOALLOC_SCRATCH_BYTES = 8 << 20
GATHER_MAX_BYTES = 1 << 20

OK, ERR_SHAPE, ERR_ALIGN, ERR_WORLD, ERR_NULL, ERR_GRID, ERR_CUDA, ERR_WORKSPACE, ERR_TIMEOUT, ERR_ARCH, \
    ERR_SCRATCH, ERR_OVERLAP = 0, -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11
REDUCE, REDUCE_NORM, REDUCE_NORM_RESIDUAL = 0, 1, 2

LIB_PATH = Path(__file__).resolve().parent / "libdlmrt_b200.so"


class DlmComm(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("rows", C.c_int32), ("n", C.c_int32),
                ("mode", C.c_int32), ("eps", C.c_float), ("scale", C.c_float),
                ("recv", C.c_void_p * MAX_WORLD), ("out", C.c_void_p), ("out_mc", C.c_void_p),
                ("out_peers", C.c_void_p * MAX_WORLD), ("rearm", C.c_void_p), ("rearm_bytes", C.c_int64),
                ("epochs", C.c_void_p), ("h", C.c_void_p), ("weight", C.c_void_p), ("status", C.c_void_p),
                ("stamps", C.c_void_p), ("timeout_ns", C.c_int64), ("pdl", C.c_int32), ("max_ctas", C.c_int32),
                ("one_shot", C.c_int32), ("reserved", C.c_int32), ("recv_mc", C.c_void_p)]


class DlmGemm(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("ldx", C.c_int64), ("ldw", C.c_int64), ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
                ("splits", C.c_int32), ("token_tiles", C.c_int32), ("w_tiled", C.c_int32), ("reserved", C.c_int32)]


class DlmMoe(C.Structure):
    _fields_ = [("act_codes", C.c_void_p), ("act_scales", C.c_void_p), ("amap", C.c_void_p), ("counts", C.c_void_p),
                ("w_codes", C.c_void_p), ("w_scales", C.c_void_p), ("g2", C.c_void_p), ("ids", C.c_void_p),
                ("weights", C.c_void_p), ("shared", C.c_void_p), ("m", C.c_int32), ("n", C.c_int32), ("f", C.c_int32),
                ("top_k", C.c_int32), ("m_max", C.c_int32), ("lo", C.c_int32), ("e_local", C.c_int32),
                ("e_total", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
                ("w_tiled", C.c_int32), ("reserved", C.c_int32)]


class DlmMoeFront(C.Structure):
    _fields_ = [("x", C.c_void_p), ("xq", C.c_void_p), ("xs", C.c_void_p), ("a1_inv", C.c_void_p), ("packed", C.c_void_p),
                ("w13_codes", C.c_void_p), ("w13_scales", C.c_void_p), ("g1", C.c_void_p), ("a2_inv", C.c_void_p),
                ("ids", C.c_void_p), ("weights", C.c_void_p), ("counts", C.c_void_p), ("amap", C.c_void_p),
                ("slot_codes", C.c_void_p), ("slot_scales", C.c_void_p), ("act_codes", C.c_void_p),
                ("act_scales", C.c_void_p), ("m", C.c_int32), ("hidden", C.c_int32), ("f", C.c_int32),
                ("top_k", C.c_int32), ("m_max", C.c_int32), ("lo", C.c_int32), ("e_local", C.c_int32),
                ("e_total", C.c_int32), ("activation", C.c_int32), ("w13_tiled", C.c_int32)]


class DlmStatus(C.Structure):
    _fields_ = [("code", C.c_int32), ("block", C.c_int32), ("slot", C.c_int32), ("phase", C.c_int32),
                ("epoch", C.c_int32)]


class DlmLoopPart(C.Structure):
    _fields_ = [("graph", C.c_void_p), ("flag", C.c_void_p)]


class DlmLoop(C.Structure):
    _fields_ = [("parts", C.POINTER(DlmLoopPart)), ("n_parts", C.c_int32), ("limit", C.c_int32),
                ("remaining", C.c_void_p), ("step", C.c_void_p)]


MAX_LOOPS, MAX_LOOP_PARTS = 8, 16


class DlmError(RuntimeError):
    """A DLM_ERR_* return code from the library; `.code` holds it."""

    def __init__(self, code, where):
        self.code = code
        detail = f" (cudaError {lib().dlm_last_cuda_error()})" if code == ERR_CUDA else ""
        super().__init__(f"{where}: {lib().dlm_strerror(code).decode()}{detail}")


_lib = None

SIGNATURES = {
    "dlm_reduce_bf16": (C.c_int, [C.c_void_p, C.POINTER(DlmComm), C.c_void_p]),
    "dlm_reduce_bf16_loopback": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(DlmComm), C.c_int, C.c_void_p]),
    "dlm_all_gather": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(DlmComm), C.c_void_p]),
    "dlm_all_gather_loopback": (C.c_int, [C.POINTER(C.c_void_p), C.c_int64, C.POINTER(DlmComm), C.c_int, C.c_void_p]),
    "dlm_gemm_bf16": (C.c_int, [C.POINTER(DlmGemm), C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "dlm_gemm_bf16_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64,
                                        C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "dlm_rowpar_bf16": (C.c_int, [C.POINTER(DlmGemm), C.POINTER(DlmComm), C.c_void_p]),
    "dlm_rowpar_bf16_loopback": (C.c_int, [C.POINTER(DlmGemm), C.POINTER(DlmComm), C.c_int, C.c_void_p]),
    "dlm_moe_nvfp4": (C.c_int, [C.POINTER(DlmMoe), C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "dlm_rowpar_nvfp4_moe": (C.c_int, [C.POINTER(DlmMoe), C.POINTER(DlmComm), C.c_void_p]),
    "dlm_rowpar_nvfp4_moe_loopback": (C.c_int, [C.POINTER(DlmMoe), C.POINTER(DlmComm), C.c_int, C.c_void_p]),
    "dlm_moe_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "dlm_moe_front_nvfp4": (C.c_int, [C.POINTER(DlmMoeFront), C.c_int, C.c_void_p]),
    "dlm_route_packed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "dlm_abi_check_front": (C.c_int, [C.c_size_t]),
    "dlm_abi_check_moe": (C.c_int, [C.c_size_t]),
    "dlm_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "dlm_choose_tiling": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "dlm_status_read": (C.c_int, [C.c_void_p, C.POINTER(DlmStatus), C.c_void_p]),
    "dlm_abi_check": (C.c_int, [C.c_size_t, C.c_size_t, C.c_size_t]),
    "dlm_strerror": (C.c_char_p, [C.c_int]),
    "dlm_last_cuda_error": (C.c_int, []),
    "dlm_device_sms": (C.c_int, []),
    "dlm_device_arch": (C.c_int, []),
    "dlm_launch_count": (C.c_int64, []),
    "dlm_device_loop_create": (C.c_int, [C.c_void_p, C.POINTER(DlmLoop), C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "dlm_device_loop_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "dlm_device_loop_destroy": (None, [C.c_void_p]),
}


def lib():
    """The loaded library; raises ImportError when it has not been built (python -m dlmrt_b200.build)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m dlmrt_b200.build` "
                              "(there is no CPU or PyTorch fallback for this path)")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        if handle.dlm_abi_check(C.sizeof(DlmComm), C.sizeof(DlmGemm), C.sizeof(DlmStatus)) != OK or \
                handle.dlm_abi_check_moe(C.sizeof(DlmMoe)) != OK or \
                handle.dlm_abi_check_front(C.sizeof(DlmMoeFront)) != OK:
            raise ImportError(f"{LIB_PATH}: struct layout differs from this binding; rebuild the library")
        _lib = handle
    return _lib


def check(code, where):
    if code != OK:
        raise DlmError(code, where)
