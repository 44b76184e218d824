"""ctypes binding of ``libhot_b200.so`` (declarations: include/hot_b200.h).

Loading fails loudly when the library has not been built: there is no Python or CPU
fallback behind any of these entry points.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libhot_b200.so")

HOT_OK, HOT_ERR_ARG, HOT_ERR_UNSUPPORTED, HOT_ERR_CUDA, HOT_ERR_TIMEOUT, HOT_ERR_WORKSPACE = range(6)
HOT_F32, HOT_BF16, HOT_I32 = 0, 1, 2
ROUND_NEAREST, ROUND_STOCH_PHILOX, ROUND_STOCH_NOISE = 0, 1, 2
SCALE_TENSOR, SCALE_ROW, SCALE_SAWB = 0, 1, 2
STORE_INT8, STORE_INT4 = 0, 1
LAYOUT_NATURAL, LAYOUT_TRANSPOSED = 0, 1

c_i64, c_i32, c_vp = ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p


class HotQuant(ctypes.Structure):
    _fields_ = [("bits", c_i32), ("storage", c_i32), ("rounding", c_i32), ("scale_mode", c_i32),
                ("seed", ctypes.c_uint64), ("offset", ctypes.c_uint64), ("noise", c_vp)]


class HotLinearCfg(ctypes.Structure):
    _fields_ = [("dtype", c_i32), ("order_o", c_i32), ("order_l", c_i32), ("rank_l", c_i32),
                ("sel_l", c_i32 * 64), ("q_gx", HotQuant), ("q_w", HotQuant), ("q_gw", HotQuant), ("q_x", HotQuant)]


class HotGemmProblem(ctypes.Structure):
    _fields_ = [("a", c_vp), ("a_storage", c_i32), ("lda", c_i64), ("b", c_vp), ("ldb", c_i64), ("M", c_i64), ("N", c_i64),
                ("K", c_i64), ("scale_a", c_vp), ("scale_a_per_row", c_i32), ("scale_b", c_vp), ("scale_b_per_row", c_i32),
                ("post", ctypes.c_float), ("out", c_vp), ("out_dtype", c_i32), ("ldo", c_i64)]


class HotError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str):
        super().__init__("%s failed: %s%s" % (where, _status_text(status), (" (" + detail + ")") if detail else ""))
        self.status = status


EXPORTS = {
    "hot_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "hot_last_error": (ctypes.c_char_p, []),
    "hot_abi_version": (ctypes.c_int, []),
    "hot_set_sm_margin": (None, [ctypes.c_int]),
    "hot_set_wait_limit_ns": (None, [ctypes.c_uint64]),
    "hot_get_wait_limit_ns": (ctypes.c_uint64, []),
    "hot_wait_probe": (ctypes.c_int, [c_vp, c_vp]),
    "hot_check_status": (ctypes.c_int, [ctypes.c_uint32]),
    "hot_row_ht_quant": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_i64, c_i64, ctypes.c_int, ctypes.POINTER(HotQuant),
                                        c_vp, c_i64, c_vp, c_vp, c_vp]),
    "hot_col_ht_quant": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_i64, c_i64, ctypes.c_int, ctypes.POINTER(c_i32),
                                        ctypes.c_int, ctypes.POINTER(HotQuant), ctypes.c_int, c_vp, c_i64, c_vp, c_vp,
                                        c_vp]),
    "hot_row_ht_quant_batched": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_i64, c_i64, c_i64, ctypes.c_int,
                                                ctypes.POINTER(HotQuant), c_vp, c_i64, c_vp, c_vp, c_vp]),
    "hot_col_ht_quant_batched": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_i64, c_i64, c_i64, ctypes.c_int,
                                                ctypes.POINTER(c_i32), ctypes.c_int, ctypes.POINTER(HotQuant), ctypes.c_int,
                                                c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "hot_gemm_i8_dual": (ctypes.c_int, [ctypes.POINTER(HotGemmProblem), ctypes.POINTER(HotGemmProblem), c_vp, c_vp]),
    "hot_gemm_i8_grouped": (ctypes.c_int, [c_vp, c_i64, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_vp, ctypes.c_int, c_vp,
                                           ctypes.c_float, c_vp, ctypes.c_int, c_i64, c_vp, c_vp]),
    "hot_hla_project": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_i64, c_i64, ctypes.c_int, ctypes.POINTER(c_i32), ctypes.c_int,
                                       c_vp, c_i64, c_vp]),
    "hot_hla_expand": (ctypes.c_int, [c_vp, c_i64, c_i64, c_i64, ctypes.c_int, ctypes.POINTER(c_i32), ctypes.c_int,
                                      ctypes.c_float, c_vp, ctypes.c_int, c_i64, c_vp]),
    "hot_col_ht_quant_scratch_words": (ctypes.c_size_t, [ctypes.c_int, c_i64, c_i64, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "hot_col_ht_quant_static": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_i64, c_i64, ctypes.c_int, ctypes.POINTER(c_i32),
                                               ctypes.c_int, ctypes.POINTER(HotQuant), ctypes.c_int, c_vp, c_i64, c_vp,
                                               c_vp]),
    "hot_go_dual_quant": (ctypes.c_int, [c_vp, c_i64, c_i64, c_i64, ctypes.POINTER(HotLinearCfg), c_vp, c_i64, c_vp, c_vp,
                                         c_i64, c_vp, c_vp, c_vp, c_vp]),
    "hot_gemm_i8": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_vp, ctypes.c_int, c_i64, c_i64, c_i64, c_i64, c_vp,
                                   ctypes.c_int, c_vp, ctypes.c_int, ctypes.c_float, c_vp, ctypes.c_int, c_i64, c_vp,
                                   c_vp]),
    "hot_gemm_i8_workspace_bytes": (ctypes.c_size_t, [c_i64, c_i64]),
    "hot_gemm_i8_ws": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, c_vp, ctypes.c_int, c_i64, c_i64, c_i64, c_i64, c_vp,
                                      ctypes.c_int, c_vp, ctypes.c_int, ctypes.c_float, c_vp, ctypes.c_int, c_i64, c_vp,
                                      ctypes.c_size_t, c_vp, c_vp]),
    "hot_linear_workspace_bytes": (ctypes.c_size_t, [c_i64, c_i64, c_i64, ctypes.POINTER(HotLinearCfg)]),
    "hot_abc_pitch": (c_i64, [c_i64, ctypes.POINTER(HotLinearCfg)]),
    "hot_abc_compress": (ctypes.c_int, [c_vp, c_i64, c_i64, c_i64, ctypes.POINTER(HotLinearCfg), c_vp, c_vp, c_vp,
                                        ctypes.c_size_t, c_vp]),
    "hot_linear_backward": (ctypes.c_int, [c_vp, c_i64, c_vp, c_i64, c_vp, c_vp, c_i64, c_i64, c_i64,
                                           ctypes.POINTER(HotLinearCfg), c_vp, c_i64, c_vp, c_i64, c_vp, ctypes.c_size_t,
                                           c_vp, c_vp]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: build it with `python -m hot_b200.build` (there is no fallback path)"
                               % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(handle, name)      # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def _status_text(status: int) -> str:
    try:
        return lib().hot_status_string(status).decode()
    except Exception:  # pragma: no cover
        return "status %d" % status


def check(status: int, where: str) -> None:
    if status != HOT_OK:
        raise HotError(status, where, lib().hot_last_error().decode())
