"""ctypes binding of libjq.so (the C ABI declared in include/jq.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int32, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))

JQ_F32, JQ_F16, JQ_BF16 = 0, 1, 2
JQ_FMT_E2M1, JQ_FMT_GF4 = 0, 1


class JqError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {strerror(status)} (status {status})")


class jq_problem(ctypes.Structure):
    _fields_ = [
        ("qweight", c_void_p), ("scales", c_void_p), ("codebook", c_void_p),
        ("x", c_void_p), ("bias", c_void_p), ("y", c_void_p),
        ("N", c_int32), ("K", c_int32), ("g", c_int32), ("had_block", c_int32),
        ("ldy", c_int32), ("reserved", c_int32 * 3),
    ]


_SIGNATURES = {
    "jq_version": (c_int, []),
    "jq_strerror": (c_char_p, [c_int]),
    "jq_dequant_e2m1": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "jq_dequant_gf4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "jq_fwht_block": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "jq_gemv_e2m1": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "jq_gemv_gf4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "jq_gemv_noalloc": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "jq_ta_workspace_bytes": (c_size_t, [c_void_p, c_int, c_int]),
    "jq_ta_plan_bytes": (c_size_t, [c_int]),
    "jq_ta_plan": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p, c_size_t]),
    "jq_gemm_ta_grouped": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "jq_gemm_ta": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "jq_ta_status": (c_int, [c_void_p, c_int, c_void_p]),
    "jq_selftest_bounded_wait": (c_int, [c_void_p, ctypes.c_uint, c_void_p]),
    "jq_grouped_plan_bytes": (c_size_t, [c_int]),
    "jq_grouped_plan": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_size_t]),
    "jq_gemv_grouped": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "jq_gemv_grouped_peers": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "jq_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "jq_jenks2_workspace_bytes": (c_size_t, [ctypes.c_longlong]),
    "jq_jenks2_break": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "jq_pack_e2m1": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "jq_pack_gf4_workspace_bytes": (c_size_t, [c_int]),
    "jq_pack_gf4": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "jq_pack_e2m1_host": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int]),
    "jq_pack_gf4_host": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int]),
    "jq_rotate_weights_host": (c_int, [c_void_p, c_int, c_int, c_int, c_int]),
}

_lib = None


def lib_path() -> str:
    return os.environ.get("JQ_LIB", os.path.join(HERE, "libjq.so"))


def load():
    """Load libjq.so once; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} not found: build it with `python -m if_i_could_turn_back_time_b200.build` "
                "(there is no CPU fallback)")
        lib = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def exported_symbols():
    return list(_SIGNATURES)


def strerror(status: int) -> str:
    return load().jq_strerror(int(status)).decode()


def check(status: int, where: str) -> None:
    if status != 0:
        raise JqError(status, where)
