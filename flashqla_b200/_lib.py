"""ctypes loader for libflashqla_sm100.so (the C ABI declared in include/flashqla.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLASHQLA_LIB", os.path.join(_PKG, "libflashqla_sm100.so"))

_lock = threading.Lock()
_lib = None

_i32, _f32, _vp, _cp = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p

# name -> argtypes; every entry point returns int unless listed in _RESTYPES
SIGNATURES = {
    "fq_version": [],
    "fq_last_error": [],
    "fq_chunk_cumsum": [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _vp],
    "fq_dg_boundary_fix": [_vp] * 6 + [_i32] * 3 + [_vp, _vp, _i32, _i32, _vp],
    "fq_kkt_solve": [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _vp],
    "fq_gdr_fwd": [_vp] * 12 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_gdr_fwd_cp": [_vp] * 14 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_cp_warmup": [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _f32, _i32, _i32, _vp, _vp, _vp],
    "fq_gdr_fwd_cp_ex": [_vp] * 13 + [_i32, _vp, _vp, _vp] + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_cp_transition_plan": [_vp] * 7 + [_i32] * 2 + [_vp],
    "fq_cp_plan": [_vp] * 12 + [_i32] * 3 + [_f32, _i32, _vp],
    "fq_cp_chain": [_vp] * 4 + [_i32] * 3 + [_vp],
    "fq_cp_chain_ex": [_vp] * 6 + [_i32] * 4 + [_vp],
    "fq_gdr_bwd_dh_cp_ex": [_vp] * 15 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_cp_transition_plan_reverse": [_vp] * 7 + [_i32] * 2 + [_vp],
    "fq_cp_chain_reverse": [_vp] * 5 + [_i32] * 3 + [_vp],
    "fq_gdr_bwd_dh": [_vp] * 10 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_gdr_bwd_dh_cp": [_vp] * 14 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_gdr_bwd_chunk": [_vp] * 16 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_gdr_bwd_chunk_gva_noalloc": [_vp] * 16 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_group_reduce": [_vp, _vp, ctypes.c_longlong, _i32, _i32, _vp],
    "fq_group_reduce_pair": [_vp, _vp, _vp, _vp, ctypes.c_longlong, _i32, _i32, _vp],
    "fq_gdr_recurrent": [_vp] * 8 + [_i32] * 4 + [_f32, _vp],
    "fq_l2norm_fwd": [_vp, _vp, ctypes.c_longlong, _f32, _vp],
    "fq_l2norm_bwd": [_vp, _vp, _vp, ctypes.c_longlong, _f32, _vp],
    "fq_kkt_solve_gated": [_vp] * 7 + [_i32] * 5 + [_vp, _vp, _i32, _i32, _f32, _vp],
    "fq_kkt_solve_fused": [_vp] * 8 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp],
    "fq_selftest_umma": [_vp, _vp, _vp, _i32, _vp, _vp],
    "fq_selftest_wait_expiry": [_vp, _vp, ctypes.c_longlong, _vp],
}
_RESTYPES = {"fq_last_error": _cp}


class FlashQLAError(RuntimeError):
    pass


def load():
    """Return the loaded library, loading it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise FlashQLAError(
                    f"{LIB_PATH} not found: build it with `python -m flashqla_b200.build` "
                    "(there is no fallback implementation)")
            lib = ctypes.CDLL(LIB_PATH)
            for name, argtypes in SIGNATURES.items():
                fn = getattr(lib, name)  # AttributeError if the symbol is missing
                fn.argtypes = argtypes
                fn.restype = _RESTYPES.get(name, _i32)
            _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().fq_last_error()
        raise FlashQLAError(f"{what} failed with code {rc}: {msg.decode() if msg else ''}")
