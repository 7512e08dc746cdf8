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
    "fq_gdr_bwd_chunk_grouped": [_vp] * 16 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_gdr_bwd_chunk_gva_noalloc": [_vp] * 16 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp, _vp],
    "fq_group_reduce": [_vp, _vp, ctypes.c_longlong, _i32, _i32, _vp],
    "fq_group_reduce_pair": [_vp, _vp, _vp, _vp, ctypes.c_longlong, _i32, _i32, _vp],
    "fq_gdr_recurrent": [_vp] * 8 + [_i32] * 4 + [_f32, _vp],
    "fq_l2norm_fwd": [_vp, _vp, ctypes.c_longlong, _f32, _vp],
    "fq_l2norm_bwd": [_vp, _vp, _vp, ctypes.c_longlong, _f32, _vp],
    "fq_kkt_solve_gated": [_vp] * 7 + [_i32] * 5 + [_vp, _vp, _i32, _i32, _f32, _vp],
    "fq_kkt_solve_fused": [_vp] * 8 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp],
    "fq_kkt_solve_fused_act": [_vp] * 5 + [_i32, _i32] + [_vp] * 4 + [_i32] * 4 + [_vp, _vp, _i32, _i32, _f32, _vp],
    "fq_gate_act_bwd": [_vp] * 6 + [_i32, _i32] + [_vp] * 4 + [ctypes.c_longlong, _i32, _vp],
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
        return _lib if _recorder is None else _RecordingLib(_lib, _recorder)
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
    return _lib if _recorder is None else _RecordingLib(_lib, _recorder)


class LaunchRecorder:
    """Optional per-launch timing for benchmarks and profiling: while a recorder is active (``with
    _lib.record_launches() as rec:``), every C-ABI call is bracketed by two CUDA events on the current stream.
    ``rec.summary()`` (after a synchronise) gives {entry point: (calls, total ms)}; calls of one entry point within a
    step are numbered (``fq_gdr_fwd_cp_ex#0`` is the state pass, ``#1`` the final pass).  Costs two event records per
    launch; off by default."""

    def __init__(self):
        self.events = []      # (name, start, stop)
        self._step_counts = {}

    def new_step(self):
        self._step_counts = {}

    def wrap(self, name, fn):
        import torch

        def call(*args):
            i = self._step_counts.get(name, 0)
            self._step_counts[name] = i + 1
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args)
            e1.record()
            self.events.append((f"{name}#{i}" if i or name in _MULTI else name, e0, e1))
            return rc
        return call

    def summary(self):
        out = {}
        for name, e0, e1 in self.events:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + e0.elapsed_time(e1))
        return out


_MULTI = {"fq_gdr_fwd_cp_ex", "fq_gdr_bwd_dh_cp_ex", "fq_gdr_fwd", "fq_gdr_fwd_cp"}
_NOT_LAUNCHES = {"fq_version", "fq_last_error"}
_recorder = None


class _RecordingLib:
    def __init__(self, lib, rec):
        self._lib, self._rec = lib, rec

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name in _NOT_LAUNCHES:
            return fn
        return self._rec.wrap(name, fn)


class record_launches:
    def __enter__(self):
        global _recorder
        _recorder = LaunchRecorder()
        return _recorder

    def __exit__(self, *exc):
        global _recorder
        _recorder = None
        return False


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().fq_last_error()
        raise FlashQLAError(f"{what} failed with code {rc}: {msg.decode() if msg else ''}")
