"""Run-time control of the cuBLAS interception layer from Python.

Same function names and constants as the reference's pybind11 module
``cumpsgemm_hijack_control`` (``python/src/main.cpp:111-172``, the functions of
``include/cumpsgemm/hijack_control.hpp``), implemented over the plain-C
``cuMpSGEMM_hijack_*`` entry points.  When the process was started with
``LD_PRELOAD=libcumpsgemm.so`` the functions act on that preloaded library (the one that
intercepts the application's cuBLAS calls); otherwise they act on the in-tree library loaded
by :mod:`cumpsgemm_b200._lib`, which is useful for calling the intercepted symbols directly.

    import cumpsgemm_b200.hijack_control as chc
    chc.set_control_function(lambda op_A, op_B, m, n, k: chc.CUMPSGEMM_FP16TCEC)
"""
from __future__ import annotations

import ctypes as C

from . import _lib

CUMPSGEMM_CUBLAS = 0
CUMPSGEMM_FP16TCEC = 1
CUMPSGEMM_TF32TCEC = 2
CUMPSGEMM_FP16TC = 3
CUMPSGEMM_TF32TC = 4
CUMPSGEMM_CUBLAS_SIMT = 5
CUMPSGEMM_CUBLAS_FP16TC = 6
CUMPSGEMM_CUBLAS_TF32TC = 7
CUMPSGEMM_DRY_RUN = 8
CUMPSGEMM_AUTO = 9
CUMPSGEMM_FP16TCEC_SCALING = 11

_CONTROL_CB = C.CFUNCTYPE(C.c_int, C.c_int, C.c_int, C.c_uint, C.c_uint, C.c_uint)
_state = {"lib": None, "preloaded": False, "callback": None}


def _library():
    if _state["lib"] is None:
        lib = None
        try:
            process = C.CDLL(None)
            process.cuMpSGEMM_hijack_is_library_loaded  # raises AttributeError when not preloaded
            lib = process
            _state["preloaded"] = True
            for name, (restype, argtypes) in _lib.PROTOTYPES.items():
                if name.startswith("cuMpSGEMM_hijack_"):
                    fn = getattr(lib, name)
                    fn.restype, fn.argtypes = restype, argtypes
        except AttributeError:
            lib = _lib.load()
        _state["lib"] = lib
    return _state["lib"]


def is_library_loaded() -> bool:
    """True when the interception library is preloaded into this process."""
    _library()
    return bool(_state["preloaded"])


def set_compute_mode(mode: int) -> None:
    if _library().cuMpSGEMM_hijack_set_compute_mode(int(mode)) != 0:
        raise RuntimeError("CUMPSGEMM_FP32_SIMT mode is currently not supported.")


def unset_compute_mode() -> None:
    _library().cuMpSGEMM_hijack_unset_compute_mode()


def enable_custom_gemm_Mx2x2() -> None:
    _library().cuMpSGEMM_hijack_enable_custom_gemm_Mx2x2()


def disable_custom_gemm_Mx2x2() -> None:
    _library().cuMpSGEMM_hijack_disable_custom_gemm_Mx2x2()


def set_exp_stats_params(ignore_threshold: float, underflow_threshold: float,
                         underflow_tolerance_rate: float) -> None:
    _library().cuMpSGEMM_hijack_set_exp_stats_params(ignore_threshold, underflow_threshold,
                                                     underflow_tolerance_rate)


def reset_exp_stats_buffer_id() -> None:
    _library().cuMpSGEMM_hijack_reset_exp_stats_buffer_id()


def enable_restoring_AB_after_scaling() -> None:
    _library().cuMpSGEMM_hijack_enable_restoring_AB_after_scaling()


def disable_restoring_AB_after_scaling() -> None:
    _library().cuMpSGEMM_hijack_disable_restoring_AB_after_scaling()


def get_last_called_function_str() -> str:
    lib = _library()
    size = lib.cuMpSGEMM_hijack_get_last_called_function_str(None, 0) + 1
    buf = C.create_string_buffer(size)
    lib.cuMpSGEMM_hijack_get_last_called_function_str(buf, size)
    return buf.value.decode()


def set_last_called_function_str(func_str: str) -> None:
    _library().cuMpSGEMM_hijack_set_last_called_function_str(func_str.encode())


def clear_last_called_function_str() -> None:
    _library().cuMpSGEMM_hijack_clear_last_called_function_str()


def set_control_function(control_function) -> None:
    """control_function(op_A, op_B, m, n, k) -> compute mode, called for every intercepted GEMM."""
    cb = _CONTROL_CB(lambda a, b, m, n, k: int(control_function(a, b, m, n, k)))
    _state["callback"] = cb  # keep the trampoline alive
    _library().cuMpSGEMM_hijack_set_control_function(C.cast(cb, C.c_void_p))


def unset_control_function() -> None:
    _library().cuMpSGEMM_hijack_set_control_function(None)
    _state["callback"] = None
