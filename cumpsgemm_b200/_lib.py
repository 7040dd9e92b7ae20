"""ctypes loader for ``libcumpsgemm.so`` and prototypes of its C ABI.

The library is loaded from ``cumpsgemm_b200/lib`` (built in-tree by
:mod:`cumpsgemm_b200.build`).  There is no fallback: if the shared object is
missing and cannot be built, importing the compute API raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

_LIB = None

u64 = C.c_uint64
u32 = C.c_uint
i32 = C.c_int
vp = C.c_void_p
f32 = C.c_float


def _proto(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


# name -> (restype, argtypes); every symbol include/cumpsgemm/*.h declares.
_GEMM_ARGS = [vp, i32, i32, u64, u64, u64, vp, vp, u64, vp, u64, vp, vp, u64, i32]
_GEMM_SB_ARGS = [vp, i32, i32, u64, u64, u64, vp, vp, u64, u64, vp, u64, u64, vp, vp, u64, u64,
                 u64, i32]
_TINY_ARGS = [vp, i32, i32, u64, vp, vp, u64, u64, vp, u64, u64, vp, vp, u64, u64, u64]
_STATS_ARGS = [vp, u32, u32, vp, u32, u32, u32]
_SCALE_ARGS = [vp, u32, u32, u32, u32, vp, u32, u32, u32]
_SCALE_C_ARGS = [vp, u32, u32, u32, u32, u32, vp, u32, u32, u32]

PROTOTYPES = {
    # include/cumpsgemm/cumpsgemm.h
    "cuMpSGEMM_create": (i32, [C.POINTER(vp)]),
    "cuMpSGEMM_destroy": (i32, [vp]),
    "cuMpSGEMM_set_stream": (i32, [vp, vp]),
    "cuMpSGEMM_get_compute_mode_string": (C.c_char_p, [i32]),
    "cuMpSGEMM_get_compute_mode": (i32, [C.c_char_p, vp, i32, i32, u32, u32, u32]),
    "cuMpSGEMM_sgemm": (i32, _GEMM_ARGS),
    "cuMpSGEMM_cgemm": (i32, _GEMM_ARGS),
    "cuMpSGEMM_sgemm_strided_batch": (i32, _GEMM_SB_ARGS),
    "cuMpSGEMM_cgemm_strided_batch": (i32, _GEMM_SB_ARGS),
    # include/cumpsgemm/cumpsgemm_ext.h
    "cuMpSGEMM_exp_stats_ext_s": (u32, _STATS_ARGS),
    "cuMpSGEMM_exp_stats_ext_c": (u32, _STATS_ARGS),
    "cuMpSGEMM_exp_max_ext_s": (u32, _STATS_ARGS),
    "cuMpSGEMM_exp_max_ext_c": (u32, _STATS_ARGS),
    "cuMpSGEMM_get_exp_stats": (None, [vp, u32, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "cuMpSGEMM_get_current_exp_stats_buffer_id": (u32, [vp]),
    "cuMpSGEMM_reset_exp_stats_buffer_id": (None, [vp]),
    "cuMpSGEMM_set_exp_stats_params": (None, [vp, f32, f32, f32]),
    "cuMpSGEMM_enable_exp_stats": (None, [vp]),
    "cuMpSGEMM_disable_exp_stats": (None, [vp]),
    "cuMpSGEMM_get_max_exp": (f32, [vp, u32]),
    "cuMpSGEMM_get_exp_stats_compute_mode_level": (i32, [vp, u32]),
    "cuMpSGEMM_scale_A_s": (None, _SCALE_ARGS),
    "cuMpSGEMM_scale_A_c": (None, _SCALE_ARGS),
    "cuMpSGEMM_scale_B_s": (None, _SCALE_ARGS),
    "cuMpSGEMM_scale_B_c": (None, _SCALE_ARGS),
    "cuMpSGEMM_scale_C_s": (None, _SCALE_C_ARGS),
    "cuMpSGEMM_scale_C_c": (None, _SCALE_C_ARGS),
    "cuMpSGEMM_reset_scale_A_s": (None, _SCALE_ARGS),
    "cuMpSGEMM_reset_scale_A_c": (None, _SCALE_ARGS),
    "cuMpSGEMM_reset_scale_B_s": (None, _SCALE_ARGS),
    "cuMpSGEMM_reset_scale_B_c": (None, _SCALE_ARGS),
    "cuMpSGEMM_get_current_dynamic_launch_buffer_id": (u32, [vp]),
    "cuMpSGEMM_get_next_dynamic_launch_buffer_id": (u32, [vp]),
    "cuMpSGEMM_get_dynamic_launch_gemm_compute_mode": (i32, [vp, u32]),
    "cuMpSGEMM_get_dynamic_launch_scaling_mode_AB": (None, [vp, u32, C.POINTER(i32),
                                                            C.POINTER(i32)]),
    "cuMpSGEMM_set_dynamic_launch_buffer_by_exp_stats": (None, [vp, u32, u32, u32]),
    "cuMpSGEMM_set_dynamic_launch_flag_buffer_id": (None, [vp, u32]),
    "cuMpSGEMM_unset_dynamic_launch_flag_buffer_id": (None, [vp]),
    "cuMpSGEMM_enable_exp_stats_profiling": (None, [vp]),
    "cuMpSGEMM_disable_exp_stats_profiling": (None, [vp]),
    "cuMpSGEMM_reset_exp_stats_profiling": (None, [vp]),
    "cuMpSGEMM_print_exp_stats_profiling": (None, [vp, u32]),
    "cuMpSGEMM_get_exp_stats_profiling_result": (i32, [vp, C.c_char_p, C.POINTER(C.c_double),
                                                       C.POINTER(C.c_ulonglong)]),
    "cuMpSGEMM_sgemm_module": (i32, _GEMM_ARGS + [C.POINTER(u32)]),
    "cuMpSGEMM_get_kernel_status": (i32, [vp]),
    "cuMpSGEMM_selftest_bounded_wait": (i32, [vp, u32, C.POINTER(C.c_double)]),
    "cuMpSGEMM_set_workspace_limit": (None, [vp, C.c_size_t]),
    "cuMpSGEMM_set_count_tail_padding": (None, [vp, i32]),
    "cuMpSGEMM_reload_tuning_env": (None, [vp]),
    "cuMpSGEMM_plan_pair_tail": (i32, [u32, u32, u32, i32, C.POINTER(u32), C.POINTER(u32),
                                       C.POINTER(u32), C.POINTER(u32)]),
    "cuMpSGEMM_set_debug_buffer": (None, [vp, vp]),
    "cuMpSGEMM_set_kernel_timing": (None, [vp, i32]),
    "cuMpSGEMM_get_kernel_timing": (C.c_ulonglong, [vp, C.POINTER(C.c_double),
                                                    C.POINTER(C.c_double)]),
    "cuMpSGEMM_hijack_get_internal_global_handle": (vp, []),
    "cuMpSGEMM_hijack_set_compute_mode": (i32, [i32]),
    "cuMpSGEMM_hijack_unset_compute_mode": (None, []),
    "cuMpSGEMM_hijack_reset_exp_stats_buffer_id": (None, []),
    "cuMpSGEMM_hijack_set_exp_stats_params": (None, [f32, f32, f32]),
    "cuMpSGEMM_hijack_enable_restoring_AB_after_scaling": (None, []),
    "cuMpSGEMM_hijack_disable_restoring_AB_after_scaling": (None, []),
    "cuMpSGEMM_hijack_get_last_called_function_str": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "cuMpSGEMM_hijack_set_last_called_function_str": (None, [C.c_char_p]),
    "cuMpSGEMM_hijack_clear_last_called_function_str": (None, []),
    "cuMpSGEMM_hijack_enable_custom_gemm_Mx2x2": (None, []),
    "cuMpSGEMM_hijack_disable_custom_gemm_Mx2x2": (None, []),
    "cuMpSGEMM_hijack_is_library_loaded": (i32, []),
    "cuMpSGEMM_hijack_set_control_function": (None, [vp]),
    "cuMpSGEMM_get_compute_mode_internal": (i32, [C.c_char_p, vp, i32, i32, u32, u32, u32]),
    "cuMpSGEMM_exp_stats_begin": (u32, [vp]),
    "cuMpSGEMM_exp_stats_stage_s": (None, [vp, i32, u32, u32, u32, vp, u32, u32, u32]),
    "cuMpSGEMM_exp_stats_stage_c": (None, [vp, i32, u32, u32, u32, vp, u32, u32, u32]),
    "cuMpSGEMM_exp_stats_decide": (None, [vp, i32, u32]),
    "cuMpSGEMM_exp_stats_export": (None, [vp, u32, vp]),
    "cuMpSGEMM_exp_stats_import": (None, [vp, u32, vp]),
    "cuMpSGEMM_sgemm_strided_batch_with_stats": (i32, _GEMM_SB_ARGS + [u32, u32]),
    "cuMpSGEMM_cgemm_strided_batch_with_stats": (i32, _GEMM_SB_ARGS + [u32, u32]),
    "cuMpSGEMM_sgemm_static_scratch": (i32, [vp] + _GEMM_ARGS[1:]),
    "cuMpSGEMM_sgemm_Mx2x2": (i32, _TINY_ARGS),
    "cuMpSGEMM_cgemm_Mx2x2": (i32, _TINY_ARGS),
    "cuMpSGEMM_sgemm_2xNx2": (i32, _TINY_ARGS),
    "cuMpSGEMM_cgemm_2xNx2": (i32, _TINY_ARGS),
    # intercepted cuBLAS symbols (prototypes of cublas_api.h)
    "cublasSgemm_v2": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp, vp, i32]),
    "cublasCgemm_v2": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp, vp, i32]),
    "cublasSgemmStridedBatched": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, C.c_longlong,
                                        vp, i32, C.c_longlong, vp, vp, i32, C.c_longlong, i32]),
    "cublasCgemmStridedBatched": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, C.c_longlong,
                                        vp, i32, C.c_longlong, vp, vp, i32, C.c_longlong, i32]),
    "cublasGemmEx": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, i32, i32, vp, vp,
                           i32, i32, i32, i32]),
    "cublasSgemmBatched": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp, vp, i32, i32]),
    "cublasCgemmBatched": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp, vp, i32, i32]),
    "cublasGemmBatchedEx": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, i32, i32, vp,
                                  vp, i32, i32, i32, i32, i32]),
    "cublasSgemm_v2_64": (i32, [vp, i32, i32] + [C.c_int64] * 3 + [vp, vp, C.c_int64, vp, C.c_int64,
                                                              vp, vp, C.c_int64]),
    "cublasCgemm_v2_64": (i32, [vp, i32, i32] + [C.c_int64] * 3 + [vp, vp, C.c_int64, vp, C.c_int64,
                                                              vp, vp, C.c_int64]),
    "cublasSgemmStridedBatched_64": (i32, [vp, i32, i32] + [C.c_int64] * 3 +
                                     [vp, vp, C.c_int64, C.c_longlong, vp, C.c_int64, C.c_longlong,
                                      vp, vp, C.c_int64, C.c_longlong, C.c_int64]),
    "cublasCgemmStridedBatched_64": (i32, [vp, i32, i32] + [C.c_int64] * 3 +
                                     [vp, vp, C.c_int64, C.c_longlong, vp, C.c_int64, C.c_longlong,
                                      vp, vp, C.c_int64, C.c_longlong, C.c_int64]),
    "cublasGemmEx_64": (i32, [vp, i32, i32] + [C.c_int64] * 3 +
                        [vp, vp, i32, C.c_int64, vp, i32, C.c_int64, vp, vp, i32, C.c_int64, i32,
                         i32]),
    "cublasGemmStridedBatchedEx_64": (i32, [vp, i32, i32] + [C.c_int64] * 3 +
                                      [vp, vp, i32, C.c_int64, C.c_longlong, vp, i32, C.c_int64,
                                       C.c_longlong, vp, vp, i32, C.c_int64, C.c_longlong,
                                       C.c_int64, i32, i32]),
    "cublasGemmStridedBatchedEx": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, i32, i32,
                                         C.c_longlong, vp, i32, i32, C.c_longlong, vp, vp, i32,
                                         i32, C.c_longlong, i32, i32, i32]),
}


def load(build_if_missing: bool = True):
    """Return the loaded library with prototypes applied (cached)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path: Path = _build.library_path()
    if not path.exists():
        if not build_if_missing:
            raise RuntimeError(f"{path} is missing; run python -m cumpsgemm_b200.build")
        _build.build()
    lib = C.CDLL(str(path), mode=C.RTLD_LOCAL)
    for name, (restype, argtypes) in PROTOTYPES.items():
        _proto(lib, name, restype, argtypes)
    _LIB = lib
    return lib
