"""The Python control module (counterpart of the reference's pybind11 module
python/src/main.cpp) against the library's mode-selection chain; no GPU needed."""
import os

import pytest


def test_python_control_module_drives_mode_selection(clib):
    import cumpsgemm_b200.hijack_control as chc

    sel = clib.cuMpSGEMM_get_compute_mode_internal
    assert chc.is_library_loaded() is False          # not preloaded in the test process
    os.environ["CUMPSGEMM_COMPUTE_MODE"] = "FP16TCEC"
    try:
        assert sel(b"cublasSgemm_v2", None, 0, 0, 2048, 2048, 2048) == chc.CUMPSGEMM_FP16TCEC
        calls = []
        chc.set_control_function(lambda op_a, op_b, m, n, k: calls.append((m, n, k)) or chc.CUMPSGEMM_AUTO)
        assert sel(b"cublasSgemm_v2", None, 0, 1, 7, 8, 9) == chc.CUMPSGEMM_AUTO
        assert calls == [(7, 8, 9)]
        chc.set_compute_mode(chc.CUMPSGEMM_TF32TCEC)
        assert sel(b"cublasSgemm_v2", None, 0, 0, 7, 8, 9) == chc.CUMPSGEMM_TF32TCEC
        with pytest.raises(RuntimeError):
            chc.set_compute_mode(12)
        chc.unset_compute_mode()
        chc.unset_control_function()
        assert sel(b"cublasSgemm_v2", None, 0, 0, 2048, 2048, 2048) == chc.CUMPSGEMM_FP16TCEC
        chc.set_last_called_function_str("cublasSgemm_v2,N,N,1,2,3,1,FP16TCEC")
        assert chc.get_last_called_function_str() == "cublasSgemm_v2,N,N,1,2,3,1,FP16TCEC"
        chc.clear_last_called_function_str()
        assert chc.get_last_called_function_str() == ""
        chc.enable_custom_gemm_Mx2x2()
        chc.disable_custom_gemm_Mx2x2()
    finally:
        os.environ.pop("CUMPSGEMM_COMPUTE_MODE", None)
        chc.unset_control_function()
        chc.unset_compute_mode()
