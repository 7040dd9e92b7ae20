"""Generates the golden fixtures in this folder from the parts of the reference that compile
with plain g++ (see oracle/Makefile, target `ref`).  Run where the reference tree is mounted
(the REF variable of oracle/Makefile):

    make -C oracle ref && python tests/golden/make_golden.py

Outputs (committed):
  rule_golden.json : default rule, (env value, m, n, k) -> mode, from the reference's
                     src/default_cumpsgemm_rule.cu compiled as oracle/_ref/libcumpsgemm_rule_ref.so.
                     The unset-variable case is left out: the reference dereferences a null
                     pointer there.
  flag_golden.json : flag-word helpers, from src/dynamic_launch_utils.hpp compiled as
                     oracle/_ref/libflag_utils_ref.so.
"""
import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE.parent.parent / "oracle" / "_ref"

ENV_VALUES = ["FP16TCEC", "TF32TCEC", "FP16TC", "TF32TC", "CUBLAS_TF32TC", "CUBLAS_FP16TC",
              "CUBLAS_SIMT", "CUBLAS", "DRY_RUN", "AUTO", "FP16TCEC_SCALING", "FP32_SIMT", "bogus"]
SHAPES = [(2048, 2048, 2048), (1024, 4096, 4096), (4096, 1024, 4096), (4096, 4096, 1024),
          (1025, 1025, 1025), (16384, 16384, 16384), (1, 1, 1)]


def rule_case(env_value, m, n, k):
    # one subprocess per environment value: getenv is read inside the rule
    code = (
        "import ctypes as C, sys\n"
        f"lib = C.CDLL({str(REF / 'libcumpsgemm_rule_ref.so')!r})\n"
        "f = lib.cuMpSGEMM_get_compute_mode\n"
        "f.restype = C.c_int\n"
        "f.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_uint, C.c_uint]\n"
        f"print(f(b'cublasSgemm_v2', None, 0, 0, {m}, {n}, {k}))\n")
    env = dict(os.environ, CUMPSGEMM_COMPUTE_MODE=env_value, CUMPSGEMM_ERROR_LOG="0")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         check=True).stdout.strip().splitlines()[-1]
    return int(out)


def main():
    rules = []
    for ev in ENV_VALUES:
        for (m, n, k) in SHAPES:
            rules.append({"env": ev, "m": m, "n": n, "k": k, "mode": rule_case(ev, m, n, k)})
    (HERE / "rule_golden.json").write_text(json.dumps(rules, indent=0))

    lib = C.CDLL(str(REF / "libflag_utils_ref.so"))
    flags = []
    for flag in [0, 1, 2, 9, 11, 0x20, 0x40, 0x60, 0x61, 0x62, 0x7f, 0x1f]:
        entry = {"flag": flag,
                 "get_gemm": lib.ref_get_gemm_flag(flag),
                 "get_scale_A": lib.ref_get_scale_A_flag(flag),
                 "get_scale_B": lib.ref_get_scale_B_flag(flag),
                 "set_gemm_2": lib.ref_set_gemm_flag(flag, 2),
                 "set_gemm_1": lib.ref_set_gemm_flag(flag, 1),
                 "set_A_on": lib.ref_set_scale_A_flag(flag, 1),
                 "set_A_off": lib.ref_set_scale_A_flag(flag, 0),
                 "set_B_on": lib.ref_set_scale_B_flag(flag, 1),
                 "set_B_off": lib.ref_set_scale_B_flag(flag, 0)}
        flags.append(entry)
    (HERE / "flag_golden.json").write_text(json.dumps(flags, indent=0))
    print("wrote", len(rules), "rule cases and", len(flags), "flag cases")


if __name__ == "__main__":
    main()
