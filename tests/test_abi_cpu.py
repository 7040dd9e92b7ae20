"""The C-ABI library loads without a GPU and exports every symbol the headers declare."""
import json
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = Path(__file__).resolve().parent / "golden"


def _declared_symbols():
    names = set()
    for hdr in ("cumpsgemm.h", "cumpsgemm_ext.h"):
        text = (ROOT / "include" / "cumpsgemm" / hdr).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(cuMpSGEMM_\w+)\s*\(", text))
    names -= {"cuMpSGEMM_control_function_c_t"}
    return names


def test_every_declared_symbol_is_exported(clib):
    declared = _declared_symbols()
    assert len(declared) > 60
    missing = [n for n in sorted(declared) if not hasattr(clib, n)]
    assert not missing, missing
    for n in ("cublasSgemm_v2", "cublasCgemm_v2", "cublasSgemmStridedBatched",
              "cublasCgemmStridedBatched", "cublasGemmEx", "cublasGemmStridedBatchedEx",
              "cublasSgemmBatched", "cublasCgemmBatched", "cublasGemmBatchedEx",
              "cublasSgemm_v2_64", "cublasCgemm_v2_64", "cublasSgemmStridedBatched_64",
              "cublasCgemmStridedBatched_64", "cublasGemmEx_64", "cublasGemmStridedBatchedEx_64"):
        assert hasattr(clib, n), n


def test_prototype_table_covers_the_headers():
    from cumpsgemm_b200 import _lib

    assert _declared_symbols() <= set(_lib.PROTOTYPES)


def test_no_link_time_dependency_on_cublas_or_torch():
    from cumpsgemm_b200 import build

    out = subprocess.run(["readelf", "-d", str(build.library_path())], capture_output=True,
                         text=True).stdout
    needed = re.findall(r"\(NEEDED\).*\[(.*?)\]", out)
    assert not any("cublas" in n or "torch" in n or "cudart" in n for n in needed), needed


def test_mode_strings(clib):
    names = ["CUBLAS", "FP16TCEC", "TF32TCEC", "FP16TC", "TF32TC", "CUBLAS_SIMT", "CUBLAS_FP16TC",
             "CUBLAS_TF32TC", "DRY_RUN", "AUTO", "UNDEFINED", "FP16TCEC_SCALING", "FP32_SIMT"]
    for i, n in enumerate(names):
        assert clib.cuMpSGEMM_get_compute_mode_string(i) == n.encode()
    assert clib.cuMpSGEMM_get_compute_mode_string(99) == b"Unknown"
    from cumpsgemm_b200 import api

    assert [m.name for m in api.ComputeMode] == names


def _rule_in_subprocess(env_value, shapes, lib_path):
    code = (
        "import ctypes as C, json, sys\n"
        f"lib = C.CDLL({str(lib_path)!r})\n"
        "f = lib.cuMpSGEMM_get_compute_mode\n"
        "f.restype = C.c_int\n"
        "f.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_uint, C.c_uint]\n"
        f"print(json.dumps([f(b'cublasSgemm_v2', None, 0, 0, m, n, k) for (m, n, k) in {shapes!r}]))\n")
    env = dict(os.environ, CUMPSGEMM_ERROR_LOG="0")
    if env_value is None:
        env.pop("CUMPSGEMM_COMPUTE_MODE", None)
    else:
        env["CUMPSGEMM_COMPUTE_MODE"] = env_value
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         check=True).stdout.strip().splitlines()[-1]
    return json.loads(out)


@pytest.mark.parametrize("which", ["libcumpsgemm.so", "libcumpsgemm_rule.so"])
def test_default_rule_against_reference_golden(which):
    """Golden vectors come from the reference's src/default_cumpsgemm_rule.cu compiled with g++
    (tests/golden/make_golden.py)."""
    from cumpsgemm_b200 import build

    lib_path = build.library_path().parent / which
    golden = json.loads((GOLDEN / "rule_golden.json").read_text())
    by_env = {}
    for g in golden:
        by_env.setdefault(g["env"], []).append(g)
    for env_value, cases in by_env.items():
        shapes = [(c["m"], c["n"], c["k"]) for c in cases]
        got = _rule_in_subprocess(env_value, shapes, lib_path)
        assert got == [c["mode"] for c in cases], env_value
    # unset variable: the reference crashes on a null string; this build selects CUBLAS
    assert _rule_in_subprocess(None, [(4096, 4096, 4096), (8, 8, 8)], lib_path) == [0, 5]


def test_mode_selection_chain(clib):
    """control function > rule library > built-in rule; static mode overrides all
    (reference: src/cumpsgemm_cublas.cu:198-220, 1193-1205)."""
    import ctypes as C

    sel = clib.cuMpSGEMM_get_compute_mode_internal
    os.environ["CUMPSGEMM_COMPUTE_MODE"] = "TF32TCEC"
    try:
        assert sel(b"cublasSgemm_v2", None, 0, 0, 4096, 4096, 4096) == 2
        assert sel(b"cublasSgemm_v2", None, 0, 0, 512, 4096, 4096) == 5
        CB = C.CFUNCTYPE(C.c_int, C.c_int, C.c_int, C.c_uint, C.c_uint, C.c_uint)
        seen = []

        def pick(op_a, op_b, m, n, k):
            seen.append((op_a, op_b, m, n, k))
            return 11

        cb = CB(pick)
        clib.cuMpSGEMM_hijack_set_control_function(C.cast(cb, C.c_void_p))
        assert sel(b"cublasSgemm_v2", None, 1, 0, 10, 20, 30) == 11
        assert seen == [(1, 0, 10, 20, 30)]
        assert clib.cuMpSGEMM_hijack_set_compute_mode(1) == 0
        assert sel(b"cublasSgemm_v2", None, 0, 0, 10, 20, 30) == 1      # static beats the callback
        assert clib.cuMpSGEMM_hijack_set_compute_mode(12) == 1          # FP32_SIMT is rejected
        clib.cuMpSGEMM_hijack_unset_compute_mode()
        assert sel(b"cublasSgemm_v2", None, 0, 0, 10, 20, 30) == 11
        clib.cuMpSGEMM_hijack_set_control_function(None)
        assert sel(b"cublasSgemm_v2", None, 0, 0, 4096, 4096, 4096) == 2
    finally:
        os.environ.pop("CUMPSGEMM_COMPUTE_MODE", None)
        clib.cuMpSGEMM_hijack_set_control_function(None)
        clib.cuMpSGEMM_hijack_unset_compute_mode()
    assert clib.cuMpSGEMM_hijack_is_library_loaded() == 1


def test_product_does_not_import_the_oracle():
    """The oracle is a checker: nothing under cumpsgemm_b200/ may reference it."""
    for p in (ROOT / "cumpsgemm_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".hpp", ".cpp", ".h") and p.is_file():
            assert "oracle" not in p.read_text(), p


def test_create_without_gpu_fails_loudly(clib):
    import ctypes as C

    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert clib.cuMpSGEMM_create(C.byref(h)) != 0
    from cumpsgemm_b200 import api

    with pytest.raises(api.CuMpSGEMMError):
        api.Handle()


def test_pair_tail_plan_host_logic():
    """How the CTA-pair kernel cuts the last, partly filled wave of tiles into K slices (a
    host-only query of the library, no GPU): every tile is covered exactly once, the slices
    of the cut tiles fit the clusters of one wave, a slice keeps at least 1024 k values, and
    nothing is cut when the last wave is more than half full or K is short."""
    import ctypes as C

    from cumpsgemm_b200 import _lib

    lib = _lib.load()

    def plan(tiles, clusters, k, tf32=0):
        out = [C.c_uint32() for _ in range(4)]
        assert lib.cuMpSGEMM_plan_pair_tail(tiles, clusters, k, tf32, *map(C.byref, out)) == 0
        return tuple(o.value for o in out)

    # m=n=k=4096 on 74 clusters: 256 tiles = 3 full waves + 34 tiles, cut in two
    assert plan(256, 74, 4096) == (222, 2, 2048, 222 + 34 * 2)
    assert plan(256, 74, 4096, 1) == (222, 2, 2048, 290)
    # m=n=k=16384: 4096 tiles, 26 in the last wave
    assert plan(4096, 74, 16384) == (4070, 2, 8192, 4070 + 52)
    # last wave more than half full, exactly full, or K too short for two slices: nothing is cut
    assert plan(1024, 74, 8192) == (1024, 1, 8192, 1024)
    assert plan(148, 74, 8192) == (148, 1, 8192, 148)
    assert plan(256, 74, 1024) == (256, 1, 1024, 256)
    # four tiles and a long K: eight slices at most
    sb, sl, sk, wi = plan(4, 74, 8192 + 64)
    assert (sb, sl, wi) == (0, 8, 32) and sk * sl >= 8192 + 64 and sk * (sl - 1) < 8192 + 64
    for tiles in (1, 5, 37, 38, 75, 100, 111, 300, 1000):
        for clusters in (1, 2, 66, 74):
            for k in (64, 1024, 2048, 3072, 65536):
                for tf32 in (0, 1):
                    sb, sl, sk, wi = plan(tiles, clusters, k, tf32)
                    rem = tiles - sb
                    assert wi == sb + rem * sl and 1 <= sl <= 8
                    if sl > 1:
                        assert sb % clusters == 0 and rem * sl <= clusters and 2 * rem <= clusters
                        assert sk >= 1024 and sk * sl >= k and sk * (sl - 1) < k
                    else:
                        assert sb == tiles and sk == k
    assert lib.cuMpSGEMM_plan_pair_tail(0, 74, 4096, 0, None, None, None, None) == 1
