"""In-tree build of the native libraries with nvcc for sm_100a.

Produces, next to this file under ``lib/``:

* ``libcumpsgemm.so``        – kernels, C ABI, C++ API and the cuBLAS
  interception layer (the ``LD_PRELOAD`` target);
* ``libcumpsgemm_static.a``  – the same objects as an archive;
* ``libcumpsgemm_rule.so``   – the default ``cuMpSGEMM_get_compute_mode`` rule.

Target names follow the reference's ``CMakeLists.txt:47-77``.  Run as
``python -m cumpsgemm_b200.build`` (``--force`` to rebuild everything).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
INCLUDE = REPO_ROOT / "include"

CUDA_SOURCES = [
    "handle.cu",
    "exp_stats.cu",
    "dynamic_scaling.cu",
    "split_kernels.cu",
    "tcec_gemm.cu",
    "tcec_gemm_pair.cu",
    "tcec_gemm_fused.cu",
    "gemm_api.cu",
    "ext_api.cu",
    "static_scratch_gemm.cu",
    "tiny_gemm.cu",
]
CPP_SOURCES = ["cublas_shim.cpp", "default_rule.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the cuMpSGEMM kernels cannot be built")


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps if d.exists())


def _compile(src: Path, obj: Path, log_dir: Path) -> None:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    (log_dir / (src.name + ".log")).write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile everything that is out of date; returns the path of libcumpsgemm.so."""
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.rglob("*.h*"))
    sources = [CSRC / s for s in CUDA_SOURCES + CPP_SOURCES if (CSRC / s).exists()]
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ_DIR / (src.name + ".o")
        objs.append(obj)
        if force or not _newer(obj, [src, *headers]):
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda j: _compile(j[0], j[1], OBJ_DIR), jobs))
        if verbose:
            print(f"compiled {len(jobs)} translation unit(s)")

    lib = LIB_DIR / "libcumpsgemm.so"
    if force or jobs or not lib.exists():
        subprocess.run(
            [_nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-cudart", "static", "-ldl",
             "-lpthread"],
            check=True,
        )
    static = LIB_DIR / "libcumpsgemm_static.a"
    if force or jobs or not static.exists():
        if static.exists():
            static.unlink()
        subprocess.run(["ar", "rcs", str(static), *map(str, objs)], check=True)
    rule = LIB_DIR / "libcumpsgemm_rule.so"
    rule_obj = OBJ_DIR / "default_rule.cpp.o"
    if force or jobs or not rule.exists():
        subprocess.run(["g++", "-shared", "-fPIC", "-o", str(rule), str(rule_obj)], check=True)
    return lib


def library_path() -> Path:
    return LIB_DIR / "libcumpsgemm.so"


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(path)
