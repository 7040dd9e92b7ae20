"""The cuBLAS interception layer: direct calls of the exported cuBLAS symbols, the log grammar,
and an unmodified cuBLAS application under LD_PRELOAD."""
import ctypes as C
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
LOG_RE = re.compile(r"^\[cuMpSGEMM LOG\] (\w+) op=\(([NTC]), ([NTC])\), shape=\((\d+), (\d+), (\d+)\), "
                    r"(?:batch=(\d+), )?mode=(\w+)\[(dynamic|static)\]\[exp_stats:([01])\]$", re.M)


def _setup():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cumpsgemm_b200 import _lib

    return torch, _lib.load()


def test_intercepted_symbols_called_directly(oracle):
    torch, lib = _setup()
    blas = torch.cuda.current_blas_handle()
    m, n, k = 300, 260, 280
    a, b = oracle.gen_uniform(1, m * k), oracle.gen_uniform(2, k * n)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    truth = oracle.gemm_f64(0, 0, m, n, k, 1.0, a, m, b, k, 0.0, None, m)
    alpha, beta = C.c_float(1.0), C.c_float(0.0)
    try:
        for mode, thr in ((1, True), (2, True), (11, True), (9, True), (5, True)):
            assert lib.cuMpSGEMM_hijack_set_compute_mode(mode) == 0
            dc = torch.zeros(m * n, device="cuda")
            st = lib.cublasSgemm_v2(blas, 0, 0, m, n, k, C.byref(alpha), da.data_ptr(), m,
                                    db.data_ptr(), k, C.byref(beta), dc.data_ptr(), m)
            assert st == 0
            torch.cuda.synchronize()
            assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(thr, k), mode
            buf = C.create_string_buffer(256)
            lib.cuMpSGEMM_hijack_get_last_called_function_str(buf, 256)
            names = ["CUBLAS", "FP16TCEC", "TF32TCEC", "FP16TC", "TF32TC", "CUBLAS_SIMT",
                     "CUBLAS_FP16TC", "CUBLAS_TF32TC", "DRY_RUN", "AUTO", "UNDEFINED",
                     "FP16TCEC_SCALING"]
            assert buf.value.decode() == f"cublasSgemm_v2,N,N,{m},{n},{k},1,{names[mode]}"
        # DRY_RUN: nothing computed
        lib.cuMpSGEMM_hijack_set_compute_mode(8)
        dc = torch.full((m * n,), 3.0, device="cuda")
        assert lib.cublasSgemm_v2(blas, 0, 0, m, n, k, C.byref(alpha), da.data_ptr(), m,
                                  db.data_ptr(), k, C.byref(beta), dc.data_ptr(), m) == 0
        assert (dc == 3.0).all()
        # zero sizes are rejected before anything else (reference: cumpsgemm_cublas.cu:233-235)
        assert lib.cublasSgemm_v2(blas, 0, 0, 0, n, k, C.byref(alpha), da.data_ptr(), m,
                                  db.data_ptr(), k, C.byref(beta), dc.data_ptr(), m) == 7
        # GemmEx with FP32 types is intercepted, other types are forwarded
        lib.cuMpSGEMM_hijack_set_compute_mode(1)
        dc = torch.zeros(m * n, device="cuda")
        CUDA_R_32F, CUDA_R_16F, COMPUTE_32F = 0, 2, 68
        st = lib.cublasGemmEx(blas, 0, 0, m, n, k, C.byref(alpha), da.data_ptr(), CUDA_R_32F, m,
                              db.data_ptr(), CUDA_R_32F, k, C.byref(beta), dc.data_ptr(),
                              CUDA_R_32F, m, COMPUTE_32F, -1)
        assert st == 0
        torch.cuda.synchronize()
        assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
        lib.cuMpSGEMM_hijack_clear_last_called_function_str()
        ha, hb = da.half(), db.half()
        hc = torch.zeros(m * n, device="cuda", dtype=torch.float16)
        st = lib.cublasGemmEx(blas, 0, 0, m, n, k, C.byref(alpha), ha.data_ptr(), CUDA_R_16F, m,
                              hb.data_ptr(), CUDA_R_16F, k, C.byref(beta), hc.data_ptr(),
                              CUDA_R_16F, m, COMPUTE_32F, -1)
        assert st == 0
        buf = C.create_string_buffer(64)
        assert lib.cuMpSGEMM_hijack_get_last_called_function_str(buf, 64) == 0   # not intercepted
        torch.cuda.synchronize()
        assert oracle.residual(truth, hc.float().cpu().numpy(), m) < 1e-2
        # strided batch through the shim, complex
        bsz, s = 3, 64
        za = oracle.gen_unit_frobenius_complex(1, bsz, s, s)
        zb = oracle.gen_unit_frobenius_complex(2, bsz, s, s)
        dza, dzb = torch.from_numpy(za).cuda(), torch.from_numpy(zb).cuda()
        dzc = torch.zeros(bsz * s * s, dtype=torch.complex64, device="cuda")
        calpha, cbeta = (C.c_float * 2)(1.0, 0.0), (C.c_float * 2)(0.0, 0.0)
        lib.cuMpSGEMM_hijack_set_compute_mode(11)
        st = lib.cublasCgemmStridedBatched(blas, 0, 0, s, s, s, calpha, dza.data_ptr(), s, s * s,
                                           dzb.data_ptr(), s, s * s, cbeta, dzc.data_ptr(), s,
                                           s * s, bsz)
        assert st == 0
        torch.cuda.synchronize()
        res = dzc.cpu().numpy()
        for i in range(bsz):
            t = oracle.gemm_f64(0, 0, s, s, s, 1.0, za[i * s * s:], s, zb[i * s * s:], s, 0.0, None, s)
            assert oracle.residual(t, res[i * s * s:(i + 1) * s * s], s) < oracle.error_threshold(True, s)
    finally:
        lib.cuMpSGEMM_hijack_unset_compute_mode()


def _client(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not available to build the cuBLAS client")
    out = tmp_path_factory.mktemp("client") / "cublas_client"
    r = subprocess.run([nvcc, "-O2", "-o", str(out), str(ROOT / "tests/clients/cublas_client.cpp"),
                        "-lcublas"], capture_output=True, text=True)
    if r.returncode != 0:
        pytest.skip("cannot build the cuBLAS client: " + r.stderr[-300:])
    return out


@pytest.fixture(scope="module")
def client(tmp_path_factory):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return _client(tmp_path_factory)


def _run_client(client, args, preload, env_extra):
    from cumpsgemm_b200 import build

    env = dict(os.environ)
    env.pop("CUMPSGEMM_COMPUTE_MODE", None)
    env.update(env_extra)
    lib_dir = str(build.library_path().parent)
    env["LD_LIBRARY_PATH"] = lib_dir + ":/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    if preload:
        env["LD_PRELOAD"] = str(build.library_path())
    r = subprocess.run([str(client), *map(str, args)], env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    res = float(re.search(r"RESIDUAL (\S+)", r.stdout).group(1))
    st = int(re.search(r"STATUS (\d+)", r.stdout).group(1))
    return res, st, r.stdout


@pytest.mark.parametrize("kind", ["s", "c", "sb", "ex"])
def test_unmodified_cublas_application_under_ld_preload(client, kind):
    """LD_PRELOAD end to end, mode chosen by libcumpsgemm_rule.so from CUMPSGEMM_COMPUTE_MODE."""
    m, n, k = (1100, 1060, 1030) if kind != "c" else (1040, 1030, 1025)
    res, st, out = _run_client(client, [kind, m, n, k], True,
                               {"CUMPSGEMM_COMPUTE_MODE": "FP16TCEC", "CUMPSGEMM_INFO": "1"})
    assert st == 0 and res < 2.0 ** -23 * np.sqrt(k)
    logs = LOG_RE.findall(out)
    assert logs, out
    func, opa, opb, lm, ln, lk, batch, mode, how, es = logs[-1]
    expect_func = {"s": "cublasSgemm_v2", "c": "cublasCgemm_v2", "sb": "cublasSgemmStridedBatched",
                   "ex": "cublasGemmEx"}[kind]
    assert (func, opa, opb, int(lm), int(ln), int(lk), mode, how, es) == \
        (expect_func, "N", "N", m, n, k, "FP16TCEC", "dynamic", "0")
    assert (batch == "3") == (kind == "sb")
    assert "[cuMpSGEMM LOG] Initialize cuMpSGEMM handle..." in out
    # small problems go to cuBLAS SIMT by the default rule; pass-through must still be correct
    res, st, out = _run_client(client, [kind, 200, 180, 160], True,
                               {"CUMPSGEMM_COMPUTE_MODE": "FP16TCEC", "CUMPSGEMM_INFO": "1"})
    assert st == 0 and res < 1e-5
    assert LOG_RE.findall(out)[-1][7] == "CUBLAS_SIMT"


def test_auto_mode_log_line_under_ld_preload(client):
    res, st, out = _run_client(client, ["s", 1100, 1060, 1030], True,
                               {"CUMPSGEMM_COMPUTE_MODE": "AUTO", "CUMPSGEMM_INFO": "1"})
    assert st == 0 and res < 2.0 ** -23 * np.sqrt(1030)
    assert re.search(r"\[cuMpSGEMM LOG\] AUTO\[ignore<\S+, uf<\S+, tolerance=\S+\]: GEMM_MODE=\w+, "
                     r"loss_A=\d+/\d+\(\S+\), scale_A=[01], loss_B=\d+/\d+\(\S+\), scale_B=[01]", out)


def test_client_without_preload_is_plain_cublas(client):
    res, st, out = _run_client(client, ["s", 1100, 1060, 1030], False, {"CUMPSGEMM_INFO": "1"})
    assert st == 0 and "[cuMpSGEMM LOG]" not in out


def test_64bit_entry_points(oracle):
    """cuBLAS 12's 64-bit integer interface (cublasSgemm_v2_64, ...) is intercepted as well, and
    the pass-through modes forward to the real cublasGemmEx_64."""
    torch, lib = _setup()
    blas = torch.cuda.current_blas_handle()
    m, n, k = 260, 300, 200
    a, b = oracle.gen_uniform(1, m * k), oracle.gen_uniform(2, k * n)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    truth = oracle.gemm_f64(0, 0, m, n, k, 1.0, a, m, b, k, 0.0, None, m)
    alpha, beta = C.c_float(1.0), C.c_float(0.0)
    try:
        for mode, thr in ((1, oracle.error_threshold(True, k)), (5, 1e-5)):
            lib.cuMpSGEMM_hijack_set_compute_mode(mode)
            dc = torch.zeros(m * n, device="cuda")
            assert lib.cublasSgemm_v2_64(blas, 0, 0, m, n, k, C.byref(alpha), da.data_ptr(), m,
                                         db.data_ptr(), k, C.byref(beta), dc.data_ptr(), m) == 0
            torch.cuda.synchronize()
            assert oracle.residual(truth, dc.cpu().numpy(), m) < thr
            buf = C.create_string_buffer(128)
            lib.cuMpSGEMM_hijack_get_last_called_function_str(buf, 128)
            assert buf.value.decode().startswith(f"cublasSgemm_v2_64,N,N,{m},{n},{k},1,")
        lib.cuMpSGEMM_hijack_set_compute_mode(2)
        dc = torch.zeros(m * n, device="cuda")
        assert lib.cublasGemmEx_64(blas, 0, 0, m, n, k, C.byref(alpha), da.data_ptr(), 0, m,
                                   db.data_ptr(), 0, k, C.byref(beta), dc.data_ptr(), 0, m, 68,
                                   -1) == 0
        torch.cuda.synchronize()
        assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
    finally:
        lib.cuMpSGEMM_hijack_unset_compute_mode()


def test_pointer_array_batched_entry_points(oracle):
    """cublasSgemmBatched / cublasCgemmBatched / cublasGemmBatchedEx (FP32): matrices scattered
    in memory, addressed through device arrays of pointers."""
    torch, lib = _setup()
    blas = torch.cuda.current_blas_handle()
    batch, m, n, k = 5, 70, 130, 90
    alpha, beta = C.c_float(2.0), C.c_float(0.5)
    a = [oracle.gen_uniform(10 + i, m * k) for i in range(batch)]
    b = [oracle.gen_uniform(20 + i, k * n) for i in range(batch)]
    c0 = [oracle.gen_uniform(30 + i, m * n) for i in range(batch)]
    da = [torch.from_numpy(x).cuda() for x in a]
    db = [torch.from_numpy(x).cuda() for x in b]

    def ptrs(ts):
        return torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device="cuda")

    try:
        for mode, thr in ((1, oracle.error_threshold(True, k)), (2, oracle.error_threshold(True, k)),
                          (5, 1e-5), (9, 1e-5)):
            lib.cuMpSGEMM_hijack_set_compute_mode(mode)
            dc = [torch.from_numpy(x.copy()).cuda() for x in c0]
            pa, pb, pc = ptrs(da), ptrs(db), ptrs(dc)
            st = lib.cublasSgemmBatched(blas, 0, 0, m, n, k, C.byref(alpha), pa.data_ptr(), m,
                                        pb.data_ptr(), k, C.byref(beta), pc.data_ptr(), m, batch)
            assert st == 0
            torch.cuda.synchronize()
            for i in range(batch):
                truth = oracle.gemm_f64(0, 0, m, n, k, 2.0, a[i], m, b[i], k, 0.5, c0[i], m)
                assert oracle.residual(truth, dc[i].cpu().numpy(), m) < thr, (mode, i)
        # Ex form, op (T, N), alpha/beta unchanged
        lib.cuMpSGEMM_hijack_set_compute_mode(1)
        at = [torch.from_numpy(np.ascontiguousarray(x.reshape((m, k), order="F").T).ravel(order="F").copy()).cuda()
              for x in a]
        dc = [torch.from_numpy(x.copy()).cuda() for x in c0]
        pa, pb, pc = ptrs(at), ptrs(db), ptrs(dc)
        st = lib.cublasGemmBatchedEx(blas, 1, 0, m, n, k, C.byref(alpha), pa.data_ptr(), 0, k,
                                     pb.data_ptr(), 0, k, C.byref(beta), pc.data_ptr(), 0, m, batch,
                                     68, -1)
        assert st == 0
        torch.cuda.synchronize()
        for i in range(batch):
            truth = oracle.gemm_f64(0, 0, m, n, k, 2.0, a[i], m, b[i], k, 0.5, c0[i], m)
            assert oracle.residual(truth, dc[i].cpu().numpy(), m) < oracle.error_threshold(True, k)
        # complex
        za = [(oracle.gen_uniform(40 + i, m * k) + 1j * oracle.gen_uniform(50 + i, m * k)).astype(np.complex64)
              for i in range(batch)]
        zb = [(oracle.gen_uniform(60 + i, k * n) + 1j * oracle.gen_uniform(70 + i, k * n)).astype(np.complex64)
              for i in range(batch)]
        dza = [torch.from_numpy(x).cuda() for x in za]
        dzb = [torch.from_numpy(x).cuda() for x in zb]
        dzc = [torch.zeros(m * n, dtype=torch.complex64, device="cuda") for _ in range(batch)]
        calpha, cbeta = (C.c_float * 2)(1.0, -1.0), (C.c_float * 2)(0.0, 0.0)
        pza, pzb, pzc = ptrs(dza), ptrs(dzb), ptrs(dzc)   # keep the pointer arrays alive
        st = lib.cublasCgemmBatched(blas, 0, 0, m, n, k, calpha, pza.data_ptr(), m,
                                    pzb.data_ptr(), k, cbeta, pzc.data_ptr(), m, batch)
        assert st == 0
        torch.cuda.synchronize()
        for i in range(batch):
            truth = oracle.gemm_f64(0, 0, m, n, k, 1 - 1j, za[i], m, zb[i], k, 0.0, None, m)
            assert oracle.residual(truth, dzc[i].cpu().numpy(), m) < oracle.error_threshold(True, k)
        buf = C.create_string_buffer(128)
        lib.cuMpSGEMM_hijack_get_last_called_function_str(buf, 128)
        assert buf.value.decode() == f"cublasCgemmBatched,N,N,{m},{n},{k},{batch},FP16TCEC"
    finally:
        lib.cuMpSGEMM_hijack_unset_compute_mode()


TORCH_CLIENT = r"""
import torch
torch.backends.cuda.matmul.allow_tf32 = False
g = torch.Generator(device="cuda"); g.manual_seed(5)
a = torch.rand(1536, 1280, device="cuda", generator=g) * 2 - 1
b = torch.rand(1280, 1152, device="cuda", generator=g) * 2 - 1
c = a @ b                                   # 2-D FP32 matmul -> cuBLAS SGEMM
z = torch.complex(a, a.flip(0)) @ torch.complex(b, b.flip(1))
a2, b2 = torch.stack([a, a.flip(0)]), torch.stack([b, b.flip(1)])   # every size above 1024:
bb = torch.bmm(a2, b2)                      # the default rule keeps smaller problems on cuBLAS
torch.cuda.synchronize()
def res(x, t): return float((x.double() - t).norm() / t.norm()) if not x.is_complex() else float((x.to(torch.complex128) - t).norm() / t.norm())
print("RES_S", res(c, a.double() @ b.double()))
print("RES_C", res(z, torch.complex(a, a.flip(0)).to(torch.complex128) @ torch.complex(b, b.flip(1)).to(torch.complex128)))
print("RES_B", res(bb, torch.bmm(a2.double(), b2.double())))
"""


def test_pytorch_under_ld_preload():
    """An unmodified PyTorch process: its FP32 / complex64 matmul and bmm reach cuBLAS through
    the interposed symbols and come back with the corrected kernels' accuracy."""
    _setup()
    from cumpsgemm_b200 import build

    env = dict(os.environ)
    env.update({"LD_PRELOAD": str(build.library_path()), "CUMPSGEMM_COMPUTE_MODE": "FP16TCEC",
                "CUMPSGEMM_INFO": "1"})
    r = subprocess.run([sys.executable, "-c", TORCH_CLIENT], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = r.stdout
    logs = LOG_RE.findall(out)
    funcs = {entry[0] for entry in logs if entry[7] == "FP16TCEC"}
    # which entry point PyTorch uses for each call is its own business; each of the three
    # calls must have been intercepted and computed in the requested mode
    assert len([entry for entry in logs if entry[7] == "FP16TCEC"]) >= 3, out[-3000:]
    assert funcs <= {"cublasSgemm_v2", "cublasCgemm_v2", "cublasGemmEx", "cublasSgemmStridedBatched",
                     "cublasCgemmStridedBatched", "cublasGemmStridedBatchedEx", "cublasSgemm_v2_64",
                     "cublasGemmEx_64", "cublasSgemmBatched", "cublasGemmBatchedEx"}, funcs
    for tag in ("RES_S", "RES_C", "RES_B"):
        val = float(re.search(tag + r" (\S+)", out).group(1))
        assert val < 2.0 ** -23 * np.sqrt(1280), (tag, val)


def test_two_streams_share_the_per_device_handle(oracle):
    """An application that runs GEMMs on two streams of one GPU: both reach the one handle the
    interception layer keeps per device, whose operand workspace and rings are shared.  The
    calls are interleaved with no host synchronisation in between; each stream's result must
    be the product of its own operands."""
    torch, lib = _setup()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(s1):
        blas1 = torch.cuda.current_blas_handle()
    with torch.cuda.stream(s2):
        blas2 = torch.cuda.current_blas_handle()
    shapes = ((1536, 1280, 2048), (640, 900, 1100))
    ops = []
    for i, (m, n, k) in enumerate(shapes):
        a, b = oracle.gen_uniform(40 + i, m * k), oracle.gen_uniform(50 + i, k * n)
        ops.append((m, n, k, a, b, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(),
                    torch.zeros(m * n, device="cuda")))
    torch.cuda.synchronize()
    alpha, beta = C.c_float(1.0), C.c_float(0.0)
    try:
        for mode in (1, 11):                         # FP16TCEC, FP16TCEC_SCALING
            assert lib.cuMpSGEMM_hijack_set_compute_mode(mode) == 0
            for (m, n, k, a, b, da, db, dc) in ops:
                dc.zero_()
            torch.cuda.synchronize()
            for _ in range(12):
                for blas, (m, n, k, a, b, da, db, dc) in zip((blas1, blas2), ops):
                    assert lib.cublasSgemm_v2(blas, 0, 0, m, n, k, C.byref(alpha), da.data_ptr(), m,
                                              db.data_ptr(), k, C.byref(beta), dc.data_ptr(), m) == 0
            torch.cuda.synchronize()
            for (m, n, k, a, b, da, db, dc) in ops:
                truth = oracle.gemm_f64(0, 0, m, n, k, 1.0, a, m, b, k, 0.0, None, m)
                assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
    finally:
        lib.cuMpSGEMM_hijack_unset_compute_mode()
