"""(m, 2, 2) and (2, n, 2) FP32 GEMMs: the device kernels against the CPU restatement, bit for
bit, and the interception layer's routing of such shapes (reference call sites:
src/cumpsgemm_cublas.cu:269-338 and :647-725)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

OPS = {"N": 0, "T": 1, "C": 2}


def _setup():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cumpsgemm_b200 import api

    return torch, api


def _shapes(long_is_m, op_a, op_b, length, pad):
    """Stored (rows, cols) of A, B, C with leading dimensions padded by `pad`."""
    a_rc = ((length, 2) if op_a == 0 else (2, length)) if long_is_m else (2, 2)
    b_rc = (2, 2) if long_is_m else ((2, length) if op_b == 0 else (length, 2))
    c_rc = (length, 2) if long_is_m else (2, length)
    return [(r, c, r + pad) for r, c in (a_rc, b_rc, c_rc)]


def _gen(oracle, seed, count, cplx):
    if not cplx:
        return oracle.gen_normal(seed, count)
    return (oracle.gen_normal(seed, count) + 1j * oracle.gen_normal(seed + 1000, count)).astype(
        np.complex64)


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("long_is_m", [True, False])
@pytest.mark.parametrize("op_a,op_b", [("N", "N"), ("T", "N"), ("N", "T"), ("C", "C")])
@pytest.mark.parametrize("length,batch,pad,beta", [(1, 1, 0, 0.0), (2, 3, 1, 0.5), (1024, 1, 0, 0.0),
                                                   (4096, 5, 3, -1.25), (1 << 18, 2, 0, 0.5)])
def test_matches_cpu_restatement_bitwise(oracle, cplx, long_is_m, op_a, op_b, length, batch, pad,
                                         beta):
    torch, api = _setup()
    if not cplx and "C" in (op_a, op_b):
        pytest.skip("conjugation only differs from transposition for complex data")
    oa, ob = OPS[op_a], OPS[op_b]
    (ar, ac, lda), (br, bc, ldb), (cr, cc, ldc) = _shapes(long_is_m, oa, ob, length, pad)
    sa, sb, sc = lda * ac + 7, ldb * bc, ldc * cc + 1
    a = _gen(oracle, 11, sa * batch, cplx)
    b = _gen(oracle, 12, max(sb * batch, 1), cplx)
    c0 = _gen(oracle, 13, sc * batch, cplx)
    alpha = (0.75 - 0.5j) if cplx else 0.75
    beta_v = (beta + 0.25j) if (cplx and beta != 0.0) else beta
    want = c0.copy()
    oracle.tiny_gemm_f32(long_is_m, oa, ob, length, alpha, a, lda, b, ldb, beta_v, want, ldc,
                         sa, sb, sc, batch)
    h = api.Handle()
    da, db, dc = (torch.from_numpy(x).cuda() for x in (a, b, c0))
    for _ in range(2):   # second call on fresh C: same bits
        dc.copy_(torch.from_numpy(c0))
        h.gemm_tiny(long_is_m, oa, ob, length, alpha, da, lda, db, ldb, beta_v, dc, ldc, sa, sb, sc,
                    batch)
        torch.cuda.synchronize()
        got = dc.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # against the FP64 truth as well: one batch entry, tolerance of a plain FP32 GEMM
    m, n = (length, 2) if long_is_m else (2, length)
    truth = oracle.gemm_f64(oa, ob, m, n, 2, alpha, a[:sa], lda, b[:sb] if sb else b, ldb, beta_v,
                            c0[:sc], ldc)
    assert oracle.residual(truth, got[:sc], ldc) < 1e-6


def test_rejects_bad_arguments():
    torch, api = _setup()
    h = api.Handle()
    x = torch.zeros(64, device="cuda")
    # not a power of two, leading dimension too small, empty batch
    assert h.gemm_tiny(True, 0, 0, 6, 1.0, x, 6, x, 2, 0.0, x, 6, check=False) == 7
    assert h.gemm_tiny(True, 0, 0, 8, 1.0, x, 4, x, 2, 0.0, x, 8, check=False) == 7
    assert h.gemm_tiny(False, 0, 0, 8, 1.0, x, 2, x, 1, 0.0, x, 2, check=False) == 7
    assert h.gemm_tiny(True, 0, 0, 8, 1.0, x, 8, x, 2, 0.0, x, 8, batch_count=0, check=False) == 7


def test_interception_routes_two_by_two_shapes(oracle):
    """With the switch on, cublasSgemm (m, 2, 2) gives the FP32 kernel's bits in every mode;
    with it off the compute mode decides (here: the corrected tensor-core kernel)."""
    torch, api = _setup()
    from cumpsgemm_b200 import _lib

    lib = _lib.load()
    blas = torch.cuda.current_blas_handle()
    m = 2048
    a, b = oracle.gen_normal(21, m * 2), oracle.gen_normal(22, 4)
    c0 = oracle.gen_normal(23, m * 2)
    want = c0.copy()
    oracle.tiny_gemm_f32(True, 0, 1, m, 1.5, a, m, b, 2, 0.5, want, m)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    alpha, beta = C.c_float(1.5), C.c_float(0.5)
    try:
        lib.cuMpSGEMM_hijack_enable_custom_gemm_Mx2x2()
        for mode in (0, 1, 9):
            lib.cuMpSGEMM_hijack_set_compute_mode(mode)
            dc = torch.from_numpy(c0).cuda()
            assert lib.cublasSgemm_v2(blas, 0, 1, m, 2, 2, C.byref(alpha), da.data_ptr(), m,
                                      db.data_ptr(), 2, C.byref(beta), dc.data_ptr(), m) == 0
            torch.cuda.synchronize()
            assert np.array_equal(dc.cpu().numpy().view(np.uint32), want.view(np.uint32)), mode
        # (2, n, 2) through the strided-batch entry point
        n, batch = 512, 3
        a2, b2 = oracle.gen_normal(24, 4 * batch), oracle.gen_normal(25, 2 * n * batch)
        c2 = np.zeros(2 * n * batch, dtype=np.float32)
        want2 = c2.copy()
        oracle.tiny_gemm_f32(False, 0, 0, n, 1.5, a2, 2, b2, 2, 0.0, want2, 2, 4, 2 * n, 2 * n, batch)
        d2a, d2b, d2c = (torch.from_numpy(x).cuda() for x in (a2, b2, c2))
        beta0 = C.c_float(0.0)
        assert lib.cublasSgemmStridedBatched(blas, 0, 0, 2, n, 2, C.byref(alpha), d2a.data_ptr(), 2,
                                             4, d2b.data_ptr(), 2, 2 * n, C.byref(beta0),
                                             d2c.data_ptr(), 2, 2 * n, batch) == 0
        torch.cuda.synchronize()
        assert np.array_equal(d2c.cpu().numpy().view(np.uint32), want2.view(np.uint32))
        # switched off: the FP16TCEC kernel runs instead (close, but not required to be equal)
        lib.cuMpSGEMM_hijack_disable_custom_gemm_Mx2x2()
        lib.cuMpSGEMM_hijack_set_compute_mode(1)
        dc = torch.from_numpy(c0).cuda()
        assert lib.cublasSgemm_v2(blas, 0, 1, m, 2, 2, C.byref(alpha), da.data_ptr(), m,
                                  db.data_ptr(), 2, C.byref(beta), dc.data_ptr(), m) == 0
        torch.cuda.synchronize()
        np.testing.assert_allclose(dc.cpu().numpy(), want, rtol=0, atol=1e-5)
    finally:
        lib.cuMpSGEMM_hijack_disable_custom_gemm_Mx2x2()
        lib.cuMpSGEMM_hijack_unset_compute_mode()
