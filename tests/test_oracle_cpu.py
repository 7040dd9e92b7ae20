"""The CPU oracle against known answers, the reference-derived golden fixtures and itself."""
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_gemm_f64_matches_numpy(oracle):
    m, n, k = 37, 29, 83
    for op_a in (0, 1):
        for op_b in (0, 1):
            am, an = (m, k) if op_a == 0 else (k, m)
            bm, bn = (k, n) if op_b == 0 else (n, k)
            lda, ldb, ldc = am + 3, bm + 1, m + 2
            a = oracle.gen_uniform(1, lda * an)
            b = oracle.gen_uniform(2, ldb * bn)
            c = oracle.gen_uniform(3, ldc * n)
            A = a.reshape((lda, an), order="F")[:am].astype(np.float64)
            B = b.reshape((ldb, bn), order="F")[:bm].astype(np.float64)
            C0 = c.reshape((ldc, n), order="F")[:m].astype(np.float64)
            expect = 1.5 * (A if op_a == 0 else A.T) @ (B if op_b == 0 else B.T) - 0.25 * C0
            got = oracle.gemm_f64(op_a, op_b, m, n, k, 1.5, a, lda, b, ldb, -0.25, c, ldc)
            np.testing.assert_allclose(got, expect, rtol=1e-13, atol=1e-13)


def test_cgemm_f64_matches_numpy(oracle):
    m, n, k = 11, 13, 17
    a = (oracle.gen_uniform(1, k * m) + 1j * oracle.gen_uniform(2, k * m)).astype(np.complex64)
    b = (oracle.gen_uniform(3, k * n) + 1j * oracle.gen_uniform(4, k * n)).astype(np.complex64)
    A = a.reshape((k, m), order="F").astype(np.complex128)
    B = b.reshape((k, n), order="F").astype(np.complex128)
    got = oracle.gemm_f64(2, 0, m, n, k, 1 + 2j, a, k, b, k, 0.0, None, m)  # op C on A
    np.testing.assert_allclose(got, (1 + 2j) * (A.conj().T @ B), rtol=1e-13, atol=1e-13)
    got = oracle.gemm_f64(1, 0, m, n, k, 1.0, a, k, b, k, 0.0, None, m)  # op T on A
    np.testing.assert_allclose(got, A.T @ B, rtol=1e-13, atol=1e-13)


def test_fp16_split_known_answers(oracle):
    # 1 + 2^-12 is not an FP16 value: hi = 1, lo = 2^-12 * 2^11 = 0.5 (exact)
    x = np.array([1.0 + 2.0 ** -12, 0.1, -3.0, 0.0, 2.0 ** -20], dtype=np.float32)
    hi, lo = oracle.split(x, 0)
    assert hi[0] == 1.0 and lo[0] == 0.5
    assert hi[2] == -3.0 and lo[2] == 0.0
    assert hi[3] == 0.0 and lo[3] == 0.0
    # hi + lo/2^11 recovers the input to about 2^-22 relative
    rec = hi.astype(np.float64) + lo.astype(np.float64) / 2048.0
    assert np.all(np.abs(rec - x) <= np.abs(x) * 2.0 ** -21)
    assert np.all(hi == x.astype(np.float16).astype(np.float32))


def test_tf32_split_known_answers(oracle):
    x = np.array([1.0 + 2.0 ** -11, 1.0 + 2.0 ** -10, 0.1], dtype=np.float32)
    hi, lo = oracle.split(x, 1)
    # ties away from zero: 1 + 2^-11 rounds up to 1 + 2^-10
    assert hi[0] == np.float32(1.0 + 2.0 ** -10) and lo[0] == np.float32(-(2.0 ** -11))
    assert hi[1] == x[1] and lo[1] == 0.0
    assert (hi.view(np.uint32) & 0x1FFF).max() == 0
    assert np.all(np.abs((hi.astype(np.float64) + lo) - x) <= np.abs(x) * 2.0 ** -20)


@pytest.mark.parametrize("kind", [0, 1])
def test_tcec_model_reaches_fp32_accuracy(oracle, kind):
    m, n, k = 48, 40, 512
    a = oracle.gen_uniform(5, m * k)
    b = oracle.gen_uniform(6, k * n)
    truth = oracle.gemm_f64(0, 0, m, n, k, 1.0, a, m, b, k, 0.0, None, m)
    model = oracle.tcec_model(kind, 0, 0, m, n, k, 1.0, a, m, b, k, 0.0, None, m, k_chunk=64)
    c32 = np.zeros(m * n, dtype=np.float32)
    oracle.gemm_f32(0, 0, m, n, k, 1.0, a, m, b, k, 0.0, c32, m)
    r_model = oracle.residual(truth, np.asfortranarray(model).ravel(order="F"), m)
    r_f32 = oracle.residual(truth, c32, m)
    assert r_model < oracle.error_threshold(True, k)   # reference criterion, test/main.cu:68-74
    assert r_model <= 2.0 * r_f32                       # "no worse than FP32 SIMT"


def test_exp_stats_known_answers(oracle):
    # 8 values: max 3.0 -> exponent bits of 2.0; one value below 2^-15; zeros count as total
    x = np.array([1.0, -3.0, 0.5, 2.0 ** -16, 0.25, -0.125, 1.5, 2.0], dtype=np.float32)
    s = oracle.exp_stats(x, 4, 2, 4, tolerance=0.5)
    assert s == {"max_exp": 2.0, "total": 8, "underflow": 1, "mode": oracle.FP16TCEC}
    # default tolerance 0: one underflow sends it to stage 2; relative thresholds
    # (2^-15 / 2) * 2.0 = 2^-15 -> 2^-16 underflows again -> TF32TCEC
    s = oracle.exp_stats(x, 4, 2, 4)
    assert s == {"max_exp": 2.0, "total": 8, "underflow": 1, "mode": oracle.TF32TCEC}
    # all tiny but tightly clustered: stage 1 fails, stage 2 (relative) passes -> scaling
    y = (x * np.float32(2.0 ** -20)).astype(np.float32)
    y[3] = y[0]
    s = oracle.exp_stats(y, 4, 2, 4)
    assert s["mode"] == oracle.FP16TCEC_SCALING and s["max_exp"] == 2.0 ** -19
    assert s["total"] == 8 and s["underflow"] == 0
    # nothing underflows -> FP16TCEC after stage 1
    z = np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float32)
    assert oracle.exp_stats(z, 2, 2, 2)["mode"] == oracle.FP16TCEC
    # ignore threshold above every value while max > 0: "total == 0" branch -> stage 2
    s = oracle.exp_stats(z, 2, 2, 2, ignore_threshold=100.0)
    assert s["mode"] in (oracle.FP16TCEC_SCALING, oracle.TF32TCEC)


def test_exp_stats_ld_batch_and_padding(oracle):
    m, n, ld, batch = 5, 3, 8, 2
    stride = ld * n + 4
    buf = np.full(stride * batch, 1e-30, dtype=np.float32)  # gaps hold tiny values
    vals = oracle.gen_uniform(9, m * n * batch)
    for b in range(batch):
        for j in range(n):
            buf[b * stride + j * ld: b * stride + j * ld + m] = vals[(b * n + j) * m:(b * n + j + 1) * m]
    s = oracle.exp_stats(buf, m, n, ld, batch, stride, tolerance=1.0)
    assert s["total"] == m * n * batch and s["underflow"] == int((np.abs(vals) < 2.0 ** -15).sum())
    # stride 0 = single matrix, whatever the batch argument says
    s1 = oracle.exp_stats(buf, m, n, ld, batch, 0, tolerance=1.0)
    assert s1["total"] == m * n
    # the reference's tail padding: (4 - 15 % 4) % 4 = 1 zero per matrix counted in total and underflow
    sp = oracle.exp_stats(buf, m, n, ld, batch, stride, tolerance=1.0, count_padding=True)
    assert sp["total"] == s["total"] + batch and sp["underflow"] == s["underflow"] + batch


def test_complex_stats_count_re_and_im(oracle):
    z = np.array([1 + 2.0 ** -16 * 1j, 2.0 ** -17 + 4j], dtype=np.complex64)
    s = oracle.exp_stats(z, 2, 1, 2, tolerance=1.0)
    assert s["total"] == 4 and s["underflow"] == 2 and s["max_exp"] == 4.0


def test_flag_word_against_reference_golden(oracle):
    golden = json.loads((GOLDEN / "flag_golden.json").read_text())
    for g in golden:
        f = g["flag"]
        assert (f & 0x1F) == g["get_gemm"]
        assert int(bool(f & 0x40)) == g["get_scale_A"]
        assert int(bool(f & 0x20)) == g["get_scale_B"]
        assert ((f & 0x60) | 2) == g["set_gemm_2"]
        assert ((f & ~0x40) | 0x40) == g["set_A_on"] and (f & ~0x40 & 0x7F) == g["set_A_off"]
        assert ((f & ~0x20) | 0x20) == g["set_B_on"] and (f & ~0x20 & 0x7F) == g["set_B_off"]
    S, F, T = oracle.FP16TCEC_SCALING, oracle.FP16TCEC, oracle.TF32TCEC
    assert oracle.flag_from_modes(F, F) == 1
    assert oracle.flag_from_modes(S, F) == (1 | 0x40)
    assert oracle.flag_from_modes(F, S) == (1 | 0x20)
    assert oracle.flag_from_modes(S, S) == (1 | 0x60)
    assert oracle.flag_from_modes(T, S) == 2 and oracle.flag_from_modes(S, T) == 2


def test_scaling_is_exact_and_reversible(oracle):
    x = oracle.gen_wide_exponent(4, 6 * 5, lo=-20, hi=-10)
    mx = oracle.exp_max(x, 6, 5, 6)
    y = x.copy()
    oracle.scale(oracle.SCALE_A, y, 6, 5, 6, 1, 0, 0x60 | 1, mx)
    assert oracle.exp_max(y, 6, 5, 6) == 2.0 ** 14
    np.testing.assert_array_equal(y, x * np.float32(2.0 ** 14 / mx))
    oracle.scale(oracle.RESET_A, y, 6, 5, 6, 1, 0, 0x60 | 1, mx)
    np.testing.assert_array_equal(y, x)
    # flag bit of A clear: scale_A is a no-op, scale_B acts
    y = x.copy()
    oracle.scale(oracle.SCALE_A, y, 6, 5, 6, 1, 0, 0x20 | 1, mx)
    np.testing.assert_array_equal(y, x)
    oracle.scale(oracle.SCALE_B, y, 6, 5, 6, 1, 0, 0x20 | 1, mx)
    assert oracle.exp_max(y, 6, 5, 6) == 2.0 ** 14
    # scale_C multiplies by the product of the applied inverse factors
    c = np.ones(4, dtype=np.float32)
    oracle.scale(oracle.SCALE_C, c, 2, 2, 2, 1, 0, 0x60 | 1, 2.0 ** -10, 2.0 ** 3)
    np.testing.assert_array_equal(c, np.full(4, 2.0 ** -24 * 2.0 ** -11, dtype=np.float32))
    c = np.ones(4, dtype=np.float32)
    oracle.scale(oracle.SCALE_C, c, 2, 2, 2, 1, 0, 0x60 | 1, 0.0, 8.0)  # max of A is zero: untouched
    np.testing.assert_array_equal(c, np.ones(4, dtype=np.float32))


def test_generators_are_seeded(oracle):
    np.testing.assert_array_equal(oracle.gen_uniform_exp(3, 100), oracle.gen_uniform_exp(3, 100))
    x = oracle.gen_wide_exponent(1, 10000)
    e = np.floor(np.log2(np.abs(x)))
    assert e.min() == -30 and e.max() == 10
    z = oracle.gen_unit_frobenius_complex(2, 3, 16, 16).reshape(3, -1)
    np.testing.assert_allclose((np.abs(z) ** 2).sum(axis=1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("long_is_m", [True, False])
@pytest.mark.parametrize("op_a,op_b", [(0, 0), (1, 0), (0, 1), (2, 2)])
def test_tiny_gemm_restatement_against_fp64(oracle, cplx, long_is_m, op_a, op_b):
    """The FP32 restatement of the (m,2,2)/(2,n,2) route agrees with the FP64 truth to FP32
    rounding, for every operand layout, with padded leading dimensions and a batch."""
    length, batch, pad = 64, 3, 2

    def gen(seed, count):
        x = oracle.gen_normal(seed, count)
        return (x + 1j * oracle.gen_normal(seed + 50, count)).astype(np.complex64) if cplx else x

    a_rc = ((length, 2) if op_a == 0 else (2, length)) if long_is_m else (2, 2)
    b_rc = (2, 2) if long_is_m else ((2, length) if op_b == 0 else (length, 2))
    c_rc = (length, 2) if long_is_m else (2, length)
    lda, ldb, ldc = a_rc[0] + pad, b_rc[0] + pad, c_rc[0] + pad
    sa, sb, sc = lda * a_rc[1] + 3, ldb * b_rc[1] + 1, ldc * c_rc[1]
    a, b, c0 = gen(1, sa * batch), gen(2, sb * batch), gen(3, sc * batch)
    alpha, beta = ((0.5 + 0.25j), (-1.0 + 0.5j)) if cplx else (0.5, -1.0)
    got = c0.copy()
    oracle.tiny_gemm_f32(long_is_m, op_a, op_b, length, alpha, a, lda, b, ldb, beta, got, ldc, sa,
                         sb, sc, batch)
    m, n = c_rc
    for bt in range(batch):
        truth = oracle.gemm_f64(op_a, op_b, m, n, 2, alpha, a[bt * sa:], lda, b[bt * sb:], ldb,
                                beta, c0[bt * sc:], ldc)
        assert oracle.residual(truth, got[bt * sc:], ldc) < 1e-6
    # padding rows of C are untouched
    g2 = got.reshape(batch, c_rc[1], ldc)
    c2 = c0.reshape(batch, c_rc[1], ldc)
    assert np.array_equal(g2[:, :, c_rc[0]:], c2[:, :, c_rc[0]:])


def test_reference_checker_library_exports_its_entry_points(oracle):
    """oracle/_ref/libref_stats.so (the reference's own statistics / scaling sources compiled for
    sm_100a) loads without a GPU and exports every entry point the GPU pin test calls."""
    import ctypes as C

    if not oracle.ReferenceStats.available():
        pytest.skip("reference checker not built (the reference tree was absent at build time)")
    L = C.CDLL(str(oracle.ReferenceStats.PATH))
    for name in ("ref_create", "ref_destroy", "ref_set_exp_stats_params", "ref_exp_stats_ext_s",
                 "ref_exp_stats_ext_c", "ref_exp_max_ext_s", "ref_exp_max_ext_c",
                 "ref_get_exp_stats", "ref_get_max_exp", "ref_get_compute_mode_level",
                 "ref_next_flag_id", "ref_set_flag_by_exp_stats", "ref_get_flag", "ref_scale_s",
                 "ref_scale_c"):
        assert hasattr(L, name), name


def test_oracle_thread_control(oracle):
    """The timed CPU baseline asks for its threads explicitly (launchers that start one process
    per GPU export OMP_NUM_THREADS=1)."""
    import os

    try:
        assert oracle.set_num_threads(2) == 2
        assert oracle.set_num_threads(1) == 1
    finally:
        oracle.set_num_threads(len(os.sched_getaffinity(0)))
