"""Exponent statistics, decisions, flag words and scaling on the GPU: bit-exact against the
literal CPU restatement of src/exp_stats.cu and src/dynamic_scaling.cu; then the AUTO and
FP16TCEC_SCALING pipelines end to end."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N, T = 0, 1
FP16TCEC, TF32TCEC, AUTO, UNDEFINED, SCALING = 1, 2, 9, 10, 11


def _dev(x):
    import torch

    return torch.from_numpy(x).cuda()


def _slot(handle, sid):
    uf, total = handle.get_exp_stats(sid)
    return {"max_exp": handle.get_max_exp(sid), "total": total, "underflow": uf,
            "mode": int(handle.get_exp_stats_compute_mode_level(sid))}


CASES = [
    # (m, n, ld, batch, stride)
    (64, 64, 64, 1, 0),
    (1000, 37, 1000, 1, 0),          # contiguous, m*n % 4 == 0
    (333, 5, 340, 1, 0),             # ld > m, not a multiple of 4
    (128, 96, 132, 3, 132 * 96 + 4),  # batch with gap
    (100, 100, 100, 4, 10000),       # contiguous batch
    (7, 3, 7, 2, 21),                # tiny
    (5000, 2, 5000, 1, 0),           # several chunks per column
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("params", [(0.0, 2.0 ** -15, 0.0), (0.0, 2.0 ** -15, 0.1),
                                    (2.0 ** -20, 2.0 ** -12, 0.05)])
def test_exp_stats_bit_exact_real(handle, oracle, case, params):
    m, n, ld, batch, stride = case
    count = (stride * batch if stride else ld * n) + 3
    x = oracle.gen_wide_exponent(m + n, count, lo=-22, hi=2)
    handle.set_exp_stats_params(*params)
    d = _dev(x)
    sid = handle.exp_stats_ext(m, n, d, ld, batch, stride)
    want = oracle.exp_stats(x, m, n, ld, batch, stride, *params)
    assert _slot(handle, sid) == want
    # unaligned base pointer: the scalar path
    sid = handle.exp_stats_ext(m, n, d[1:], ld, batch, stride)
    want = oracle.exp_stats(x[1:], m, n, ld, batch, stride, *params)
    assert _slot(handle, sid) == want
    mid = handle.exp_max_ext(m, n, d, ld, batch, stride)
    assert handle.get_max_exp(mid) == oracle.exp_max(x, m, n, ld, batch, stride)


@pytest.mark.parametrize("case", CASES)
def test_one_launch_and_five_launch_paths_agree(handle, oracle, case):
    """exp_stats_ext runs two fused launches normally and the reference's five separate steps
    under the profiler (named timers): both leave the same slot, equal to the oracle's, for
    every decision outcome; a large scan (many CTAs, every ticket drawn) is included."""
    m, n, ld, batch, stride = case
    count = (stride * batch if stride else ld * n) + 3
    for seed, (lo, hi), params in ((1, (-3, 2), (0.0, 2.0 ** -15, 0.0)),
                                   (2, (-24, -20), (0.0, 2.0 ** -15, 0.0)),
                                   (3, (-30, 10), (0.0, 2.0 ** -15, 0.05))):
        x = oracle.gen_wide_exponent(seed, count, lo=lo, hi=hi)
        d = _dev(x)
        handle.set_exp_stats_params(*params)
        want = oracle.exp_stats(x, m, n, ld, batch, stride, *params)
        fused = _slot(handle, handle.exp_stats_ext(m, n, d, ld, batch, stride))
        fused_max = handle.get_max_exp(handle.exp_max_ext(m, n, d, ld, batch, stride))
        handle.enable_exp_stats_profiling()
        try:
            stepwise = _slot(handle, handle.exp_stats_ext(m, n, d, ld, batch, stride))
            stepwise_max = handle.get_max_exp(handle.exp_max_ext(m, n, d, ld, batch, stride))
        finally:
            handle.disable_exp_stats_profiling()
        assert fused == want and stepwise == want
        assert fused_max == stepwise_max == oracle.exp_max(x, m, n, ld, batch, stride)


def test_fused_scan_on_a_large_matrix(handle, oracle):
    m = n = 4096                       # 16 Mi values: more work items than resident CTAs
    x = oracle.gen_wide_exponent(9, m * n, lo=-28, hi=4)
    handle.set_exp_stats_params(0.0, 2.0 ** -15, 0.0)
    d = _dev(x)
    for _ in range(2):                 # the ticket counter is back at zero after every launch
        sid = handle.exp_stats_ext(m, n, d, m)
        assert _slot(handle, sid) == oracle.exp_stats(x, m, n, m, 1, 0, 0.0, 2.0 ** -15, 0.0)
        mid = handle.exp_max_ext(m, n, d, m)
        assert handle.get_max_exp(mid) == oracle.exp_max(x, m, n, m, 1, 0)


def test_exp_stats_bit_exact_complex(handle, oracle):
    m, n, ld, batch, stride = 90, 40, 96, 3, 96 * 40
    cnt = stride * batch
    z = (oracle.gen_wide_exponent(1, cnt, -20, 0) + 1j * oracle.gen_wide_exponent(2, cnt, -24, -2)).astype(np.complex64)
    handle.set_exp_stats_params(0.0, 2.0 ** -15, 0.3)
    sid = handle.exp_stats_ext(m, n, _dev(z), ld, batch, stride)
    assert _slot(handle, sid) == oracle.exp_stats(z, m, n, ld, batch, stride, 0.0, 2.0 ** -15, 0.3)


def test_decision_branches(handle, oracle):
    """Each decision outcome of src/exp_stats.cu:169-184 and :277-293."""
    handle.set_exp_stats_params(0.0, 2.0 ** -15, 0.0)
    well = oracle.gen_uniform(1, 4096) + np.float32(2.0)          # nothing underflows
    tiny = (well * np.float32(2.0 ** -22)).astype(np.float32)      # all tiny, tight range
    wide = oracle.gen_wide_exponent(2, 4096, -30, 10)              # wide range
    for x, mode in ((well, FP16TCEC), (tiny, SCALING), (wide, TF32TCEC)):
        sid = handle.exp_stats_ext(64, 64, _dev(x), 64)
        want = oracle.exp_stats(x, 64, 64, 64)
        assert want["mode"] == mode
        assert _slot(handle, sid) == want
    zeros = np.zeros(4096, dtype=np.float32)
    sid = handle.exp_stats_ext(64, 64, _dev(zeros), 64)
    assert _slot(handle, sid) == oracle.exp_stats(zeros, 64, 64, 64)


def test_ring_ids_and_reserved_slots(handle, oracle):
    import torch

    x = torch.ones(16, device="cuda")
    handle.reset_exp_stats_buffer_id()
    assert handle.get_current_exp_stats_buffer_id() == 1
    ids = [handle.exp_stats_ext(4, 4, x, 4) for _ in range(3)]
    assert ids == [2, 3, 4]                      # 0 and 1 are reserved
    assert int(handle.get_exp_stats_compute_mode_level(0)) == TF32TCEC
    assert int(handle.get_exp_stats_compute_mode_level(1)) == FP16TCEC
    # reserved flag slots (src/dynamic_launch.cu:6-9)
    assert int(handle.get_dynamic_launch_gemm_compute_mode(0)) == TF32TCEC
    assert int(handle.get_dynamic_launch_gemm_compute_mode(1)) == FP16TCEC
    assert handle.get_dynamic_launch_scaling_mode_AB(1) == (1, 1)
    first = handle.get_next_dynamic_launch_buffer_id()
    assert first == 2 and handle.get_current_dynamic_launch_buffer_id() == 2


def test_flag_from_stats_matches_oracle(handle, oracle):
    well = oracle.gen_uniform(1, 1024) + np.float32(2.0)
    tiny = (well * np.float32(2.0 ** -22)).astype(np.float32)
    wide = oracle.gen_wide_exponent(2, 1024, -30, 10)
    mats = {"F": well, "S": tiny, "T": wide}
    for ka, xa in mats.items():
        for kb, xb in mats.items():
            ia = handle.exp_stats_ext(32, 32, _dev(xa), 32)
            ib = handle.exp_stats_ext(32, 32, _dev(xb), 32)
            fid = handle.get_next_dynamic_launch_buffer_id()
            handle.set_dynamic_launch_buffer_by_exp_stats(fid, ia, ib)
            want = oracle.flag_from_modes(oracle.exp_stats(xa, 32, 32, 32)["mode"],
                                          oracle.exp_stats(xb, 32, 32, 32)["mode"])
            got = int(handle.get_dynamic_launch_gemm_compute_mode(fid))
            sa, sb = handle.get_dynamic_launch_scaling_mode_AB(fid)
            assert got | (sa << 6) | (sb << 5) == want, (ka, kb)


@pytest.mark.parametrize("cplx", [False, True])
def test_scaling_bit_exact_and_restoring(handle, oracle, cplx):
    import torch

    m, n, ld, batch, stride = 70, 50, 72, 2, 72 * 50 + 8
    cnt = stride * batch
    if cplx:
        x = (oracle.gen_wide_exponent(1, cnt, -24, -12) + 1j * oracle.gen_wide_exponent(2, cnt, -24, -12)).astype(np.complex64)
    else:
        x = oracle.gen_wide_exponent(1, cnt, -24, -12)
    d = _dev(x.copy())
    sid = handle.exp_max_ext(m, n, d, ld, batch, stride)
    mx = handle.get_max_exp(sid)
    assert mx == oracle.exp_max(x, m, n, ld, batch, stride)
    # flag slot 1: both operands scaled
    handle.scale_A(sid, 1, m, n, d, ld, batch, stride)
    want = x.copy()
    oracle.scale(oracle.SCALE_A, want, m, n, ld, batch, stride, 0x61, mx)
    np.testing.assert_array_equal(d.cpu().numpy().view(np.float32), want.view(np.float32))
    handle.reset_scale_A(sid, 1, m, n, d, ld, batch, stride)
    np.testing.assert_array_equal(d.cpu().numpy().view(np.float32), x.view(np.float32))
    # flag slot 0 (TF32TCEC, no scale bits): scale_B must not touch the data
    handle.scale_B(sid, 0, m, n, d, ld, batch, stride)
    np.testing.assert_array_equal(d.cpu().numpy().view(np.float32), x.view(np.float32))
    # scale_C with both bits: C *= maxA/2^14 * maxB/2^14
    sid_b = handle.exp_max_ext(m, n, d, ld, batch, stride)
    c = torch.ones(cnt, dtype=d.dtype, device="cuda")
    handle.scale_C(sid, sid_b, 1, m, n, c, ld, batch, stride)
    want_c = np.ones(cnt, dtype=x.dtype)
    oracle.scale(oracle.SCALE_C, want_c, m, n, ld, batch, stride, 0x61, mx, mx)
    np.testing.assert_array_equal(c.cpu().numpy().view(np.float32), want_c.view(np.float32))


def test_config3_statistics_8192(handle, oracle):
    """Benchmark config 3 inputs: sign uniform, exponent uniform over [-30, 10], 8192 x 8192.
    Counts, max exponent, decision and flag are compared bit-exactly."""
    n = 8192
    x = oracle.gen_wide_exponent(33, n * n)
    d = _dev(x)
    for params in ((0.0, 2.0 ** -15, 0.0), (0.0, 2.0 ** -15, 0.1)):
        handle.set_exp_stats_params(*params)
        sid = handle.exp_stats_ext(n, n, d, n)
        assert _slot(handle, sid) == oracle.exp_stats(x, n, n, n, 1, 0, *params)


def _auto_like(handle, oracle, mode, a, b, m, n, k, beta=0.0, c0=None):
    import torch

    da, db = _dev(a.copy()), _dev(b.copy())
    dc = _dev(c0.copy()) if c0 is not None else torch.zeros(m * n, device="cuda")
    handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, beta, dc, m, mode)
    # operands are never modified by the fused pipeline
    np.testing.assert_array_equal(da.cpu().numpy(), a)
    np.testing.assert_array_equal(db.cpu().numpy(), b)
    return dc


def test_scaling_mode_recovers_tiny_inputs(handle, oracle):
    """Tiny magnitudes: plain FP16TCEC loses the lo parts, FP16TCEC_SCALING does not."""
    m = n = k = 512
    a = (oracle.gen_uniform(1, m * k) * np.float32(2.0 ** -26)).astype(np.float32)
    b = (oracle.gen_uniform(2, k * n) * np.float32(2.0 ** -22)).astype(np.float32)
    truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m, b, k, 0.0, None, m)
    good = _auto_like(handle, oracle, SCALING, a, b, m, n, k).cpu().numpy()
    assert oracle.residual(truth, good, m) < oracle.error_threshold(True, k)
    import torch

    plain = torch.zeros(m * n, device="cuda")
    handle.gemm(N, N, m, n, k, 1.0, _dev(a), m, _dev(b), k, 0.0, plain, m, FP16TCEC)
    assert oracle.residual(truth, plain.cpu().numpy(), m) > 10 * oracle.error_threshold(True, k)


def test_fused_scaling_equals_explicit_sequence(handle, oracle):
    """The fused pipeline gives bit-identical results to the reference's explicit sequence
    exp_max -> scale_A/B (in place) -> gemm(FP16TCEC) -> scale_C -> reset (beta = 0)."""
    import torch

    m, n, k = 300, 200, 260
    a = (oracle.gen_uniform(3, m * k) * np.float32(2.0 ** -20)).astype(np.float32)
    b = (oracle.gen_uniform(4, k * n) * np.float32(2.0 ** -18)).astype(np.float32)
    fused = _auto_like(handle, oracle, SCALING, a, b, m, n, k)
    da, db = _dev(a.copy()), _dev(b.copy())
    dc = torch.zeros(m * n, device="cuda")
    ia = handle.exp_max_ext(m, k, da, m)
    ib = handle.exp_max_ext(k, n, db, k)
    handle.scale_A(ia, 1, m, k, da, m)
    handle.scale_B(ib, 1, k, n, db, k)
    handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.0, dc, m, FP16TCEC)
    handle.scale_C(ia, ib, 1, m, n, dc, m)
    handle.reset_scale_A(ia, 1, m, k, da, m)
    handle.reset_scale_B(ib, 1, k, n, db, k)
    assert torch.equal(fused, dc)
    np.testing.assert_array_equal(da.cpu().numpy(), a)
    np.testing.assert_array_equal(db.cpu().numpy(), b)


def test_auto_via_explicit_flag_slot(handle, oracle):
    """Reference-style direct API use: exp_stats_ext on A and B, flag from the statistics,
    set_dynamic_launch_flag_buffer_id, gemm(..., AUTO) launches both kinds gated by the flag."""
    import torch

    m = n = k = 256
    well = oracle.gen_uniform(1, m * k) + np.float32(2)
    wide = oracle.gen_wide_exponent(5, k * n, -28, 4)
    for a, b, kind in ((well, well, FP16TCEC), (well, wide, TF32TCEC)):
        da, db = _dev(a), _dev(b)
        ia = handle.exp_stats_ext(m, k, da, m)
        ib = handle.exp_stats_ext(k, n, db, k)
        fid = handle.get_next_dynamic_launch_buffer_id()
        handle.set_dynamic_launch_buffer_by_exp_stats(fid, ia, ib)
        assert int(handle.get_dynamic_launch_gemm_compute_mode(fid)) == kind
        handle.set_dynamic_launch_flag_buffer_id(fid)
        dc = torch.zeros(m * n, device="cuda")
        handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.0, dc, m, AUTO)
        handle.unset_dynamic_launch_flag_buffer_id()
        ref = torch.zeros(m * n, device="cuda")
        handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.0, ref, m, kind)
        assert torch.equal(dc, ref)          # the gated launch is the same kernel


def test_with_stats_entry_point_auto(handle, oracle):
    """Fused AUTO through decided statistics slots (the multi-GPU entry point, world size 1)."""
    import torch

    m, n, k = 200, 180, 320
    a = (oracle.gen_uniform(1, m * k) * np.float32(2.0 ** -25) + np.float32(2.0 ** -24)).astype(np.float32)
    b = oracle.gen_uniform(2, k * n) + np.float32(2)
    c0 = oracle.gen_uniform(3, m * n)
    da, db, dc = _dev(a), _dev(b), _dev(c0.copy())
    ia = handle.exp_stats_ext(m, k, da, m)
    ib = handle.exp_stats_ext(k, n, db, k)
    assert int(handle.get_exp_stats_compute_mode_level(ia)) == SCALING
    handle.gemm_strided_batch_with_stats(N, N, m, n, k, 1.0, da, m, 0, db, k, 0, 0.5, dc, m, 0, 1,
                                         AUTO, ia, ib)
    # beta*C is not multiplied by the un-scaling factor: result is alpha*A*B + beta*C0
    truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c0, m)
    assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)


def test_config4_strided_batch_cgemm_scaling(handle, oracle):
    """Benchmark config 4, reduced batch: complex 256^3 with unit-Frobenius operands,
    FP16TCEC_SCALING, statistics over the whole batch."""
    import torch

    batch, s = 8, 256
    za = oracle.gen_unit_frobenius_complex(1, batch, s, s)
    zb = oracle.gen_unit_frobenius_complex(2, batch, s, s)
    da, db = _dev(za), _dev(zb)
    dc = torch.zeros(batch * s * s, dtype=torch.complex64, device="cuda")
    handle.gemm_strided_batch(N, N, s, s, s, 1.0, da, s, s * s, db, s, s * s, 0.0, dc, s, s * s,
                              batch, SCALING)
    res = dc.cpu().numpy()
    for i in range(batch):
        truth = oracle.gemm_f64(N, N, s, s, s, 1.0, za[i * s * s:], s, zb[i * s * s:], s, 0.0, None, s)
        assert oracle.residual(truth, res[i * s * s:(i + 1) * s * s], s) < oracle.error_threshold(True, s)


def test_named_timers(handle, oracle):
    """Timer names the reference's bandwidth test looks up (test/main.cu:1329-1337)."""
    import torch

    x = torch.ones(1 << 20, device="cuda")
    handle.enable_exp_stats_profiling()
    sid = handle.exp_stats_ext(1024, 1024, x, 1024)
    handle.scale_A(sid, 1, 1024, 1024, x, 1024)
    handle.scale_C(sid, sid, 1, 1024, 1024, x, 1024)
    handle.disable_exp_stats_profiling()
    for name in ("exp_stats_init", "exp_stats_1", "exp_stats_set_1", "exp_stats_2", "exp_stats_set_2",
                 "scaling_AB", "scaling_C"):
        r = handle.get_exp_stats_profiling_result(name)
        assert r is not None and r[1] == 1 and r[0] > 0
    handle.reset_exp_stats_profiling()
    assert handle.get_exp_stats_profiling_result("exp_stats_1") is None


def test_gemm_call_statistics_equal_separate_calls(handle, oracle):
    """A GEMM call in AUTO / FP16TCEC_SCALING takes the statistics of A and B in shared
    launches and derives flag and scaling constants in one more; the slots it leaves are the
    ones separate exp_stats_ext / exp_max_ext calls leave (= the oracle's), for every decision
    outcome of the pair, and so are flag word and result."""
    import ctypes as C
    import torch
    from cumpsgemm_b200 import _lib, api

    lib = _lib.load()
    blas = torch.cuda.current_blas_handle()
    m, n, k = 1100, 1060, 1030                      # above the default rule's size threshold
    alpha, beta = C.c_float(1.0), C.c_float(0.0)
    well = lambda s, cnt: oracle.gen_uniform(s, cnt) + np.float32(2.0)
    tiny = lambda s, cnt: ((oracle.gen_uniform(s, cnt) + np.float32(2.0)) * np.float32(2.0 ** -22)).astype(np.float32)
    wide = lambda s, cnt: oracle.gen_wide_exponent(s, cnt, -30, 10)
    # a non-owning view of the interception layer's own handle
    gh = api.Handle.__new__(api.Handle)
    gh._lib = lib
    try:
        for ga, gb in ((well, well), (tiny, well), (well, tiny), (wide, well), (tiny, wide)):
            a, b = ga(1, m * k), gb(2, k * n)
            da, db = _dev(a), _dev(b)
            for mode in (9, 11):                    # AUTO, FP16TCEC_SCALING
                assert lib.cuMpSGEMM_hijack_set_compute_mode(mode) == 0
                dc = torch.zeros(m * n, device="cuda")
                assert lib.cublasSgemm_v2(blas, 0, 0, m, n, k, C.byref(alpha), da.data_ptr(), m,
                                          db.data_ptr(), k, C.byref(beta), dc.data_ptr(), m) == 0
                torch.cuda.synchronize()
                gh._h = C.c_void_p(lib.cuMpSGEMM_hijack_get_internal_global_handle())
                id_b = gh.get_current_exp_stats_buffer_id()
                id_a = id_b - 1
                if mode == 9:
                    assert _slot(gh, id_a) == oracle.exp_stats(a, m, k, m)
                    assert _slot(gh, id_b) == oracle.exp_stats(b, k, n, k)
                    fid = gh.get_current_dynamic_launch_buffer_id()
                    want_flag = oracle.flag_from_modes(oracle.exp_stats(a, m, k, m)["mode"],
                                                       oracle.exp_stats(b, k, n, k)["mode"])
                    got_mode = int(gh.get_dynamic_launch_gemm_compute_mode(fid))
                    sa, sb = gh.get_dynamic_launch_scaling_mode_AB(fid)
                    assert (got_mode | (0x40 if sa else 0) | (0x20 if sb else 0)) == want_flag
                else:
                    assert gh.get_max_exp(id_a) == oracle.exp_max(a, m, k, m)
                    assert gh.get_max_exp(id_b) == oracle.exp_max(b, k, n, k)
                truth = oracle.gemm_f64(0, 0, m, n, k, 1.0, a, m, b, k, 0.0, None, m)
                assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
    finally:
        lib.cuMpSGEMM_hijack_unset_compute_mode()
        gh._h = None
