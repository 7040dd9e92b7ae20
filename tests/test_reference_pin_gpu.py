"""Statistics, decisions, flag words and scaling pinned to the reference's own kernels.

``oracle/_ref/libref_stats.so`` holds the reference's src/exp_stats.cu, src/dynamic_scaling.cu
and src/dynamic_launch.cu, compiled unmodified for sm_100a against stand-in headers for the
absent cutf library (``make -C oracle ref_gpu``).  Reference and product run here on the same
device buffers and must leave the same bits: slot contents (maximum exponent, total,
underflow, decision), flag words and scaled matrices.  The CPU restatement in oracle/ is
checked against the reference in the same pass, which is what pins it.

Where m*n is not a multiple of 4 the reference counts the zeros its 4-wide loop appends
(src/exp_stats.cu:101-116); the product reproduces that only with the compatibility switch
on, and the difference with the switch off must be exactly what the oracle's `count_padding`
models.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FP16TCEC, TF32TCEC, UNDEFINED, SCALING = 1, 2, 10, 11
SCALE_A, SCALE_B, SCALE_C, RESET_A, RESET_B = 0, 1, 2, 3, 4


@pytest.fixture(scope="module")
def ref(oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not oracle.ReferenceStats.available():
        pytest.skip("oracle/_ref/libref_stats.so is not built (needs the reference tree at build time)")
    r = oracle.ReferenceStats()
    yield r
    r.close()


def _dev(x):
    import torch

    return torch.from_numpy(x).cuda()


def _slot(handle, sid):
    uf, total = handle.get_exp_stats(sid)
    return {"max_exp": handle.get_max_exp(sid), "total": total, "underflow": uf,
            "mode": int(handle.get_exp_stats_compute_mode_level(sid))}


def _flag_word(handle, fid):
    sa, sb = handle.get_dynamic_launch_scaling_mode_AB(fid)
    return int(handle.get_dynamic_launch_gemm_compute_mode(fid)) | (0x40 if sa else 0) | \
        (0x20 if sb else 0)


# (m, n, ld, batch, stride); element counts both divisible and not divisible by 4
CASES = [
    (64, 64, 64, 1, 0),
    (1000, 37, 1000, 1, 0),
    (333, 5, 340, 1, 0),              # 1665 elements: one padded zero
    (127, 63, 127, 1, 0),             # 8001 elements: three padded zeros
    (128, 96, 132, 3, 132 * 96 + 4),
    (101, 3, 101, 4, 303),            # 303 elements per matrix, four matrices
    (7, 3, 7, 2, 21),
    (2048, 2048, 2048, 1, 0),         # 1024-thread variant of the reference's kernels
]
PARAMS = [(0.0, 2.0 ** -15, 0.0), (0.0, 2.0 ** -15, 0.1), (2.0 ** -20, 2.0 ** -12, 0.05)]
RANGES = [(-3, 2), (-24, -20), (-30, 10)]   # decided at stage 1 / SCALING / TF32TCEC (mostly)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("params", PARAMS)
def test_statistics_equal_the_reference_real(handle, oracle, ref, case, params):
    m, n, ld, batch, stride = case
    count = (stride * batch if stride else ld * n) + 3
    handle.set_exp_stats_params(*params)
    ref.set_exp_stats_params(*params)
    padded = (m * n) % 4 != 0
    for seed, (lo, hi) in enumerate(RANGES):
        x = oracle.gen_wide_exponent(100 + seed + m, count, lo=lo, hi=hi)
        d = _dev(x)
        want = ref.slot(ref.exp_stats_ext(m, n, d.data_ptr(), ld, batch, stride))
        # the CPU restatement, with the reference's padding rule, equals the reference
        assert oracle.exp_stats(x, m, n, ld, batch, stride, *params, count_padding=True) == want
        handle.set_count_tail_padding(True)
        try:
            got = _slot(handle, handle.exp_stats_ext(m, n, d, ld, batch, stride))
        finally:
            handle.set_count_tail_padding(False)
        assert got == want
        plain = _slot(handle, handle.exp_stats_ext(m, n, d, ld, batch, stride))
        assert plain == oracle.exp_stats(x, m, n, ld, batch, stride, *params)
        if not padded:
            assert plain == want
        # maximum exponent only
        assert handle.get_max_exp(handle.exp_max_ext(m, n, d, ld, batch, stride)) == \
            ref.max_exp(ref.exp_max_ext(m, n, d.data_ptr(), ld, batch, stride))


@pytest.mark.parametrize("case", [(96, 40, 96, 1, 0), (33, 7, 35, 1, 0), (50, 9, 50, 3, 450),
                                  (256, 256, 256, 8, 65536)])
@pytest.mark.parametrize("params", PARAMS[:2])
def test_statistics_equal_the_reference_complex(handle, oracle, ref, case, params):
    m, n, ld, batch, stride = case
    count = (stride * batch if stride else ld * n) + 2
    handle.set_exp_stats_params(*params)
    ref.set_exp_stats_params(*params)
    for seed, (lo, hi) in enumerate(RANGES):
        re = oracle.gen_wide_exponent(7 + seed, count, lo=lo, hi=hi)
        im = oracle.gen_wide_exponent(70 + seed, count, lo=lo - 2, hi=hi - 1)
        z = (re + 1j * im).astype(np.complex64)
        d = _dev(z)
        want = ref.slot(ref.exp_stats_ext(m, n, d.data_ptr(), ld, batch, stride, complex=True))
        assert oracle.exp_stats(z, m, n, ld, batch, stride, *params, count_padding=True) == want
        handle.set_count_tail_padding(True)
        try:
            got = _slot(handle, handle.exp_stats_ext(m, n, d, ld, batch, stride))
        finally:
            handle.set_count_tail_padding(False)
        assert got == want
        assert handle.get_max_exp(handle.exp_max_ext(m, n, d, ld, batch, stride)) == \
            ref.max_exp(ref.exp_max_ext(m, n, d.data_ptr(), ld, batch, stride, complex=True))


def test_compatibility_switch_by_environment(oracle, ref, monkeypatch):
    """CUMPSGEMM_COUNT_TAIL_PADDING=1 at handle creation = the setter."""
    from cumpsgemm_b200 import api

    monkeypatch.setenv("CUMPSGEMM_COUNT_TAIL_PADDING", "1")
    m, n = 127, 63
    x = oracle.gen_wide_exponent(5, m * n, lo=-24, hi=-20)
    d = _dev(x)
    ref.set_exp_stats_params(0.0, 2.0 ** -15, 0.0)
    want = ref.slot(ref.exp_stats_ext(m, n, d.data_ptr(), m, 1, 0))
    with api.Handle() as h:
        h.use_current_torch_stream()
        assert _slot(h, h.exp_stats_ext(m, n, d, m)) == want
    monkeypatch.delenv("CUMPSGEMM_COUNT_TAIL_PADDING")
    with api.Handle() as h:
        h.use_current_torch_stream()
        got = _slot(h, h.exp_stats_ext(m, n, d, m))
    assert got == oracle.exp_stats(x, m, n, m)
    assert got["total"] == want["total"] - 3


@pytest.mark.parametrize("ranges", [((-3, 2), (-3, 2)), ((-24, -20), (-3, 2)),
                                    ((-3, 2), (-22, -19)), ((-24, -20), (-23, -19)),
                                    ((-30, 10), (-3, 2)), ((-24, -20), (-30, 10))])
def test_flag_words_and_scaling_equal_the_reference(handle, oracle, ref, ranges):
    """AUTO pipeline pieces in the reference's order (src/cumpsgemm_cublas.cu:445-577):
    statistics of A and B -> flag word -> scale A, B -> (GEMM) -> scale C -> restore A, B.
    Every matrix after every step equals the reference's bit for bit."""
    import torch

    m, n, k = 200, 120, 160
    lda, ldb, ldc = 208, 160, 200
    params = (0.0, 2.0 ** -15, 0.0)
    handle.set_exp_stats_params(*params)
    ref.set_exp_stats_params(*params)
    a = oracle.gen_wide_exponent(31, lda * k, lo=ranges[0][0], hi=ranges[0][1])
    b = oracle.gen_wide_exponent(32, ldb * n, lo=ranges[1][0], hi=ranges[1][1])
    c = oracle.gen_uniform(33, ldc * n)
    da, db, dc = _dev(a), _dev(b), _dev(c)
    ra, rb, rc = da.clone(), db.clone(), dc.clone()

    ida, idb = handle.exp_stats_ext(m, k, da, lda), handle.exp_stats_ext(k, n, db, ldb)
    rida = ref.exp_stats_ext(m, k, ra.data_ptr(), lda)
    ridb = ref.exp_stats_ext(k, n, rb.data_ptr(), ldb)
    assert _slot(handle, ida) == ref.slot(rida)
    assert _slot(handle, idb) == ref.slot(ridb)

    fid = handle.get_next_dynamic_launch_buffer_id()
    handle.set_dynamic_launch_buffer_by_exp_stats(fid, ida, idb)
    rfid, rflag = ref.flag_from_stats(rida, ridb)
    assert _flag_word(handle, fid) == rflag
    assert rflag == oracle.flag_from_modes(ref.slot(rida)["mode"], ref.slot(ridb)["mode"])

    handle.scale_A(ida, fid, m, k, da, lda)
    handle.scale_B(idb, fid, k, n, db, ldb)
    ref.scale(SCALE_A, m, k, ra.data_ptr(), lda, 1, 0, rida, 0, rfid)
    ref.scale(SCALE_B, k, n, rb.data_ptr(), ldb, 1, 0, ridb, 0, rfid)
    torch.cuda.synchronize()
    assert torch.equal(da, ra) and torch.equal(db, rb)
    handle.scale_C(ida, idb, fid, m, n, dc, ldc)
    ref.scale(SCALE_C, m, n, rc.data_ptr(), ldc, 1, 0, rida, ridb, rfid)
    handle.reset_scale_A(ida, fid, m, k, da, lda)
    handle.reset_scale_B(idb, fid, k, n, db, ldb)
    ref.scale(RESET_A, m, k, ra.data_ptr(), lda, 1, 0, rida, 0, rfid)
    ref.scale(RESET_B, k, n, rb.data_ptr(), ldb, 1, 0, ridb, 0, rfid)
    torch.cuda.synchronize()
    assert torch.equal(dc, rc)
    assert torch.equal(da, ra) and torch.equal(db, rb)
    # restored operands equal the originals (powers of two; nothing under- or overflowed here)
    assert torch.equal(da, _dev(a)) and torch.equal(db, _dev(b))


def test_forced_scaling_slot_and_complex_batches_equal_the_reference(handle, oracle, ref):
    """FP16TCEC_SCALING path: exp_max on both operands, reserved flag slot 1 (both scale bits,
    src/dynamic_launch.cu:6-9), strided complex batches."""
    import torch

    batch, s = 6, 48
    za = oracle.gen_unit_frobenius_complex(3, batch, s, s)
    zb = oracle.gen_unit_frobenius_complex(4, batch, s, s)
    zc = (oracle.gen_uniform(5, batch * s * s) + 1j * oracle.gen_uniform(6, batch * s * s)).astype(
        np.complex64)
    da, db, dc = _dev(za), _dev(zb), _dev(zc)
    ra, rb, rc = da.clone(), db.clone(), dc.clone()
    ida, idb = handle.exp_max_ext(s, s, da, s, batch, s * s), handle.exp_max_ext(s, s, db, s, batch, s * s)
    rida = ref.exp_max_ext(s, s, ra.data_ptr(), s, batch, s * s, complex=True)
    ridb = ref.exp_max_ext(s, s, rb.data_ptr(), s, batch, s * s, complex=True)
    assert handle.get_max_exp(ida) == ref.max_exp(rida)
    assert handle.get_max_exp(idb) == ref.max_exp(ridb)
    assert ref.flag(1) == (FP16TCEC | 0x60) == _flag_word(handle, 1)
    assert ref.flag(0) == TF32TCEC == _flag_word(handle, 0)
    handle.scale_A(ida, 1, s, s, da, s, batch, s * s)
    handle.scale_B(idb, 1, s, s, db, s, batch, s * s)
    handle.scale_C(ida, idb, 1, s, s, dc, s, batch, s * s)
    ref.scale(SCALE_A, s, s, ra.data_ptr(), s, batch, s * s, rida, 0, 1, complex=True)
    ref.scale(SCALE_B, s, s, rb.data_ptr(), s, batch, s * s, ridb, 0, 1, complex=True)
    ref.scale(SCALE_C, s, s, rc.data_ptr(), s, batch, s * s, rida, ridb, 1, complex=True)
    torch.cuda.synchronize()
    assert torch.equal(torch.view_as_real(da), torch.view_as_real(ra))
    assert torch.equal(torch.view_as_real(db), torch.view_as_real(rb))
    assert torch.equal(torch.view_as_real(dc), torch.view_as_real(rc))
    handle.reset_scale_A(ida, 1, s, s, da, s, batch, s * s)
    ref.scale(RESET_A, s, s, ra.data_ptr(), s, batch, s * s, rida, 0, 1, complex=True)
    torch.cuda.synchronize()
    assert torch.equal(torch.view_as_real(da), torch.view_as_real(ra))
