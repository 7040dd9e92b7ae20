"""The GEMM kernel that splits its FP32 operands on the fly (tcec_gemm_fused.cu), forced on with
CUMPSGEMM_FUSED=1 and compared, through the C ABI, with the FP64 oracle and with the two-kernel
(pre-split) path on the same inputs.

The reference splits at fragment load inside its GEMM kernels
(src/device_tcec_wrapper.hpp:72-80); both paths here feed the tensor core the same hi / lo
bits, only the lengths of the accumulation chunks differ, so the two results agree far inside
the pass criterion residual < 2^-23 * sqrt(K) (test/main.cu:68-74).
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N, T, Cj = 0, 1, 2
FP16TCEC, TF32TCEC, SCALING = 1, 2, 11


def _dev(x):
    import torch

    return torch.from_numpy(x).cuda()


class _Fused:
    """CUMPSGEMM_FUSED (and optionally CUMPSGEMM_TILE_N) set for the duration of a block."""

    def __init__(self, handle, value, tile_n=None):
        self.handle, self.value, self.tile_n = handle, value, tile_n

    def __enter__(self):
        os.environ["CUMPSGEMM_FUSED"] = self.value
        if self.tile_n is not None:
            os.environ["CUMPSGEMM_TILE_N"] = str(self.tile_n)
        self.handle.reload_tuning_env()

    def __exit__(self, *exc):
        os.environ.pop("CUMPSGEMM_FUSED", None)
        os.environ.pop("CUMPSGEMM_TILE_N", None)
        self.handle.reload_tuning_env()


def _both_paths(handle, call, c0):
    """Run `call(c)` with the on-the-fly split forced on and forced off."""
    outs = []
    for value in ("1", "0"):
        c = _dev(c0.copy())
        with _Fused(handle, value):
            call(c)
        outs.append(c.cpu().numpy())
    return outs


def _close(x, y, ld, tol=2e-6):
    """Relative Frobenius distance of two results (flat column-major storage)."""
    xv, yv = x.view(np.float32).astype(np.float64), y.view(np.float32).astype(np.float64)
    return np.sqrt(((xv - yv) ** 2).sum() / max((yv ** 2).sum(), 1e-300)) < tol


@pytest.mark.parametrize("op_a", [N, T])
@pytest.mark.parametrize("op_b", [N, T])
@pytest.mark.parametrize("shape", [(256, 256, 256, 0), (200, 300, 100, 4), (129, 257, 65, 8),
                                   (1024, 896, 520, 0), (64, 48, 7, 4), (3, 5, 1, 0)])
def test_real_ops_and_ragged_shapes(handle, oracle, op_a, op_b, shape):
    m, n, k, pad = shape
    am, an = (m, k) if op_a == N else (k, m)
    bm, bn = (k, n) if op_b == N else (n, k)
    # leading dimensions: multiples of 4 floats so that the on-the-fly path is applicable
    lda, ldb, ldc = -(-am // 4) * 4 + pad, -(-bm // 4) * 4 + pad, m + 3
    a = oracle.gen_uniform_exp(m + n, lda * an, -6, 6)
    b = oracle.gen_uniform_exp(m + n + 1, ldb * bn, -6, 6)
    c0 = oracle.gen_uniform(m + n + 2, ldc * n)
    da, db = _dev(a), _dev(b)
    fused, split = _both_paths(
        handle, lambda c: handle.gemm(op_a, op_b, m, n, k, -1.25, da, lda, db, ldb, 0.75, c, ldc,
                                      FP16TCEC), c0)
    truth = oracle.gemm_f64(op_a, op_b, m, n, k, -1.25, a, lda, b, ldb, 0.75, c0, ldc)
    thr = oracle.error_threshold(True, max(k, 16))
    assert oracle.residual(truth, fused, ldc) < thr
    assert oracle.residual(truth, split, ldc) < thr
    assert _close(fused, split, ldc)
    # rows of C between m and ldc are not touched
    got = fused.reshape((ldc, n), order="F")
    np.testing.assert_array_equal(got[m:], c0.reshape((ldc, n), order="F")[m:])


def test_long_k_several_drain_chunks(handle, oracle):
    """K = 2600: 41 stages, a first chunk of 4 stages and 19 more drains per tile."""
    m, n, k = 300, 260, 2600
    a, b = oracle.gen_uniform(1, m * k), oracle.gen_uniform(2, k * n)
    c0 = oracle.gen_uniform(3, m * n)
    da, db = _dev(a), _dev(b)
    fused, split = _both_paths(
        handle, lambda c: handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.5, c, m, FP16TCEC), c0)
    truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c0, m)
    assert oracle.residual(truth, fused, m) < oracle.error_threshold(True, k)
    assert _close(fused, split, m)
    c32 = c0.copy()
    oracle.gemm_f32(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c32, m)
    assert oracle.residual(truth, fused, m) <= 1.5 * oracle.residual(truth, c32, m)


@pytest.mark.parametrize("tile_n", [128, 64])
def test_strided_batches_more_tiles_than_sms(handle, oracle, tile_n):
    """Real batches: 40 x (260 x 200 x 130) = 240 (128-wide) or 480 (64-wide) tiles on 148
    persistent CTAs, so CTAs walk several tiles, with gaps between the batch entries."""
    import torch

    batch, m, n, k = 40, 260, 200, 132
    lda, ldb, ldc = 264, 132, 260
    sa, sb, sc = lda * k + 8, ldb * n + 4, ldc * n + 1
    a = oracle.gen_uniform(5, sa * batch)
    b = oracle.gen_uniform(6, sb * batch)
    c0 = oracle.gen_uniform(7, sc * batch)
    da, db, dc = _dev(a), _dev(b), _dev(c0.copy())
    with _Fused(handle, "1", tile_n):
        handle.gemm_strided_batch(N, N, m, n, k, 1.5, da, lda, sa, db, ldb, sb, -0.5, dc, ldc, sc,
                                  batch, FP16TCEC)
    res = dc.cpu().numpy()
    for i in range(batch):
        truth = oracle.gemm_f64(N, N, m, n, k, 1.5, a[i * sa:], lda, b[i * sb:], ldb, -0.5,
                                c0[i * sc:], ldc)
        assert oracle.residual(truth, res[i * sc:i * sc + ldc * n], ldc) < \
            oracle.error_threshold(True, k)
    assert handle.kernel_status() == 0


def test_complex_batches_with_on_the_fly_expansion(handle, oracle):
    """Complex N/N strided batch (the state-vector contraction shape, reduced): A is expanded
    to [[re, -im], [im, re]] inside the converter, complex alpha and beta in the epilogue."""
    import torch

    batch, m, n, k = 24, 130, 96, 70
    lda, ldb, ldc = 132, 70, 131
    sa, sb, sc = lda * k, ldb * n, ldc * n

    def cgen(s, count):
        return (oracle.gen_uniform(s, count) + 1j * oracle.gen_uniform(s + 50, count)).astype(np.complex64)

    za, zb, zc0 = cgen(1, sa * batch), cgen(2, sb * batch), cgen(3, sc * batch)
    da, db = _dev(za), _dev(zb)
    alpha, beta = 0.5 - 1.5j, -0.25 + 2j
    fused, split = _both_paths(
        handle, lambda c: handle.gemm_strided_batch(N, N, m, n, k, alpha, da, lda, sa, db, ldb, sb,
                                                    beta, c, ldc, sc, batch, FP16TCEC), zc0)
    for i in range(batch):
        truth = oracle.gemm_f64(N, N, m, n, k, alpha, za[i * sa:], lda, zb[i * sb:], ldb, beta,
                                zc0[i * sc:], ldc)
        assert oracle.residual(truth, fused[i * sc:(i + 1) * sc], ldc) < oracle.error_threshold(True, k)
    assert _close(fused, split, ldc)


def test_config4_shape_with_scaling(handle, oracle):
    """512 x complex 256^3 reduced to 64 batches, unit-Frobenius operands, FP16TCEC_SCALING: the
    scale factors are applied inside the converter, the un-scaling in the epilogue; equal bits
    of hi / lo in both paths, so the results agree closely."""
    import torch

    batch, s = 64, 256
    za = oracle.gen_unit_frobenius_complex(1, batch, s, s)
    zb = oracle.gen_unit_frobenius_complex(2, batch, s, s)
    da, db = _dev(za), _dev(zb)
    zero = np.zeros(batch * s * s, dtype=np.complex64)
    fused, split = _both_paths(
        handle, lambda c: handle.gemm_strided_batch(N, N, s, s, s, 1.0, da, s, s * s, db, s, s * s,
                                                    0.0, c, s, s * s, batch, SCALING), zero)
    thr = oracle.error_threshold(True, s)
    for i in (0, 17, batch - 1):
        truth = oracle.gemm_f64(N, N, s, s, s, 1.0, za[i * s * s:], s, zb[i * s * s:], s, 0.0, None, s)
        assert oracle.residual(truth, fused[i * s * s:(i + 1) * s * s], s) < thr
    assert _close(fused, split, s)


def test_scale_factors_reach_the_converter(handle, oracle):
    """Tiny magnitudes: the lo parts underflow FP16 unless the operands are scaled first.  With
    the on-the-fly split forced on, FP16TCEC_SCALING is accurate and plain FP16TCEC is not."""
    import torch

    m = n = k = 512
    a = (oracle.gen_uniform(1, m * k) * np.float32(2.0 ** -26)).astype(np.float32)
    b = (oracle.gen_uniform(2, k * n) * np.float32(2.0 ** -22)).astype(np.float32)
    da, db = _dev(a), _dev(b)
    truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m, b, k, 0.0, None, m)
    with _Fused(handle, "1"):
        good = torch.zeros(m * n, device="cuda")
        handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.0, good, m, SCALING)
        plain = torch.zeros(m * n, device="cuda")
        handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.0, plain, m, FP16TCEC)
    assert oracle.residual(truth, good.cpu().numpy(), m) < oracle.error_threshold(True, k)
    assert oracle.residual(truth, plain.cpu().numpy(), m) > 10 * oracle.error_threshold(True, k)
    np.testing.assert_array_equal(da.cpu().numpy(), a)


def test_inapplicable_calls_fall_back(handle, oracle):
    """Unaligned leading dimension, transposed complex operands and TF32TCEC are not handled by
    the converters: with the on-the-fly path forced on such calls still give the right result
    (through the pre-split path)."""
    m, n, k = 130, 90, 77
    a, b = oracle.gen_uniform(1, (m + 1) * k), oracle.gen_uniform(2, (k + 3) * n)
    da, db = _dev(a), _dev(b)
    import torch

    with _Fused(handle, "1"):
        c = torch.zeros(m * n, device="cuda")
        handle.gemm(N, N, m, n, k, 1.0, da, m + 1, db, k + 3, 0.0, c, m, FP16TCEC)
        truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m + 1, b, k + 3, 0.0, None, m)
        assert oracle.residual(truth, c.cpu().numpy(), m) < oracle.error_threshold(True, k)
        c = torch.zeros(m * n, device="cuda")
        handle.gemm(N, N, m, n, k, 1.0, da, m + 1, db, k + 3, 0.0, c, m, TF32TCEC)
        assert oracle.residual(truth, c.cpu().numpy(), m) < oracle.error_threshold(True, k)
        za = (oracle.gen_uniform(3, k * m) + 1j * oracle.gen_uniform(4, k * m)).astype(np.complex64)
        zb = (oracle.gen_uniform(5, k * n) + 1j * oracle.gen_uniform(6, k * n)).astype(np.complex64)
        zc = torch.zeros(m * n, dtype=torch.complex64, device="cuda")
        handle.gemm(Cj, N, m, n, k, 1.0, _dev(za), k, _dev(zb), k, 0.0, zc, m, FP16TCEC)
        truth = oracle.gemm_f64(Cj, N, m, n, k, 1.0, za, k, zb, k, 0.0, None, m)
        assert oracle.residual(truth, zc.cpu().numpy(), m) < oracle.error_threshold(True, k)
    assert handle.kernel_status() == 0


def test_run_to_run_determinism(handle, oracle):
    import torch

    m, n, k = 700, 520, 300
    a, b = _dev(oracle.gen_uniform(1, m * k)), _dev(oracle.gen_uniform(2, k * n))
    c1 = torch.zeros(m * n, device="cuda")
    c2 = torch.zeros(m * n, device="cuda")
    with _Fused(handle, "1"):
        handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c1, m, FP16TCEC)
        handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c2, m, FP16TCEC)
    assert torch.equal(c1, c2)


@pytest.mark.parametrize("case", ["real_tn", "real_nn_ragged", "complex", "scaling_batch"])
def test_split_k_inside_the_on_the_fly_kernel(handle, oracle, case):
    """Few tiles and a long K loop on the on-the-fly route: the kernel's K loop is cut into
    slices over the SMs, every slice writes plain partial sums, the reduction kernel adds them
    in ascending order and applies alpha, beta (complex too) and the un-scaling.  Reported as
    module 100, bit-identical from run to run, inside the pass criterion, and the default rule
    takes this route by itself for a handful of tiles with k >= 8192."""
    import torch

    if case == "real_tn":
        m, n, k, op_a = 256, 128, 8192 + 64, T
        a, b = oracle.gen_uniform(1, m * k), oracle.gen_uniform(2, k * n)
        c0 = oracle.gen_uniform(3, m * n)
        da, db = _dev(a), _dev(b)
        truth = oracle.gemm_f64(op_a, N, m, n, k, 1.5, a, k, b, k, -0.5, c0, m)
        outs = []
        for rep in range(2):
            dc = _dev(c0.copy())
            st, mod = handle.gemm_module(op_a, N, m, n, k, 1.5, da, k, db, k, -0.5, dc, m, FP16TCEC)
            assert st == 0 and mod == 100          # the default rule, nothing forced
            outs.append(dc)
        assert torch.equal(outs[0], outs[1])
        assert oracle.residual(truth, outs[0].cpu().numpy(), m) < oracle.error_threshold(True, k)
        _, split = _both_paths(
            handle, lambda c: handle.gemm(op_a, N, m, n, k, 1.5, da, k, db, k, -0.5, c, m, FP16TCEC), c0)
        assert _close(outs[0].cpu().numpy(), split, m)
    elif case == "real_nn_ragged":
        m, n, k = 200, 72, 2500                    # forced: edge tiles, K not a multiple of 64
        lda, ldb, ldc = 200, 2500, 203
        a, b = oracle.gen_uniform(4, lda * k), oracle.gen_uniform(5, ldb * n)
        c0 = oracle.gen_uniform(6, ldc * n)
        da, db = _dev(a), _dev(b)
        truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, lda, b, ldb, 0.25, c0, ldc)
        with _Fused(handle, "1"):
            dc = _dev(c0.copy())
            st, mod = handle.gemm_module(N, N, m, n, k, 1.0, da, lda, db, ldb, 0.25, dc, ldc, FP16TCEC)
            assert st == 0 and mod == 100
        assert oracle.residual(truth, dc.cpu().numpy(), ldc) < oracle.error_threshold(True, k)
    elif case == "complex":
        m, n, k = 96, 64, 4100
        gen = lambda s, cnt: (oracle.gen_uniform(s, cnt) + 1j * oracle.gen_uniform(s + 50, cnt)).astype(np.complex64)
        a, b, c0 = gen(7, m * k), gen(8, k * n), gen(9, m * n)
        da, db = _dev(a), _dev(b)
        alpha, beta = 0.5 - 1.5j, -0.25 + 2j
        truth = oracle.gemm_f64(N, N, m, n, k, alpha, a, m, b, k, beta, c0, m)
        with _Fused(handle, "1"):
            dc = _dev(c0.copy())
            assert handle.gemm(N, N, m, n, k, alpha, da, m, db, k, beta, dc, m, FP16TCEC) == 0
        assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
    else:
        batch, m, n, k = 3, 128, 128, 2048         # tiny operands: the un-scaling is the reduction's
        a = (oracle.gen_uniform(10, batch * m * k) * np.float32(2.0 ** -24)).astype(np.float32)
        b = (oracle.gen_uniform(11, batch * k * n) * np.float32(2.0 ** -20)).astype(np.float32)
        c0 = np.zeros(batch * m * n, dtype=np.float32)
        da, db = _dev(a), _dev(b)
        with _Fused(handle, "1"):
            dc = _dev(c0.copy())
            assert handle.gemm_strided_batch(T, N, m, n, k, 1.0, da, k, m * k, db, k, k * n, 0.0, dc,
                                             m, m * n, batch, SCALING) == 0
        res = dc.cpu().numpy()
        for i in range(batch):
            truth = oracle.gemm_f64(T, N, m, n, k, 1.0, a[i * m * k:], k, b[i * k * n:], k, 0.0,
                                    c0[i * m * n:], m)
            assert oracle.residual(truth, res[i * m * n:(i + 1) * m * n], m) < \
                oracle.error_threshold(True, k)
    assert handle.kernel_status() == 0
