"""Parity of the CUDA GEMM path (through the C ABI) with the FP64 oracle.

Pass criterion for the error-corrected modes is the reference's own:
relative Frobenius residual against FP64 below 2^-23 * sqrt(K)
(test/main.cu:68-74, 372-375); the non-corrected modes use 2^-10 * sqrt(K).
On top of it the benchmark's stated bar is checked: mean relative error at most
1e-6 for well-scaled inputs and errors no worse than an FP32 GEMM's.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N, T, Cj = 0, 1, 2
FP16TCEC, TF32TCEC, FP16TC, TF32TC, DRY_RUN, AUTO, SCALING = 1, 2, 3, 4, 8, 9, 11


def _torch():
    import torch

    return torch


def _dev(x):
    return _torch().from_numpy(x).cuda()


def _run_real(handle, oracle, op_a, op_b, m, n, k, mode, alpha=1.0, beta=0.0, pad=(0, 0, 0),
              seed=0, gen=None):
    gen = gen or oracle.gen_uniform
    am, an = (m, k) if op_a == N else (k, m)
    bm, bn = (k, n) if op_b == N else (n, k)
    lda, ldb, ldc = am + pad[0], bm + pad[1], m + pad[2]
    a = gen(seed, lda * an)
    b = gen(seed + 1, ldb * bn)
    c0 = oracle.gen_uniform(seed + 2, ldc * n)
    da, db, dc = _dev(a), _dev(b), _dev(c0.copy())
    handle.gemm(op_a, op_b, m, n, k, alpha, da, lda, db, ldb, beta, dc, ldc, mode)
    res = dc.cpu().numpy()
    truth = oracle.gemm_f64(op_a, op_b, m, n, k, alpha, a, lda, b, ldb, beta, c0, ldc)
    return a, b, c0, res, truth, (lda, ldb, ldc)


def test_config1_sgemm_1024_fp16tcec(handle, oracle):
    """Benchmark config 1: m=n=k=1024, NN, alpha=1, beta=0, uniform(-1,1), seed 0."""
    m = n = k = 1024
    a, b, c0, res, truth, _ = _run_real(handle, oracle, N, N, m, n, k, FP16TCEC, seed=0)
    r = oracle.residual(truth, res, m)
    assert r < oracle.error_threshold(True, k)
    c32 = np.zeros(m * n, dtype=np.float32)
    oracle.gemm_f32(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c32, m)
    mx, mean = oracle.relative_errors(truth, res, m)
    mx32, mean32 = oracle.relative_errors(truth, c32, m)
    assert mean <= 1e-6
    assert mean <= 1.5 * mean32          # no worse than FP32 SIMT on the same inputs
    assert r <= 1.5 * oracle.residual(truth, c32, m)


def test_reference_input_distribution_normal(handle, oracle):
    """The reference's own test inputs: N(0,1) (test/main.cu:552-558)."""
    m = n = k = 512
    for mode in (FP16TCEC, TF32TCEC):
        _, _, _, res, truth, _ = _run_real(handle, oracle, N, N, m, n, k, mode, seed=3,
                                           gen=oracle.gen_normal)
        assert oracle.residual(truth, res, m) < oracle.error_threshold(True, k)


@pytest.mark.parametrize("mode", [FP16TCEC, TF32TCEC])
def test_config2_row_2048(handle, oracle, mode):
    """Benchmark config 2 at N=2048: inputs u*2^e, e in [-8,8]; alpha=1, beta=0.5."""
    m = n = k = 2048
    a, b, c0, res, truth, _ = _run_real(handle, oracle, N, N, m, n, k, mode, beta=0.5, seed=1,
                                        gen=oracle.gen_uniform_exp)
    r = oracle.residual(truth, res, m)
    assert r < oracle.error_threshold(True, k)
    c32 = c0.copy()
    oracle.gemm_f32(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c32, m)
    assert r <= 1.5 * oracle.residual(truth, c32, m)


@pytest.mark.parametrize("op_a", [N, T])
@pytest.mark.parametrize("op_b", [N, T])
@pytest.mark.parametrize("mode", [FP16TCEC, TF32TCEC])
def test_sgemm_ops_and_ragged_shapes(handle, oracle, op_a, op_b, mode):
    for (m, n, k, pad) in [(200, 300, 100, (0, 0, 0)), (129, 257, 65, (3, 5, 7)), (64, 64, 64, (1, 1, 1))]:
        _, _, _, res, truth, ld = _run_real(handle, oracle, op_a, op_b, m, n, k, mode, alpha=-1.25,
                                            beta=0.75, pad=pad, seed=m + n)
        assert oracle.residual(truth, res[: ld[2] * n].reshape(-1), ld[2]) < \
            oracle.error_threshold(True, k)
        # rows between m and ldc must be untouched
        if pad[2]:
            c0 = oracle.gen_uniform(m + n + 2, ld[2] * n).reshape((ld[2], n), order="F")
            got = res.reshape((ld[2], n), order="F")
            np.testing.assert_array_equal(got[m:], c0[m:])


@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 513, 7), (300, 1, 33), (5, 3, 1), (127, 63, 4097)])
def test_sgemm_degenerate_shapes(handle, oracle, shape):
    m, n, k = shape
    _, _, _, res, truth, _ = _run_real(handle, oracle, N, T, m, n, k, FP16TCEC, beta=1.0, seed=11)
    assert oracle.residual(truth, res, m) < oracle.error_threshold(True, max(k, 16))


@pytest.mark.parametrize("tile", [64, 128, 256, "256-single-cta"])
def test_every_tile_width(handle, oracle, tile):
    """All kernel variants: 128x64, 128x128, 256x256 on CTA pairs, 128x256 on one CTA."""
    if tile == "256-single-cta":
        tile = 256
        os.environ["CUMPSGEMM_PAIR"] = "0"
    os.environ["CUMPSGEMM_TILE_N"] = str(tile)
    handle.reload_tuning_env()
    try:
        m, n, k = 384, 520, 200
        _, _, _, res, truth, _ = _run_real(handle, oracle, N, N, m, n, k, FP16TCEC, beta=0.5, seed=5)
        assert oracle.residual(truth, res, m) < oracle.error_threshold(True, k)
        _, _, _, res, truth, _ = _run_real(handle, oracle, T, N, m, n, k, TF32TCEC, seed=6)
        assert oracle.residual(truth, res, m) < oracle.error_threshold(True, k)
        r = _run_complex(handle, oracle, Cj, N, 130, 300, 70, FP16TCEC, 1.0 - 1.0j, 0.5j, seed=8)
        assert r < oracle.error_threshold(True, 70)
    finally:
        os.environ.pop("CUMPSGEMM_TILE_N", None)
        os.environ.pop("CUMPSGEMM_PAIR", None)


def test_tile_choice_is_reported(handle, oracle):
    torch = _torch()
    big = torch.zeros(4096 * 4096, device="cuda")
    st, mod = handle.gemm_module(N, N, 4096, 4096, 64, 1.0, big, 4096, big, 64, 0.0, big, 4096,
                                 FP16TCEC)
    assert st == 0 and mod == 0          # 128x256 tiles fill the GPU
    st, mod = handle.gemm_module(N, N, 128, 128, 64, 1.0, big, 128, big, 64, 0.0, big, 128, FP16TCEC)
    assert st == 0 and mod == 2          # a single small problem takes the narrow tile


def _run_complex(handle, oracle, op_a, op_b, m, n, k, mode, alpha, beta, seed=0, pad=0):
    am, an = (m, k) if op_a == N else (k, m)
    bm, bn = (k, n) if op_b == N else (n, k)
    lda, ldb, ldc = am + pad, bm + pad, m + pad

    def cgen(s, count):
        return (oracle.gen_uniform(s, count) + 1j * oracle.gen_uniform(s + 100, count)).astype(np.complex64)

    a, b, c0 = cgen(seed, lda * an), cgen(seed + 1, ldb * bn), cgen(seed + 2, ldc * n)
    da, db, dc = _dev(a), _dev(b), _dev(c0.copy())
    handle.gemm(op_a, op_b, m, n, k, alpha, da, lda, db, ldb, beta, dc, ldc, mode)
    truth = oracle.gemm_f64(op_a, op_b, m, n, k, alpha, a, lda, b, ldb, beta, c0, ldc)
    return oracle.residual(truth, dc.cpu().numpy(), ldc)


@pytest.mark.parametrize("op_a", [N, T, Cj])
@pytest.mark.parametrize("op_b", [N, T, Cj])
def test_cgemm_all_op_pairs(handle, oracle, op_a, op_b):
    """The reference tests {N,T,C}^2 for complex (test/main.cu:539-629)."""
    for mode in (FP16TCEC, TF32TCEC):
        r = _run_complex(handle, oracle, op_a, op_b, 70, 90, 50, mode, 1.0, 0.0, seed=op_a * 3 + op_b)
        assert r < oracle.error_threshold(True, 50)
    r = _run_complex(handle, oracle, op_a, op_b, 33, 65, 129, FP16TCEC, 0.5 - 1.5j, -0.25 + 2j,
                     seed=9, pad=3)
    assert r < oracle.error_threshold(True, 129)


def test_cgemm_square_256(handle, oracle):
    """Per-batch shape of benchmark config 4 (complex 256^3)."""
    r = _run_complex(handle, oracle, N, N, 256, 256, 256, FP16TCEC, 1.0, 0.0, seed=21)
    assert r < oracle.error_threshold(True, 256)


@pytest.mark.parametrize("mode", [FP16TC, TF32TC])
def test_uncorrected_modes(handle, oracle, mode):
    m = n = k = 256
    _, _, _, res, truth, _ = _run_real(handle, oracle, N, N, m, n, k, mode, seed=2)
    r = oracle.residual(truth, res, m)
    assert r < oracle.error_threshold(False, k)
    assert r > 1e-6                      # really is the uncorrected arithmetic


def test_strided_batch_sgemm_and_cgemm(handle, oracle):
    torch = _torch()
    batch, m, n, k = 5, 96, 130, 70
    sa, sb, sc = m * k + 8, k * n + 4, m * n
    a = oracle.gen_uniform(1, sa * batch)
    b = oracle.gen_uniform(2, sb * batch)
    c0 = oracle.gen_uniform(3, sc * batch)
    da, db, dc = _dev(a), _dev(b), _dev(c0.copy())
    handle.gemm_strided_batch(N, N, m, n, k, 2.0, da, m, sa, db, k, sb, 0.5, dc, m, sc, batch,
                              FP16TCEC)
    res = dc.cpu().numpy()
    for i in range(batch):
        truth = oracle.gemm_f64(N, N, m, n, k, 2.0, a[i * sa:], m, b[i * sb:], k, 0.5, c0[i * sc:], m)
        assert oracle.residual(truth, res[i * sc:(i + 1) * sc], m) < oracle.error_threshold(True, k)
    # chunked workspace: same numbers when the batch is processed in pieces
    handle.set_workspace_limit(1 << 20)
    dc2 = _dev(c0.copy())
    handle.gemm_strided_batch(N, N, m, n, k, 2.0, da, m, sa, db, k, sb, 0.5, dc2, m, sc, batch,
                              FP16TCEC)
    handle.set_workspace_limit(0)
    assert torch.equal(dc, dc2)
    # complex batch, stride 0 on B (one matrix shared by every batch)
    za = (oracle.gen_uniform(4, m * k * batch) + 1j * oracle.gen_uniform(5, m * k * batch)).astype(np.complex64)
    zb = (oracle.gen_uniform(6, k * n) + 1j * oracle.gen_uniform(7, k * n)).astype(np.complex64)
    dza, dzb = _dev(za), _dev(zb)
    dzc = torch.zeros(m * n * batch, dtype=torch.complex64, device="cuda")
    handle.gemm_strided_batch(N, N, m, n, k, 1.0, dza, m, m * k, dzb, k, 0, 0.0, dzc, m, m * n,
                              batch, TF32TCEC)
    zres = dzc.cpu().numpy()
    for i in range(batch):
        truth = oracle.gemm_f64(N, N, m, n, k, 1.0, za[i * m * k:], m, zb, k, 0.0, None, m)
        assert oracle.residual(truth, zres[i * m * n:(i + 1) * m * n], m) < oracle.error_threshold(True, k)


@pytest.mark.parametrize("mode", [FP16TCEC, TF32TCEC])
def test_pair_kernel_ragged_multiwave_batched(handle, oracle, mode):
    """The persistent CTA-pair kernel where all of its scheduling features are active at once:
    more tiles than cluster slots (several waves, paced), a K loop long enough for the longer
    first drain chunk, m / n / k that are not multiples of the tile, padded leading dimensions,
    beta != 0, a batch of two, and the same for complex operands."""
    torch = _torch()
    batch, m, n, k = 4, 612, 2381, 2088          # 3 x 10 pair tiles per entry: 120 on 74 slots
    os.environ["CUMPSGEMM_TILE_N"] = "256"       # force the pair kernel whatever the tile rule says
    os.environ["CUMPSGEMM_PAIR"] = "1"
    handle.reload_tuning_env()
    try:
        lda, ldb, ldc = m + 4, k + 8, m + 12
        sa, sb, sc = lda * k + 16, ldb * n + 4, ldc * n
        a = oracle.gen_uniform_exp(21, sa * batch, -4, 4)
        b = oracle.gen_uniform_exp(22, sb * batch, -4, 4)
        c0 = oracle.gen_uniform(23, sc * batch)
        da, db, dc = _dev(a), _dev(b), _dev(c0.copy())
        handle.gemm_strided_batch(N, N, m, n, k, 1.5, da, lda, sa, db, ldb, sb, -0.5, dc, ldc, sc,
                                  batch, mode)
        res = dc.cpu().numpy()
        for i in range(batch):
            truth = oracle.gemm_f64(N, N, m, n, k, 1.5, a[i * sa:], lda, b[i * sb:], ldb, -0.5,
                                    c0[i * sc:], ldc)
            assert oracle.residual(truth, res[i * sc:(i + 1) * sc], ldc) < oracle.error_threshold(True, k)
            # rows of C beyond m (padding of the leading dimension) are untouched
            pad_got = res[i * sc:(i + 1) * sc].reshape(n, ldc)[:, m:]
            pad_was = c0[i * sc:(i + 1) * sc].reshape(n, ldc)[:, m:]
            assert np.array_equal(pad_got, pad_was)
        # complex, transposed / conjugated operands
        mz, nz, kz = 330, 2330, 1100
        za = (oracle.gen_uniform(31, kz * mz) + 1j * oracle.gen_uniform(32, kz * mz)).astype(np.complex64)
        zb = (oracle.gen_uniform(33, nz * kz) + 1j * oracle.gen_uniform(34, nz * kz)).astype(np.complex64)
        zc0 = (oracle.gen_uniform(35, mz * nz) + 1j * oracle.gen_uniform(36, mz * nz)).astype(np.complex64)
        dza, dzb, dzc = _dev(za), _dev(zb), _dev(zc0.copy())
        handle.gemm(Cj, T, mz, nz, kz, 1.0 - 0.5j, dza, kz, dzb, nz, 0.25 + 0.5j, dzc, mz, mode)
        truth = oracle.gemm_f64(Cj, T, mz, nz, kz, 1.0 - 0.5j, za, kz, zb, nz, 0.25 + 0.5j, zc0, mz)
        assert oracle.residual(truth, dzc.cpu().numpy(), mz) < oracle.error_threshold(True, kz)
        assert handle.kernel_status() == 0
    finally:
        os.environ.pop("CUMPSGEMM_TILE_N", None)
        os.environ.pop("CUMPSGEMM_PAIR", None)


def test_beta_zero_ignores_nan_in_c(handle, oracle):
    torch = _torch()
    m = n = k = 128
    a, b = _dev(oracle.gen_uniform(1, m * k)), _dev(oracle.gen_uniform(2, k * n))
    c = torch.full((m * n,), float("nan"), device="cuda")
    handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c, m, FP16TCEC)
    assert torch.isfinite(c).all()


def test_dry_run_and_argument_errors(handle, oracle):
    from cumpsgemm_b200 import api

    torch = _torch()
    m = n = k = 64
    a = torch.ones(m * k, device="cuda")
    c = torch.full((m * n,), 7.0, device="cuda")
    assert handle.gemm(N, N, m, n, k, 1.0, a, m, a, k, 0.0, c, m, DRY_RUN) == 0
    assert (c == 7.0).all()
    inv = api.CUBLAS_STATUS_INVALID_VALUE
    assert handle.gemm(N, N, 0, n, k, 1.0, a, m, a, k, 0.0, c, m, FP16TCEC, check=False) == inv
    assert handle.gemm(N, N, m, n, k, 1.0, a, m - 1, a, k, 0.0, c, m, FP16TCEC, check=False) == inv
    assert handle.gemm(Cj, N, m, n, k, 1.0, a, m, a, k, 0.0, c, m, FP16TCEC, check=False) == inv
    assert handle.gemm(N, N, m, n, k, 1.0, a, m, a, k, 0.0, c, m, 0, check=False) == \
        api.CUBLAS_STATUS_NOT_SUPPORTED
    assert (c == 7.0).all()


def test_power_of_two_scaling_commutes_bitwise(handle, oracle):
    """Size-independent property: scaling A by 2^p scales C by 2^p exactly, as long as no lo
    part leaves the FP16 normal range (inputs in [1, 3) keep every non-zero lo >= 2^-12)."""
    torch = _torch()
    m = n = k = 1024
    a = _dev(oracle.gen_uniform(1, m * k) + np.float32(2.0))
    b = _dev(oracle.gen_uniform(2, k * n) + np.float32(2.0))
    c1 = torch.zeros(m * n, device="cuda")
    c2 = torch.zeros(m * n, device="cuda")
    for mode in (FP16TCEC, TF32TCEC):
        handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c1, m, mode)
        handle.gemm(N, N, m, n, k, 1.0, a * 4.0, m, b * 0.5, k, 0.0, c2, m, mode)
        assert torch.equal(c1 * 2.0, c2)
        handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c2, m, mode)   # run-to-run determinism
        assert torch.equal(c1, c2)


@pytest.mark.parametrize("n", [8192])
def test_large_size_against_sampled_fp64(handle, oracle, n):
    """Full-size check: FP64 truth on sampled rows of C (CPU oracle) plus bitwise properties."""
    torch = _torch()
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    a = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
    b = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
    c0 = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
    c = c0.clone()
    handle.gemm(N, N, n, n, n, 1.0, a, n, b, n, 0.5, c, n, FP16TCEC)
    ah, bh, c0h, ch = (x.cpu().numpy() for x in (a, b, c0, c))
    rows = [0, 1, 127, 128, n // 2 + 3, n - 1]
    for i in rows:
        # row i of C: op(A) restricted to one row = pointer offset i with the same lda
        truth = oracle.gemm_f64(N, N, 1, n, n, 1.0, ah[i:], n, bh, n, 0.5, c0h[i:], n)
        got = ch.reshape((n, n), order="F")[i].copy()
        assert oracle.residual(truth, got, 1) < oracle.error_threshold(True, n)
    cols = [0, 255, 256, n - 1]
    for j in cols:
        truth = oracle.gemm_f64(N, N, n, 1, n, 1.0, ah, n, bh[j * n:], n, 0.5, c0h[j * n:], n)
        assert oracle.residual(truth, ch[j * n:(j + 1) * n], n) < oracle.error_threshold(True, n)
    # whole-matrix cross-check against the GPU's own FP64 GEMM
    A = a.view(n, n).t().double()
    B = b.view(n, n).t().double()
    truth_gpu = (A @ B + 0.5 * c0.view(n, n).t().double())
    diff = (truth_gpu - c.view(n, n).t().double()).norm() / truth_gpu.norm()
    assert diff.item() < oracle.error_threshold(True, n)


def test_scheduling_aids_do_not_change_results(handle, oracle):
    """Wave pacing only delays tile starts and repeated calls take the same path: a GEMM with
    several waves of tiles per cluster and a long K loop gives the same bits with pacing on,
    with pacing off, and on a second call; the kernel's status word stays clear."""
    torch = _torch()
    m, n, k = 4096, 8192, 2560            # 512 pair tiles (about 7 waves), 40 K stages
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    a = torch.rand(m * k, device="cuda", generator=g) * 2 - 1
    b = torch.rand(k * n, device="cuda", generator=g) * 2 - 1
    c0 = torch.rand(m * n, device="cuda", generator=g) * 2 - 1
    outs = []
    old = os.environ.get("CUMPSGEMM_PACE")
    try:
        for pace in ("1", "0", "1"):
            os.environ["CUMPSGEMM_PACE"] = pace
            handle.reload_tuning_env()
            c = c0.clone()
            handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c, m, FP16TCEC)
            outs.append(c)
    finally:
        if old is None:
            os.environ.pop("CUMPSGEMM_PACE", None)
        else:
            os.environ["CUMPSGEMM_PACE"] = old
    assert handle.kernel_status() == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    # and the result is right: sampled columns against the FP64 oracle
    ah, bh, c0h, ch = (x.cpu().numpy() for x in (a, b, c0, outs[0]))
    for j in (0, 300, n - 1):
        truth = oracle.gemm_f64(N, N, m, 1, k, 1.0, ah, m, bh[j * k:], k, 0.5, c0h[j * m:], m)
        assert oracle.residual(truth, ch[j * m:(j + 1) * m], m) < oracle.error_threshold(True, k)


def test_calls_replay_from_a_cuda_graph(oracle):
    """After one warm-up call of the same shape (workspace, kernel attributes and occupancy
    queries are set up then) a GEMM call is launches and one 4-byte memset only, so it can be
    captured into a CUDA graph; replays give the bits of the direct call, also after the
    inputs changed in place."""
    torch = _torch()
    from cumpsgemm_b200 import api

    h = api.Handle()
    m, n, k = 2304, 2048, 2560      # more than one wave of pair tiles: paced pair kernel
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    a = torch.rand(m * k, device="cuda", generator=g) * 2 - 1
    b = torch.rand(k * n, device="cuda", generator=g) * 2 - 1
    c = torch.zeros(m * n, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        h.use_current_torch_stream()
        for mode in (FP16TCEC, TF32TCEC):
            h.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c, m, mode)       # warm-up
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for mode in (FP16TCEC, TF32TCEC):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            h.use_current_torch_stream()
            h.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c, m, mode)
        for scale in (1.0, 0.5):
            a.mul_(scale)
            graph.replay()
            torch.cuda.synchronize()
            replayed = c.clone()
            h.use_current_torch_stream()
            h.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c, m, mode)
            torch.cuda.synchronize()
            assert torch.equal(replayed, c)
    assert h.kernel_status() == 0
    h.destroy()


def test_two_handles_on_two_streams_at_once(oracle):
    """Two persistent GEMM kernels that share the GPU: the clusters of the second are not all
    resident while the first runs, so its pacing waits run out (and pacing switches itself off
    for that launch).  That may cost time, never correctness: both results equal the ones
    computed alone, bit for bit, and no bounded wait of the pipeline itself expires."""
    torch = _torch()
    from cumpsgemm_b200 import api

    m, n, k = 3072, 4096, 2304                    # 192 pair tiles, 36 K stages: paced
    g = torch.Generator(device="cuda")
    g.manual_seed(17)
    ops = []
    for _ in range(2):
        a = torch.rand(m * k, device="cuda", generator=g) * 2 - 1
        b = torch.rand(k * n, device="cuda", generator=g) * 2 - 1
        ops.append((a, b, torch.zeros(m * n, device="cuda"), torch.zeros(m * n, device="cuda")))
    handles = [api.Handle(), api.Handle()]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    # alone, one after the other
    for h, s, (a, b, c_alone, _) in zip(handles, streams, ops):
        with torch.cuda.stream(s):
            h.use_current_torch_stream()
            h.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c_alone, m, FP16TCEC)
        s.synchronize()
    # together, several rounds so that the launches really overlap
    for _ in range(4):
        for h, s, (a, b, _, c_both) in zip(handles, streams, ops):
            with torch.cuda.stream(s):
                h.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c_both, m, FP16TCEC)
    torch.cuda.synchronize()
    for h, (a, b, c_alone, c_both) in zip(handles, ops):
        assert torch.equal(c_alone, c_both)
        assert h.kernel_status() == 0
    ah, bh, ch = (x.cpu().numpy() for x in ops[1][:3])
    truth = oracle.gemm_f64(N, N, m, 1, k, 1.0, ah, m, bh[5 * k:], k, 0.0, None, m)
    assert oracle.residual(truth, ch[5 * m:6 * m], m) < oracle.error_threshold(True, k)
    for h in handles:
        h.destroy()


def test_handles_can_be_created_and_destroyed_repeatedly():
    """Create / use / destroy in a loop leaves device memory where it was (workspace, ring
    buffers and scratch are freed; reference leak: src/handle.cu:40-46)."""
    torch = _torch()
    from cumpsgemm_b200 import api

    x = torch.rand(512 * 512, device="cuda")
    y = torch.zeros(512 * 512, device="cuda")
    torch.cuda.synchronize()

    def cycle():
        h = api.Handle()
        h.use_current_torch_stream()
        h.gemm(N, N, 512, 512, 512, 1.0, x, 512, x, 512, 0.0, y, 512, FP16TCEC)
        h.exp_stats_ext(512, 512, x, 512)
        torch.cuda.synchronize()
        h.destroy()

    cycle()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(20):
        cycle()
    free_after = torch.cuda.mem_get_info()[0]
    assert free_before - free_after < (8 << 20), (free_before, free_after)


def test_host_buffer_gemm_pipelined_matches_resident(handle, oracle):
    """api.HostGemm (pinned host operands, column-block pipeline) against the resident call."""
    from cumpsgemm_b200 import api

    torch = _torch()
    m, n, k = 300, 1000, 260
    a, b, c0 = oracle.gen_uniform(1, m * k), oracle.gen_uniform(2, k * n), oracle.gen_uniform(3, m * n)
    ah, bh = torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()
    for blocks in (1, 7):
        ch = torch.from_numpy(c0.copy()).pin_memory()
        host = api.HostGemm(handle, column_blocks=blocks)
        h2d, d2h = host.gemm(N, N, m, n, k, 1.5, ah, m, bh, k, 0.5, ch, m, FP16TCEC)
        torch.cuda.synchronize()
        assert (h2d, d2h) == ((m * k + k * n + m * n) * 4, m * n * 4)
        truth = oracle.gemm_f64(N, N, m, n, k, 1.5, a, m, b, k, 0.5, c0, m)
        assert oracle.residual(truth, ch.numpy(), m) < oracle.error_threshold(True, k)
    handle.use_current_torch_stream()


def test_bounded_wait_gives_up_cleanly(handle, oracle):
    """Failure detection without a fault: a wait on a barrier nothing signals runs out after
    its limit, the status word carries the code, and the context keeps working."""
    torch = _torch()
    status, waited = handle.selftest_bounded_wait(200)
    assert status == 2                      # "MMA issuer waited for operands"
    assert 200.0 <= waited < 1000.0
    assert handle.kernel_status() == 0      # cleared by the read
    m = n = k = 128
    a, b = _dev(oracle.gen_uniform(1, m * k)), _dev(oracle.gen_uniform(2, k * n))
    c = torch.zeros(m * n, device="cuda")
    handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c, m, FP16TCEC)
    truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a.cpu().numpy(), m, b.cpu().numpy(), k, 0.0, None, m)
    assert oracle.residual(truth, c.cpu().numpy(), m) < oracle.error_threshold(True, k)


# ---------------------------------------------------------------- split-K
def _split_k_env(handle, value):
    if value is None:
        os.environ.pop("CUMPSGEMM_SPLIT_K", None)
    else:
        os.environ["CUMPSGEMM_SPLIT_K"] = str(value)
    handle.reload_tuning_env()


def test_split_k_small_c_long_k(handle, oracle):
    """Few tiles and a long K loop (the shapes the reference gives to its atomic split-K kernel,
    src/cumpsgemm.cu:272-304): K is cut into slices over many CTAs and the partial sums are
    added in a fixed order, so the result is right, reported as module 100, and bit-identical
    from run to run (the reference's atomics are not)."""
    torch = _torch()
    m, n, k = 256, 200, 65536
    a, b = oracle.gen_uniform(1, m * k), oracle.gen_uniform(2, k * n)
    c0 = oracle.gen_uniform(3, m * n)
    da, db = _dev(a), _dev(b)
    truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c0, m)
    outs = []
    try:
        for mode in (FP16TCEC, TF32TCEC):
            for rep in range(2):
                dc = _dev(c0.copy())
                st, mod = handle.gemm_module(N, N, m, n, k, 1.0, da, m, db, k, 0.5, dc, m, mode)
                assert st == 0 and mod == 100
                outs.append(dc)
            assert torch.equal(outs[-1], outs[-2])
            assert oracle.residual(truth, outs[-1].cpu().numpy(), m) < oracle.error_threshold(True, k)
        # no worse than an FP32 GEMM, and the unsplit path agrees
        c32 = c0.copy()
        oracle.gemm_f32(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c32, m)
        assert oracle.residual(truth, outs[0].cpu().numpy(), m) <= 1.5 * oracle.residual(truth, c32, m)
        _split_k_env(handle, 0)
        dc = _dev(c0.copy())
        st, mod = handle.gemm_module(N, N, m, n, k, 1.0, da, m, db, k, 0.5, dc, m, FP16TCEC)
        assert st == 0 and mod != 100
        assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
    finally:
        _split_k_env(handle, None)


@pytest.mark.parametrize("slices", [2, 3, 7])
def test_split_k_forced_uneven_slices_complex_and_batches(handle, oracle, slices):
    """Slice counts that do not divide the K loop, ragged sizes, complex alpha / beta (applied by
    the reduction kernel on interleaved rows), a strided batch, and FP16TCEC_SCALING (the
    un-scaling factor belongs to the reduction as well)."""
    torch = _torch()
    _split_k_env(handle, slices)
    try:
        r = _run_complex(handle, oracle, N, Cj, 70, 90, 333, FP16TCEC, 0.5 - 1.5j, -0.25 + 2j, seed=4,
                         pad=3)
        assert r < oracle.error_threshold(True, 333)
        batch, m, n, k = 3, 129, 65, 700
        a = oracle.gen_uniform(5, m * k * batch)
        b = oracle.gen_uniform(6, k * n * batch)
        c0 = oracle.gen_uniform(7, m * n * batch)
        for mode in (FP16TCEC, TF32TCEC):
            dc = _dev(c0.copy())
            handle.gemm_strided_batch(T, N, m, n, k, 2.0, _dev(a), k, m * k, _dev(b), k, k * n, -1.0,
                                      dc, m, m * n, batch, mode)
            res = dc.cpu().numpy()
            for i in range(batch):
                truth = oracle.gemm_f64(T, N, m, n, k, 2.0, a[i * m * k:], k, b[i * k * n:], k, -1.0,
                                        c0[i * m * n:], m)
                assert oracle.residual(truth, res[i * m * n:(i + 1) * m * n], m) < \
                    oracle.error_threshold(True, k)
        tiny_a = (oracle.gen_uniform(8, 200 * 512) * np.float32(2.0 ** -26)).astype(np.float32)
        tiny_b = (oracle.gen_uniform(9, 512 * 100) * np.float32(2.0 ** -22)).astype(np.float32)
        dc = torch.zeros(200 * 100, device="cuda")
        handle.gemm(N, N, 200, 100, 512, 1.0, _dev(tiny_a), 200, _dev(tiny_b), 512, 0.0, dc, 200,
                    SCALING)
        truth = oracle.gemm_f64(N, N, 200, 100, 512, 1.0, tiny_a, 200, tiny_b, 512, 0.0, None, 200)
        assert oracle.residual(truth, dc.cpu().numpy(), 200) < oracle.error_threshold(True, 512)
        assert handle.kernel_status() == 0
    finally:
        _split_k_env(handle, None)


class _PairEnv:
    """Force the CTA-pair kernel and set the tail-split switch for the calls inside."""

    def __init__(self, handle, tail_split):
        self.handle, self.tail_split = handle, tail_split

    def __enter__(self):
        os.environ["CUMPSGEMM_TILE_N"] = "256"
        os.environ["CUMPSGEMM_PAIR"] = "1"
        if self.tail_split is not None:
            os.environ["CUMPSGEMM_TAIL_SPLIT"] = str(self.tail_split)
        self.handle.reload_tuning_env()

    def __exit__(self, *exc):
        for name in ("CUMPSGEMM_TILE_N", "CUMPSGEMM_PAIR", "CUMPSGEMM_TAIL_SPLIT"):
            os.environ.pop(name, None)
        self.handle.reload_tuning_env()


@pytest.mark.parametrize("m,n,k", [(1024, 2048, 4096),    # 32 tiles, no full wave: every tile in two slices
                                   (3072, 1792, 2048),    # 84 tiles = one full wave + 10 split in two
                                   (512, 512, 8192 + 64)])  # 4 tiles in eight uneven slices
def test_pair_kernel_tail_split(handle, oracle, m, n, k):
    """The last, partly filled wave of CTA-pair tiles is cut into K slices that run on otherwise
    idle clusters; the CTA that finishes last adds the slices in ascending order.  The result is
    right, the same on every run, and differs from the unsplit one only by summation order."""
    torch = _torch()
    a, b = oracle.gen_uniform(31, m * k), oracle.gen_uniform(32, k * n)
    c0 = oracle.gen_uniform(33, m * n)
    da, db = _dev(a), _dev(b)
    truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m, b, k, 0.5, c0, m)
    for mode in (FP16TCEC, TF32TCEC):
        outs = []
        with _PairEnv(handle, None):
            for rep in range(3):
                dc = _dev(c0.copy())
                assert handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.5, dc, m, mode) == 0
                outs.append(dc)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        assert oracle.residual(truth, outs[0].cpu().numpy(), m) < oracle.error_threshold(True, k)
        with _PairEnv(handle, 0):
            dc = _dev(c0.copy())
            assert handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.5, dc, m, mode) == 0
        assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
        assert not torch.equal(dc, outs[0])          # the split really happened
        assert (dc - outs[0]).abs().max().item() < 1e-3
    assert handle.kernel_status() == 0


def test_pair_kernel_tail_split_complex_scaling_and_auto(handle, oracle):
    """Tail split with complex alpha / beta (the last CTA's epilogue works on the summed
    interleaved rows), with FP16TCEC_SCALING (un-scaling in that epilogue) and through the
    one-launch AUTO kernel (the split plan differs by kind)."""
    torch = _torch()
    with _PairEnv(handle, None):
        r = _run_complex(handle, oracle, N, N, 512, 2048, 1024, FP16TCEC, 0.5 - 1.5j, -0.25 + 2j, seed=41)
        assert r < oracle.error_threshold(True, 1024)
        m, n, k = 1024, 2048, 2048
        a = (oracle.gen_uniform(42, m * k) * np.float32(2.0 ** -20)).astype(np.float32)
        b = (oracle.gen_uniform(43, k * n) * np.float32(2.0 ** -18)).astype(np.float32)
        c0 = np.zeros(m * n, dtype=np.float32)
        truth = oracle.gemm_f64(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c0, m)
        da, db = _dev(a), _dev(b)
        dc = _dev(c0.copy())
        assert handle.gemm(N, N, m, n, k, 1.0, da, m, db, k, 0.0, dc, m, SCALING) == 0
        assert oracle.residual(truth, dc.cpu().numpy(), m) < oracle.error_threshold(True, k)
        for rep in range(2):
            dca = _dev(c0.copy())
            ia = handle.exp_stats_ext(m, k, da, m)
            ib = handle.exp_stats_ext(k, n, db, k)
            st = handle.gemm_strided_batch_with_stats(N, N, m, n, k, 1.0, da, m, 0, db, k, 0, 0.0, dca,
                                                      m, 0, 1, AUTO, ia, ib)
            assert st == 0
            assert oracle.residual(truth, dca.cpu().numpy(), m) < oracle.error_threshold(True, k)
    assert handle.kernel_status() == 0
