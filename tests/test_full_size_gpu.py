"""The benchmark configurations at their stated sizes (the shapes of the reference's own
large runs, test/main.cu:539-629 and :726-819).

Inputs are generated on the GPU from fixed seeds.  Every case is checked three ways where the
size allows: sampled rows of C against the host oracle's FP64 GEMM, sampled rows and columns
against an FP64 product computed on the GPU, and the whole matrix against the GPU's FP64
product.  The criterion is the reference's relative Frobenius residual < 2^-23 * sqrt(K)
(test/main.cu:68-74) and, on top, "no worse than an FP32 SGEMM on the same inputs".
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N, T = 0, 1
FP16TCEC, TF32TCEC, AUTO, SCALING = 1, 2, 9, 11


def _torch():
    import torch

    return torch


def _gen(seed):
    torch = _torch()
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return g


def _uniform_exp(g, count, lo=-8, hi=8):
    torch = _torch()
    u = torch.rand(count, device="cuda", generator=g) * 2 - 1
    e = torch.randint(lo, hi + 1, (count,), device="cuda", generator=g, dtype=torch.int32)
    return torch.ldexp(u, e)


def _wide_exponent(g, count, lo=-30, hi=10):
    torch = _torch()
    s = torch.where(torch.rand(count, device="cuda", generator=g) < 0.5, -1.0, 1.0)
    f = 1 + torch.rand(count, device="cuda", generator=g)
    e = torch.randint(lo, hi + 1, (count,), device="cuda", generator=g, dtype=torch.int32)
    return torch.ldexp(s * f, e)


def _residual(truth, got):
    return ((truth - got).pow(2).sum() / truth.pow(2).sum()).sqrt().item()


def _rows_truth(a, b, c0, m, n, k, beta, rows, chunk=2048):
    """FP64 rows of A B + beta C0 (column-major flat operands, op N/N) as an (n, R) tensor."""
    torch = _torch()
    a_rows = a.view(k, m)[:, rows].double()
    out = torch.empty(n, len(rows), dtype=torch.float64, device="cuda")
    bv = b.view(n, k)
    for j0 in range(0, n, chunk):
        j1 = min(n, j0 + chunk)
        out[j0:j1] = bv[j0:j1].double() @ a_rows
    if c0 is not None and beta != 0:
        out += beta * c0.view(n, m)[:, rows].double()
    return out


def _cols_truth(a, b, c0, m, n, k, beta, cols, chunk=2048):
    """FP64 columns as a (C, m) tensor."""
    torch = _torch()
    b_cols = b.view(n, k)[cols].double()
    out = torch.zeros(len(cols), m, dtype=torch.float64, device="cuda")
    av = a.view(k, m)
    for l0 in range(0, k, chunk):
        l1 = min(k, l0 + chunk)
        out += b_cols[:, l0:l1] @ av[l0:l1].double()
    if c0 is not None and beta != 0:
        out += beta * c0.view(n, m)[cols].double()
    return out


def _whole_truth(a, b, c0, m, n, k, beta):
    """Row-major (n, m) FP64 product = column-major C."""
    t = b.view(n, k).double() @ a.view(k, m).double()
    if c0 is not None and beta != 0:
        t += beta * c0.view(n, m).double()
    return t


def _check_rows_on_host(oracle, a, b, c0, c, m, n, k, beta, rows, thr):
    ah, bh, ch = a.cpu().numpy(), b.cpu().numpy(), c.cpu().numpy()
    c0h = c0.cpu().numpy() if c0 is not None else None
    for i in rows:
        truth = oracle.gemm_f64(N, N, 1, n, k, 1.0, ah[i:], m, bh, k, beta,
                                c0h[i:] if c0h is not None else None, m)
        got = ch.reshape((n, m))[:, i].copy()
        assert oracle.residual(truth, got, 1) < thr


@pytest.mark.parametrize("mode", [FP16TCEC, TF32TCEC])
@pytest.mark.parametrize("n", [4096, 8192, 16384])
def test_config2_square_sweep(handle, oracle, n, mode):
    """Config 2: m=n=k=N, inputs uniform(-1,1) * 2^e, e in [-8, 8], alpha=1, beta=0.5."""
    torch = _torch()
    g = _gen(20 + n // 4096)
    a, b = _uniform_exp(g, n * n), _uniform_exp(g, n * n)
    c0 = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
    c = c0.clone()
    handle.gemm(N, N, n, n, n, 1.0, a, n, b, n, 0.5, c, n, mode)
    thr = oracle.error_threshold(True, n)
    rows = [0, 127, 128, n // 2 + 3, n - 1]
    cols = [0, 255, 256, n - 1]
    t_rows = _rows_truth(a, b, c0, n, n, n, 0.5, rows)
    t_cols = _cols_truth(a, b, c0, n, n, n, 0.5, cols)
    cv = c.view(n, n)
    for j, i in enumerate(rows):
        assert _residual(t_rows[:, j], cv[:, i].double()) < thr
    for j, col in enumerate(cols):
        assert _residual(t_cols[j], cv[col].double()) < thr
    _check_rows_on_host(oracle, a, b, c0, c, n, n, n, 0.5, rows[1:3], thr)
    # whole matrix, and the FP32 comparator on the same inputs
    truth = _whole_truth(a, b, c0, n, n, n, 0.5)
    r = _residual(truth, cv.double())
    assert r < thr
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    c32 = torch.addmm(c0.view(n, n), b.view(n, n), a.view(n, n), beta=0.5)
    torch.backends.cuda.matmul.allow_tf32 = prev
    r32 = _residual(truth, c32.double())
    assert r <= 1.5 * r32, (r, r32)
    err = (truth - cv.double()).abs()
    err32 = (truth - c32.double()).abs()
    nz = truth != 0
    assert (err[nz] / truth[nz].abs()).mean().item() <= 1.5 * (err32[nz] / truth[nz].abs()).mean().item()


@pytest.mark.parametrize("mode", [SCALING, AUTO])
def test_config3_wide_exponent_product(handle, oracle, mode):
    """Config 3: m=n=k=8192, sign uniform, exponent uniform over [-30, 10]; the product itself in
    FP16TCEC_SCALING and AUTO, the decision AUTO takes, and the operands left untouched."""
    torch = _torch()
    n = 8192
    g = _gen(33)
    a, b = _wide_exponent(g, n * n), _wide_exponent(g, n * n)
    a_keep, b_keep = a.clone(), b.clone()
    c = torch.zeros(n * n, device="cuda")
    handle.set_exp_stats_params(0.0, 2.0 ** -15, 0.0)
    if mode == SCALING:
        handle.gemm(N, N, n, n, n, 1.0, a, n, b, n, 0.0, c, n, mode)
    else:
        ia, ib = handle.exp_stats_ext(n, n, a, n), handle.exp_stats_ext(n, n, b, n)
        # values span 40 binades: some stay below the relative underflow threshold after
        # scaling, so both operands decide TF32TCEC and the flag carries no scale bit
        assert int(handle.get_exp_stats_compute_mode_level(ia)) == TF32TCEC
        assert int(handle.get_exp_stats_compute_mode_level(ib)) == TF32TCEC
        handle.gemm_strided_batch_with_stats(N, N, n, n, n, 1.0, a, n, 0, b, n, 0, 0.0, c, n, 0, 1,
                                             AUTO, ia, ib)
        # the decision is the oracle's on the same data (bit-exact counts)
        want = oracle.exp_stats(a.cpu().numpy(), n, n, n)
        uf, total = handle.get_exp_stats(ia)
        assert (uf, total, handle.get_max_exp(ia)) == (want["underflow"], want["total"],
                                                       want["max_exp"])
    assert torch.equal(a, a_keep) and torch.equal(b, b_keep)
    thr = oracle.error_threshold(True, n)
    truth = _whole_truth(a, b, None, n, n, n, 0.0)
    assert _residual(truth, c.view(n, n).double()) < thr
    rows = [0, 4097, n - 1]
    t_rows = _rows_truth(a, b, None, n, n, n, 0.0, rows)
    for j, i in enumerate(rows):
        assert _residual(t_rows[:, j], c.view(n, n)[:, i].double()) < thr
    _check_rows_on_host(oracle, a, b, None, c, n, n, n, 0.0, rows[1:2], thr)


def test_config4_full_batch_cgemm_scaling(handle, oracle):
    """Config 4 at its full batch: 512 complex 256^3 products, unit Frobenius norm per operand
    matrix, FP16TCEC_SCALING with one scale factor for the whole batch; 16 sampled batches
    against FP64 on the GPU, two of them also against the host oracle."""
    torch = _torch()
    batch, s = 512, 256
    g = _gen(44)

    def unit():
        z = torch.complex(torch.randn(batch, s * s, device="cuda", generator=g),
                          torch.randn(batch, s * s, device="cuda", generator=g))
        return (z / z.abs().pow(2).sum(1, keepdim=True).sqrt()).to(torch.complex64).contiguous()

    za, zb = unit(), unit()
    zc = torch.zeros(batch * s * s, dtype=torch.complex64, device="cuda")
    handle.gemm_strided_batch(N, N, s, s, s, 1.0, za, s, s * s, zb, s, s * s, 0.0, zc, s, s * s,
                              batch, SCALING)
    thr = oracle.error_threshold(True, s)
    picked = list(range(0, batch, 37)) + [batch - 1, batch - 2]
    assert len(picked) == 16
    for i in picked:
        A = za[i].view(s, s).t().to(torch.complex128)
        B = zb[i].view(s, s).t().to(torch.complex128)
        got = zc.view(batch, s, s)[i].t().to(torch.complex128)
        truth = A @ B
        r = ((truth - got).abs().pow(2).sum() / truth.abs().pow(2).sum()).sqrt().item()
        assert r < thr, (i, r)
    zah, zbh, zch = za.cpu().numpy().reshape(-1), zb.cpu().numpy().reshape(-1), zc.cpu().numpy()
    for i in (0, 300):
        truth = oracle.gemm_f64(N, N, s, s, s, 1.0, zah[i * s * s:], s, zbh[i * s * s:], s, 0.0,
                                None, s)
        assert oracle.residual(truth, zch[i * s * s:(i + 1) * s * s], s) < thr
    # the scale factor covers the whole batch: the call's statistics slots hold the batch-wide
    # maximum exponents, equal to the oracle's
    id_b = handle.get_current_exp_stats_buffer_id()
    assert handle.get_max_exp(id_b - 1) == oracle.exp_max(zah, s, s, s, batch, s * s)
    assert handle.get_max_exp(id_b) == oracle.exp_max(zbh, s, s, s, batch, s * s)


def test_config5a_one_ranks_batch_share_auto(handle, oracle):
    """Config 5, batch part, one rank's share at 8 GPUs: 8 products of 8192^3, N(0,1), AUTO."""
    torch = _torch()
    n, batch = 8192, 8
    g = _gen(55)
    a = torch.randn(batch * n * n, device="cuda", generator=g)
    b = torch.randn(batch * n * n, device="cuda", generator=g)
    c = torch.zeros(batch * n * n, device="cuda")
    handle.set_exp_stats_params(0.0, 2.0 ** -15, 0.0)
    ia = handle.exp_stats_ext(n, n, a, n, batch, n * n)
    ib = handle.exp_stats_ext(n, n, b, n, batch, n * n)
    handle.gemm_strided_batch_with_stats(N, N, n, n, n, 1.0, a, n, n * n, b, n, n * n, 0.0, c, n,
                                         n * n, batch, AUTO, ia, ib)
    # counts over the whole batch: every value is counted once
    uf, total = handle.get_exp_stats(ia)
    mode_a = int(handle.get_exp_stats_compute_mode_level(ia))
    assert mode_a in (FP16TCEC, TF32TCEC, SCALING)
    if mode_a == FP16TCEC:               # decided at stage 1: the counters hold every value
        assert total == batch * n * n
    thr = oracle.error_threshold(True, n)
    rows = [0, 130, n - 1]
    for i in (0, 3, batch - 1):
        sl = slice(i * n * n, (i + 1) * n * n)
        t_rows = _rows_truth(a[sl], b[sl], None, n, n, n, 0.0, rows)
        for j, r in enumerate(rows):
            assert _residual(t_rows[:, j], c[sl].view(n, n)[:, r].double()) < thr
    sl = slice(2 * n * n, 3 * n * n)
    truth = _whole_truth(a[sl], b[sl], None, n, n, n, 0.0)
    assert _residual(truth, c[sl].view(n, n).double()) < thr
    del truth
    _check_rows_on_host(oracle, a[sl], b[sl], None, c[sl], n, n, n, 0.0, [4096], thr)


def test_config5b_one_ranks_column_block(handle, oracle):
    """Config 5, single-GEMM part, one rank's column block at 8 GPUs: C[:, J] of the
    65536 x 65536 x 8192 product with |J| = 8192, N(0,1), FP16TCEC."""
    torch = _torch()
    m, n, k = 65536, 8192, 8192
    g = _gen(56)
    a = torch.randn(m * k, device="cuda", generator=g)
    b = torch.randn(k * n, device="cuda", generator=g)
    c = torch.zeros(m * n, device="cuda")
    handle.gemm(N, N, m, n, k, 1.0, a, m, b, k, 0.0, c, m, FP16TCEC)
    thr = oracle.error_threshold(True, k)
    rows = [0, 255, 256, 40000, m - 1]
    cols = [0, 4097, n - 1]
    t_rows = _rows_truth(a, b, None, m, n, k, 0.0, rows)
    t_cols = _cols_truth(a, b, None, m, n, k, 0.0, cols)
    cv = c.view(n, m)
    for j, i in enumerate(rows):
        assert _residual(t_rows[:, j], cv[:, i].double()) < thr
    for j, col in enumerate(cols):
        assert _residual(t_cols[j], cv[col].double()) < thr
    _check_rows_on_host(oracle, a, b, None, c, m, n, k, 0.0, [40000], thr)
