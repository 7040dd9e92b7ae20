"""Seeded random sweep over shapes, operations, leading dimensions, batches, scalars and modes:
every case is checked against an FP64 product computed by torch on the same GPU with the
reference's own tolerance (relative Frobenius residual below 2^-23 sqrt(k) for the corrected
modes, 2^-10 sqrt(k) for the others; test/main.cu:68-74).  The point is breadth: edge tiles,
tiny and skinny problems, every tile width and both kernels, as the dispatcher picks them."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N, T, Cj = 0, 1, 2
MODES = {1: True, 2: True, 3: False, 4: False}      # mode -> error corrected


def _colmajor(torch, rows, cols, ld, gen, cplx):
    """(flat storage with leading dimension ld, logical rows x cols view) on the GPU."""
    store = torch.rand(cols, ld, device="cuda", generator=gen) * 2 - 1
    if cplx:
        store = torch.complex(store, torch.rand(cols, ld, device="cuda", generator=gen) * 2 - 1)
    return store, store[:, :rows].t()


def _op(view, op):
    if op == N:
        return view
    return view.t().conj() if op == Cj else view.t()


@pytest.mark.parametrize("seed", range(12))
def test_random_cases_against_fp64(handle, seed):
    import torch

    rng = np.random.default_rng(1000 + seed)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2000 + seed)
    for case in range(14):
        cplx = bool(rng.integers(0, 2))
        big = case % 7 == 0
        m, n, k = (int(rng.integers(1, 2200 if big else 420)) for _ in range(3))
        if case % 5 == 1:
            m = int(rng.integers(1, 9))              # skinny
        if case % 5 == 2:
            n = int(rng.integers(1, 9))
        op_a = int(rng.choice([N, T, Cj] if cplx else [N, T]))
        op_b = int(rng.choice([N, T, Cj] if cplx else [N, T]))
        mode = int(rng.choice(list(MODES)))
        batch = int(rng.choice([1, 1, 2, 5]))
        ar, ac = (m, k) if op_a == N else (k, m)
        br, bc = (k, n) if op_b == N else (n, k)
        lda, ldb, ldc = (x + int(rng.integers(0, 7)) for x in (ar, br, m))
        alpha = complex(rng.uniform(-2, 2), rng.uniform(-2, 2)) if cplx else float(rng.uniform(-2, 2))
        beta = rng.choice([0.0, 1.0, -0.75])
        beta = complex(beta, 0.5 * beta) if cplx else float(beta)
        stores, views = [], []
        for rows, cols, ld in ((ar, ac, lda), (br, bc, ldb), (m, n, ldc)):
            ss, vv = zip(*[_colmajor(torch, rows, cols, ld, gen, cplx) for _ in range(batch)])
            stores.append(torch.stack([s.reshape(-1) for s in ss]).contiguous())
            views.append(None)
        sa, sb, sc = (s.shape[1] for s in stores)
        c0 = stores[2].clone()
        wide = torch.complex128 if cplx else torch.float64

        def view(flat, rows, cols, ld):
            return flat.view(cols, ld)[:, :rows].t()

        handle.gemm_strided_batch(op_a, op_b, m, n, k, alpha, stores[0], lda, sa, stores[1], ldb, sb,
                                  beta, stores[2], ldc, sc, batch, mode, complex=cplx)
        torch.cuda.synchronize()
        for b in range(batch):
            A = _op(view(stores[0][b], ar, ac, lda), op_a).to(wide)
            B = _op(view(stores[1][b], br, bc, ldb), op_b).to(wide)
            truth = alpha * (A @ B) + beta * view(c0[b], m, n, ldc).to(wide)
            got = view(stores[2][b], m, n, ldc).to(wide)
            denom = truth.norm().item()
            res = (truth - got).norm().item() / denom if denom > 0 else (truth - got).norm().item()
            tol = (2.0 ** -23 if MODES[mode] else 2.0 ** -10) * np.sqrt(k)
            assert res < tol, (seed, case, cplx, m, n, k, op_a, op_b, mode, batch, lda, ldb, ldc, res)
            # the padding rows of C are not written
            if ldc > m:
                assert torch.equal(stores[2][b].view(n, ldc)[:, m:], c0[b].view(n, ldc)[:, m:])
    assert handle.kernel_status() == 0
