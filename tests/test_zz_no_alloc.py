"""cuMpSGEMM_sgemm_static_scratch: the GEMM entry point for callers that cannot allocate.

Some callers of the library are not allowed to obtain device memory at call time (fixed memory
budget, no tolerance for the device synchronisation cudaMalloc implies, no handle).  For them
the split operand panels live in a 32 MiB array inside the library.  The test calls the entry
point through the C ABI twice in a row, with different shapes and operands so that the second
call reuses array contents left by the first, and compares each result with the regular
cuMpSGEMM_sgemm on the same inputs, within the suite's usual tolerance (relative Frobenius
residual below 2^-23 * sqrt(K)).  The shapes cover the three single-CTA tile widths and the
CTA-pair kernel, including the largest problem that fits the array exactly and one k beyond it.
Where the regular entry point runs the same split pass and the same GEMM kernel (it reports
the tile class it used), the results are also bit-identical.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  It does not depend on state left by other tests and passes in a fresh process.
"""
import pytest

pytestmark = pytest.mark.gpu

FP16TCEC, TF32TCEC = 1, 2
# shapes for which the handle-based entry point is known to run the same split pass and GEMM
# kernel as the allocation-free one (it may choose other kernels for other shapes)
SAME_KERNELS = {(2048, 2048), (2560, 2304)}


def test_static_scratch_matches_regular_entry_point(oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cumpsgemm_b200 import api

    stream = torch.cuda.current_stream()
    handle = api.Handle()
    handle.use_current_torch_stream()
    try:
        # two calls in a row; the second is smaller and transposed, so it runs on a region of
        # the array that still holds the first call's panels
        cases = [(FP16TCEC, 0, 0, 700, 520, 900, 1.0, 0.5),       # 128 x 64 tiles
                 (TF32TCEC, 1, 0, 300, 200, 260, -2.0, 0.0),      # smaller, transposed A
                 (FP16TCEC, 0, 0, 2048, 2048, 2048, 1.0, 0.5),    # fills the array exactly
                 (FP16TCEC, 0, 1, 1536, 1536, 640, 1.0, 0.0),     # 128 x 128 tiles
                 (FP16TCEC, 0, 0, 2560, 2304, 512, 0.5, 0.25)]    # CTA pairs (256 x 256)
        inputs, results = [], []
        for i, (mode, op_a, op_b, m, n, k, alpha, beta) in enumerate(cases):
            am, an = (m, k) if op_a == 0 else (k, m)
            bm, bn = (k, n) if op_b == 0 else (n, k)
            a = oracle.gen_uniform(10 + i, am * an)
            b = oracle.gen_uniform(20 + i, bm * bn)
            c0 = oracle.gen_uniform(30 + i, m * n)
            da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
            dc = torch.from_numpy(c0.copy()).cuda()
            st = api.sgemm_static_scratch(stream, op_a, op_b, m, n, k, alpha, da, am, db, bm, beta,
                                          dc, m, mode)
            assert st == api.CUBLAS_STATUS_SUCCESS
            inputs.append((mode, op_a, op_b, m, n, k, alpha, beta, a, b, c0, da, db, am, bm))
            results.append(dc)
        torch.cuda.synchronize()
        for (mode, op_a, op_b, m, n, k, alpha, beta, a, b, c0, da, db, am, bm), got in zip(inputs, results):
            ref = torch.from_numpy(c0.copy()).cuda()
            handle.gemm(op_a, op_b, m, n, k, alpha, da, am, db, bm, beta, ref, m, mode)
            torch.cuda.synchronize()
            truth = oracle.gemm_f64(op_a, op_b, m, n, k, alpha, a, am, b, bm, beta, c0, m)
            thr = oracle.error_threshold(True, k)
            assert oracle.residual(truth, got.cpu().numpy(), m) < thr
            ref64 = ref.double().cpu().numpy().reshape((m, n), order="F")
            assert oracle.residual(ref64, got.cpu().numpy(), m) < thr
            if (m, n) in SAME_KERNELS:
                assert torch.equal(got, ref)
        assert handle.kernel_status() == 0
        # beyond the built-in array: rejected before anything is launched
        big = torch.zeros(1, device="cuda")
        st = api.sgemm_static_scratch(stream, 0, 0, 4096, 4096, 4096, 1.0, big, 4096, big, 4096,
                                      0.0, big, 4096, FP16TCEC)
        assert st == api.CUBLAS_STATUS_INVALID_VALUE
        st = api.sgemm_static_scratch(stream, 0, 0, 2048, 2048, 2049, 1.0, big, 2048, big, 2049,
                                      0.0, big, 2048, FP16TCEC)      # one k past the exact fit
        assert st == api.CUBLAS_STATUS_INVALID_VALUE
        huge = 0x3fffffff                                            # sizes whose byte count
        st = api.sgemm_static_scratch(stream, 0, 0, huge, huge, huge, 1.0, big, huge, big, huge,
                                      0.0, big, huge, TF32TCEC)      # would wrap 64 bits
        assert st == api.CUBLAS_STATUS_INVALID_VALUE
        st = api.sgemm_static_scratch(stream, 0, 0, 64, 64, 64, 1.0, big, 64, big, 64, 0.0, big, 64, 9)
        assert st == api.CUBLAS_STATUS_NOT_SUPPORTED
    finally:
        handle.destroy()
