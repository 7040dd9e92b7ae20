"""Host-side mirror of the cuMpSGEMM operator interface.

Names, argument order and error behaviour follow the reference's public API
(``include/cumpsgemm/cumpsgemm.h:7-57``, ``cumpsgemm.hpp:8-129``): column-major
matrices in device memory, ``alpha``/``beta`` as host scalars, sizes in
elements.  Matrices are passed as torch CUDA tensors (any shape; only the
storage is used) or as raw device addresses (``int``).  Every call goes
through the C ABI of ``libcumpsgemm.so``; there is no Python or CPU
implementation behind it.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Optional, Tuple, Union

from . import _lib

CUBLAS_OP_N = 0
CUBLAS_OP_T = 1
CUBLAS_OP_C = 2

CUBLAS_STATUS_SUCCESS = 0
CUBLAS_STATUS_NOT_INITIALIZED = 1
CUBLAS_STATUS_ALLOC_FAILED = 3
CUBLAS_STATUS_INVALID_VALUE = 7
CUBLAS_STATUS_ARCH_MISMATCH = 8
CUBLAS_STATUS_EXECUTION_FAILED = 13
CUBLAS_STATUS_NOT_SUPPORTED = 15


class ComputeMode(enum.IntEnum):
    """cuMpSGEMM_compute_mode_t (reference: include/cumpsgemm/detail/common.h:6-20)."""

    CUBLAS = 0
    FP16TCEC = 1
    TF32TCEC = 2
    FP16TC = 3
    TF32TC = 4
    CUBLAS_SIMT = 5
    CUBLAS_FP16TC = 6
    CUBLAS_TF32TC = 7
    DRY_RUN = 8
    AUTO = 9
    UNDEFINED = 10
    FP16TCEC_SCALING = 11
    FP32_SIMT = 12


class CuMpSGEMMError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what} failed with cublasStatus_t {status}")
        self.status = status


DevPtr = Union[int, "torch.Tensor"]  # noqa: F821


def _ptr(x: DevPtr) -> int:
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        if not x.is_cuda:
            raise ValueError("matrix operands must live in device memory")
        return x.data_ptr()
    raise TypeError(f"expected a CUDA tensor or a device address, got {type(x)}")


def _is_complex(x: DevPtr, hint: Optional[bool]) -> bool:
    if hint is not None:
        return hint
    if hasattr(x, "is_complex"):
        return bool(x.is_complex())
    raise ValueError("pass complex=True/False when operands are raw addresses")


def _scalar(value, is_complex: bool):
    if is_complex:
        z = complex(value)
        arr = (C.c_float * 2)(z.real, z.imag)
    else:
        arr = (C.c_float * 1)(float(value))
    return arr


def compute_mode_string(mode: int) -> str:
    """cuMpSGEMM_get_compute_mode_string."""
    return _lib.load().cuMpSGEMM_get_compute_mode_string(int(mode)).decode()


class Handle:
    """cuMpSGEMM_handle_t with the C and C++ API as methods."""

    def __init__(self):
        self._lib = _lib.load()
        h = C.c_void_p()
        st = self._lib.cuMpSGEMM_create(C.byref(h))
        if st != CUBLAS_STATUS_SUCCESS:
            raise CuMpSGEMMError(st, "cuMpSGEMM_create")
        self._h = h

    # ------------------------------------------------------------------ life cycle
    def destroy(self) -> None:
        if self._h is not None:
            self._lib.cuMpSGEMM_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.destroy()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    @property
    def raw(self) -> C.c_void_p:
        return self._h

    def set_stream(self, stream) -> None:
        """Accepts a torch.cuda.Stream, a raw cudaStream_t (int) or None (default stream)."""
        s = 0 if stream is None else getattr(stream, "cuda_stream", stream)
        st = self._lib.cuMpSGEMM_set_stream(self._h, C.c_void_p(int(s)))
        if st != CUBLAS_STATUS_SUCCESS:
            raise CuMpSGEMMError(st, "cuMpSGEMM_set_stream")

    def use_current_torch_stream(self) -> None:
        import torch

        self.set_stream(torch.cuda.current_stream())

    # ------------------------------------------------------------------ GEMM
    def gemm(self, op_A: int, op_B: int, m: int, n: int, k: int, alpha, A: DevPtr, lda: int,
             B: DevPtr, ldb: int, beta, Cmat: DevPtr, ldc: int, mode: int,
             complex: Optional[bool] = None, check: bool = True) -> int:
        """cuMpSGEMM_sgemm / cuMpSGEMM_cgemm.  Returns the cublasStatus_t."""
        cplx = _is_complex(A, complex)
        fn = self._lib.cuMpSGEMM_cgemm if cplx else self._lib.cuMpSGEMM_sgemm
        a, b = _scalar(alpha, cplx), _scalar(beta, cplx)
        st = fn(self._h, op_A, op_B, m, n, k, C.cast(a, C.c_void_p), _ptr(A), lda, _ptr(B), ldb,
                C.cast(b, C.c_void_p), _ptr(Cmat), ldc, int(mode))
        if check and st != CUBLAS_STATUS_SUCCESS:
            raise CuMpSGEMMError(st, "cuMpSGEMM_cgemm" if cplx else "cuMpSGEMM_sgemm")
        return st

    def gemm_strided_batch(self, op_A: int, op_B: int, m: int, n: int, k: int, alpha, A: DevPtr,
                           lda: int, stridea: int, B: DevPtr, ldb: int, strideb: int, beta,
                           Cmat: DevPtr, ldc: int, stridec: int, batch_count: int, mode: int,
                           complex: Optional[bool] = None, check: bool = True) -> int:
        """cuMpSGEMM_sgemm_strided_batch / cuMpSGEMM_cgemm_strided_batch."""
        cplx = _is_complex(A, complex)
        fn = (self._lib.cuMpSGEMM_cgemm_strided_batch if cplx
              else self._lib.cuMpSGEMM_sgemm_strided_batch)
        a, b = _scalar(alpha, cplx), _scalar(beta, cplx)
        st = fn(self._h, op_A, op_B, m, n, k, C.cast(a, C.c_void_p), _ptr(A), lda, stridea,
                _ptr(B), ldb, strideb, C.cast(b, C.c_void_p), _ptr(Cmat), ldc, stridec,
                batch_count, int(mode))
        if check and st != CUBLAS_STATUS_SUCCESS:
            raise CuMpSGEMMError(st, "cuMpSGEMM_*gemm_strided_batch")
        return st

    def gemm_strided_batch_with_stats(self, op_A, op_B, m, n, k, alpha, A, lda, stridea, B, ldb,
                                      strideb, beta, Cmat, ldc, stridec, batch_count, mode,
                                      stats_id_a: int, stats_id_b: int,
                                      complex: Optional[bool] = None) -> int:
        """GEMM driven by statistics slots decided beforehand (multi-GPU path)."""
        cplx = _is_complex(A, complex)
        fn = (self._lib.cuMpSGEMM_cgemm_strided_batch_with_stats if cplx
              else self._lib.cuMpSGEMM_sgemm_strided_batch_with_stats)
        a, b = _scalar(alpha, cplx), _scalar(beta, cplx)
        st = fn(self._h, op_A, op_B, m, n, k, C.cast(a, C.c_void_p), _ptr(A), lda, stridea,
                _ptr(B), ldb, strideb, C.cast(b, C.c_void_p), _ptr(Cmat), ldc, stridec,
                batch_count, int(mode), stats_id_a, stats_id_b)
        if st != CUBLAS_STATUS_SUCCESS:
            raise CuMpSGEMMError(st, "cuMpSGEMM_*gemm_strided_batch_with_stats")
        return st

    def gemm_tiny(self, long_is_m: bool, op_A: int, op_B: int, length: int, alpha, A: DevPtr,
                  lda: int, B: DevPtr, ldb: int, beta, Cmat: DevPtr, ldc: int, stridea: int = 0,
                  strideb: int = 0, stridec: int = 0, batch_count: int = 1,
                  complex: Optional[bool] = None, check: bool = True) -> int:
        """cuMpSGEMM_{s,c}gemm_Mx2x2 (long_is_m) / cuMpSGEMM_{s,c}gemm_2xNx2: plain FP32 GEMM
        with the two short dimensions equal to 2 and a power-of-two long one."""
        cplx = _is_complex(A, complex)
        name = "cuMpSGEMM_%sgemm_%s" % ("c" if cplx else "s", "Mx2x2" if long_is_m else "2xNx2")
        a, b = _scalar(alpha, cplx), _scalar(beta, cplx)
        st = getattr(self._lib, name)(self._h, op_A, op_B, length, C.cast(a, C.c_void_p), _ptr(A),
                                      lda, stridea, _ptr(B), ldb, strideb, C.cast(b, C.c_void_p),
                                      _ptr(Cmat), ldc, stridec, batch_count)
        if check and st != CUBLAS_STATUS_SUCCESS:
            raise CuMpSGEMMError(st, name)
        return st

    def gemm_module(self, op_A, op_B, m, n, k, alpha, A, lda, B, ldb, beta, Cmat, ldc,
                    mode) -> Tuple[int, int]:
        """cumpsgemm::gemm<float> with its used_kernel_module_id out-parameter."""
        a, b = _scalar(alpha, False), _scalar(beta, False)
        mod = C.c_uint(0xFFFFFFFF)
        st = self._lib.cuMpSGEMM_sgemm_module(self._h, op_A, op_B, m, n, k,
                                              C.cast(a, C.c_void_p), _ptr(A), lda, _ptr(B), ldb,
                                              C.cast(b, C.c_void_p), _ptr(Cmat), ldc, int(mode),
                                              C.byref(mod))
        return st, mod.value

    def kernel_status(self) -> int:
        """Synchronise and return (then clear) the GEMM kernel's bounded-wait status word."""
        return self._lib.cuMpSGEMM_get_kernel_status(self._h)

    def selftest_bounded_wait(self, limit_ms: int = 200) -> Tuple[int, float]:
        """(status code, milliseconds waited) of a wait on a barrier nothing signals."""
        t = C.c_double(0)
        st = self._lib.cuMpSGEMM_selftest_bounded_wait(self._h, limit_ms, C.byref(t))
        return st, t.value

    def set_workspace_limit(self, nbytes: int) -> None:
        self._lib.cuMpSGEMM_set_workspace_limit(self._h, nbytes)

    def reload_tuning_env(self) -> None:
        """Read the CUMPSGEMM_TILE_N / PAIR / DRAIN_CHUNK / FIRST_CHUNK / PACE / FUSED variables
        again (a handle reads them once, at creation)."""
        self._lib.cuMpSGEMM_reload_tuning_env(self._h)

    def set_count_tail_padding(self, enable: bool) -> None:
        """Count the zeros the reference appends to matrices whose element count is not a
        multiple of 4 (src/exp_stats.cu:101-116); off by default."""
        self._lib.cuMpSGEMM_set_count_tail_padding(self._h, 1 if enable else 0)

    def set_debug_buffer(self, dev_words8) -> None:
        """Stall-breakdown buffer (8 x int64 CUDA tensor) or None."""
        self._lib.cuMpSGEMM_set_debug_buffer(self._h, 0 if dev_words8 is None else _ptr(dev_words8))

    def set_kernel_timing(self, enable: bool) -> None:
        self._lib.cuMpSGEMM_set_kernel_timing(self._h, 1 if enable else 0)

    def get_kernel_timing(self) -> Tuple[int, float, float]:
        """(launch groups, summed split-pass ms, summed GEMM-kernel ms) since the last query."""
        s, g = C.c_double(0), C.c_double(0)
        n = self._lib.cuMpSGEMM_get_kernel_timing(self._h, C.byref(s), C.byref(g))
        return int(n), s.value, g.value

    # ------------------------------------------------------------------ statistics
    def exp_stats_ext(self, m, n, ptr: DevPtr, ld, batch_size=1, stride=0,
                      complex: Optional[bool] = None) -> int:
        cplx = _is_complex(ptr, complex)
        fn = self._lib.cuMpSGEMM_exp_stats_ext_c if cplx else self._lib.cuMpSGEMM_exp_stats_ext_s
        return fn(self._h, m, n, _ptr(ptr), ld, batch_size, stride)

    def exp_max_ext(self, m, n, ptr: DevPtr, ld, batch_size=1, stride=0,
                    complex: Optional[bool] = None) -> int:
        cplx = _is_complex(ptr, complex)
        fn = self._lib.cuMpSGEMM_exp_max_ext_c if cplx else self._lib.cuMpSGEMM_exp_max_ext_s
        return fn(self._h, m, n, _ptr(ptr), ld, batch_size, stride)

    def get_exp_stats(self, buffer_id: int) -> Tuple[int, int]:
        """(underflow count, total count) – the reference's order."""
        uf, total = C.c_size_t(0), C.c_size_t(0)
        self._lib.cuMpSGEMM_get_exp_stats(self._h, buffer_id, C.byref(uf), C.byref(total))
        return uf.value, total.value

    def get_current_exp_stats_buffer_id(self) -> int:
        return self._lib.cuMpSGEMM_get_current_exp_stats_buffer_id(self._h)

    def reset_exp_stats_buffer_id(self) -> None:
        self._lib.cuMpSGEMM_reset_exp_stats_buffer_id(self._h)

    def set_exp_stats_params(self, ignore_threshold: float, underflow_threshold: float,
                             underflow_ratio_tolerance: float) -> None:
        self._lib.cuMpSGEMM_set_exp_stats_params(self._h, ignore_threshold, underflow_threshold,
                                                 underflow_ratio_tolerance)

    def enable_exp_stats(self) -> None:
        self._lib.cuMpSGEMM_enable_exp_stats(self._h)

    def disable_exp_stats(self) -> None:
        self._lib.cuMpSGEMM_disable_exp_stats(self._h)

    def get_max_exp(self, buffer_id: int) -> float:
        return self._lib.cuMpSGEMM_get_max_exp(self._h, buffer_id)

    def get_exp_stats_compute_mode_level(self, buffer_id: int) -> ComputeMode:
        return ComputeMode(self._lib.cuMpSGEMM_get_exp_stats_compute_mode_level(self._h,
                                                                                buffer_id))

    # staged statistics for multi-GPU callers
    def exp_stats_begin(self) -> int:
        return self._lib.cuMpSGEMM_exp_stats_begin(self._h)

    def exp_stats_stage(self, stage: int, buffer_id: int, m, n, ptr: DevPtr, ld, batch_size=1,
                        stride=0, complex: Optional[bool] = None) -> None:
        cplx = _is_complex(ptr, complex)
        fn = (self._lib.cuMpSGEMM_exp_stats_stage_c if cplx
              else self._lib.cuMpSGEMM_exp_stats_stage_s)
        fn(self._h, stage, buffer_id, m, n, _ptr(ptr), ld, batch_size, stride)

    def exp_stats_decide(self, decision: int, buffer_id: int) -> None:
        self._lib.cuMpSGEMM_exp_stats_decide(self._h, decision, buffer_id)

    def exp_stats_export(self, buffer_id: int, dev_words4: DevPtr) -> None:
        self._lib.cuMpSGEMM_exp_stats_export(self._h, buffer_id, _ptr(dev_words4))

    def exp_stats_import(self, buffer_id: int, dev_words4: DevPtr) -> None:
        self._lib.cuMpSGEMM_exp_stats_import(self._h, buffer_id, _ptr(dev_words4))

    # ------------------------------------------------------------------ scaling
    def _scale(self, base: str, ids, flag_id, m, n, ptr, ld, batch_size, stride, complex):
        cplx = _is_complex(ptr, complex)
        fn = getattr(self._lib, f"cuMpSGEMM_{base}_{'c' if cplx else 's'}")
        fn(self._h, *ids, flag_id, m, n, _ptr(ptr), ld, batch_size, stride)

    def scale_A(self, exp_stats_buffer_id, dynamic_launch_flag_buffer_id, m, n, ptr, ld,
                batch_size=1, stride=0, complex=None):
        self._scale("scale_A", (exp_stats_buffer_id,), dynamic_launch_flag_buffer_id, m, n, ptr,
                    ld, batch_size, stride, complex)

    def scale_B(self, exp_stats_buffer_id, dynamic_launch_flag_buffer_id, m, n, ptr, ld,
                batch_size=1, stride=0, complex=None):
        self._scale("scale_B", (exp_stats_buffer_id,), dynamic_launch_flag_buffer_id, m, n, ptr,
                    ld, batch_size, stride, complex)

    def scale_C(self, exp_stats_buffer_A_id, exp_stats_buffer_B_id, dynamic_launch_flag_buffer_id,
                m, n, ptr, ld, batch_size=1, stride=0, complex=None):
        self._scale("scale_C", (exp_stats_buffer_A_id, exp_stats_buffer_B_id),
                    dynamic_launch_flag_buffer_id, m, n, ptr, ld, batch_size, stride, complex)

    def reset_scale_A(self, exp_stats_buffer_id, dynamic_launch_flag_buffer_id, m, n, ptr, ld,
                      batch_size=1, stride=0, complex=None):
        self._scale("reset_scale_A", (exp_stats_buffer_id,), dynamic_launch_flag_buffer_id, m, n,
                    ptr, ld, batch_size, stride, complex)

    def reset_scale_B(self, exp_stats_buffer_id, dynamic_launch_flag_buffer_id, m, n, ptr, ld,
                      batch_size=1, stride=0, complex=None):
        self._scale("reset_scale_B", (exp_stats_buffer_id,), dynamic_launch_flag_buffer_id, m, n,
                    ptr, ld, batch_size, stride, complex)

    # ------------------------------------------------------------------ dynamic launch
    def get_current_dynamic_launch_buffer_id(self) -> int:
        return self._lib.cuMpSGEMM_get_current_dynamic_launch_buffer_id(self._h)

    def get_next_dynamic_launch_buffer_id(self) -> int:
        return self._lib.cuMpSGEMM_get_next_dynamic_launch_buffer_id(self._h)

    def get_dynamic_launch_gemm_compute_mode(self, buffer_id: int) -> ComputeMode:
        return ComputeMode(self._lib.cuMpSGEMM_get_dynamic_launch_gemm_compute_mode(self._h,
                                                                                    buffer_id))

    def get_dynamic_launch_scaling_mode_AB(self, buffer_id: int) -> Tuple[int, int]:
        a, b = C.c_int(0), C.c_int(0)
        self._lib.cuMpSGEMM_get_dynamic_launch_scaling_mode_AB(self._h, buffer_id, C.byref(a),
                                                               C.byref(b))
        return a.value, b.value

    def set_dynamic_launch_buffer_by_exp_stats(self, dynamic_launch_buffer_id: int,
                                               A_exp_stats_buffer_id: int,
                                               B_exp_stats_buffer_id: int) -> None:
        self._lib.cuMpSGEMM_set_dynamic_launch_buffer_by_exp_stats(
            self._h, dynamic_launch_buffer_id, A_exp_stats_buffer_id, B_exp_stats_buffer_id)

    def set_dynamic_launch_flag_buffer_id(self, buffer_id: int) -> None:
        self._lib.cuMpSGEMM_set_dynamic_launch_flag_buffer_id(self._h, buffer_id)

    def unset_dynamic_launch_flag_buffer_id(self) -> None:
        self._lib.cuMpSGEMM_unset_dynamic_launch_flag_buffer_id(self._h)

    # ------------------------------------------------------------------ timers
    def enable_exp_stats_profiling(self) -> None:
        self._lib.cuMpSGEMM_enable_exp_stats_profiling(self._h)

    def disable_exp_stats_profiling(self) -> None:
        self._lib.cuMpSGEMM_disable_exp_stats_profiling(self._h)

    def reset_exp_stats_profiling(self) -> None:
        self._lib.cuMpSGEMM_reset_exp_stats_profiling(self._h)

    def get_exp_stats_profiling_result(self, name: str) -> Optional[Tuple[float, int]]:
        t, n = C.c_double(0), C.c_ulonglong(0)
        ok = self._lib.cuMpSGEMM_get_exp_stats_profiling_result(self._h, name.encode(),
                                                                C.byref(t), C.byref(n))
        return (t.value, n.value) if ok else None


def sgemm_static_scratch(stream, op_A: int, op_B: int, m: int, n: int, k: int, alpha, A: DevPtr,
                         lda: int, B: DevPtr, ldb: int, beta, Cmat: DevPtr, ldc: int,
                         mode: int) -> int:
    """cuMpSGEMM_sgemm_static_scratch: handle-free FP32 GEMM that allocates nothing.

    For callers that must not call cudaMalloc: the split operand panels go to a 32 MiB array
    built into the library (problems that need more are rejected with INVALID_VALUE).  Calls
    that overlap in time on one GPU race on that array; make the first call on a device
    outside any stream capture.  `stream` is a torch stream, a raw cudaStream_t or None.
    Returns the cublasStatus_t."""
    lib = _lib.load()
    s = 0 if stream is None else getattr(stream, "cuda_stream", stream)
    a, b = _scalar(alpha, False), _scalar(beta, False)
    return lib.cuMpSGEMM_sgemm_static_scratch(C.c_void_p(int(s)), op_A, op_B, m, n, k,
                                              C.cast(a, C.c_void_p), _ptr(A), lda, _ptr(B), ldb,
                                              C.cast(b, C.c_void_p), _ptr(Cmat), ldc, int(mode))


# ---------------------------------------------------------------------- convenience
def matmul(handle: Handle, A, B, mode: int = ComputeMode.FP16TCEC, out=None, alpha=1.0, beta=0.0):
    """Row-major ``A @ B`` for contiguous 2-D (or batched 3-D) torch CUDA tensors.

    A row-major (m, k) array is a column-major (k, m) one, so the product is
    computed as C^T = B^T A^T with the operands swapped and no data movement.
    """
    import torch

    if A.dim() == 2:
        m, k = A.shape
        k2, n = B.shape
        assert k == k2 and A.is_contiguous() and B.is_contiguous()
        if out is None:
            out = torch.empty((m, n), dtype=A.dtype, device=A.device)
        handle.gemm(CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, alpha, B, n, A, k, beta, out, n, mode)
        return out
    bsz, m, k = A.shape
    _, k2, n = B.shape
    assert k == k2 and A.is_contiguous() and B.is_contiguous()
    if out is None:
        out = torch.empty((bsz, m, n), dtype=A.dtype, device=A.device)
    handle.gemm_strided_batch(CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, alpha, B, n, k * n, A, k, m * k,
                              beta, out, n, m * n, bsz, mode)
    return out


class HostGemm:
    """GEMM on operands that live in (pinned) host memory.

    Each call copies A, B (and C when beta != 0) to the device, runs the GEMM and copies C
    back; device staging buffers are kept between calls.  This is the path a caller takes
    whose matrices are not resident on the GPU, e.g. a host BLAS client.

    With op_B == N the call is pipelined over column blocks of B and C: A is uploaded first,
    then for every block the upload of B_j / C_j (copy-in stream), the GEMM of the block (the
    handle's stream) and the download of C_j (copy-out stream) overlap, so that the call
    costs about the host-to-device transfer time alone.  The call is stream-ordered on the
    stream current at call time: work queued after it on that stream sees the result in
    C_host once that stream reaches it.
    """

    def __init__(self, handle: Handle, device=None, column_blocks: int = 16):
        import torch

        self.handle = handle
        self.torch = torch
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.column_blocks = max(1, int(column_blocks))
        self._bufs = {}
        self._streams = None

    def adopt_staging(self, A=None, B=None, C=None) -> None:
        """Use caller-owned device tensors as the staging buffers of A, B and C (same element
        count and dtype as the host operands passed to `gemm` later) instead of allocating
        new ones, e.g. buffers that already exist for a device-resident run of the same
        problem."""
        for key, t in (("A", A), ("B", B), ("C", C)):
            if t is not None:
                self._bufs[key] = t.reshape(-1)

    def _staging(self, key, host_tensor):
        t = self._bufs.get(key)
        if t is None or t.numel() != host_tensor.numel() or t.dtype != host_tensor.dtype:
            t = self.torch.empty(host_tensor.numel(), dtype=host_tensor.dtype, device=self.device)
            self._bufs[key] = t
        return t

    def gemm(self, op_A, op_B, m, n, k, alpha, A_host, lda, B_host, ldb, beta, C_host, ldc, mode,
             A_device=None, A_ready=None):
        """Returns (bytes copied host->device, bytes copied device->host).

        A_device: A is already (or is being made) resident in this device tensor, e.g. because
        another rank uploaded it and it arrives over NVLink; A_host is then ignored and not
        counted.  A_ready: event after which A_device holds the data; the uploads of B and C
        do not wait for it, only the GEMMs do."""
        torch = self.torch
        dA = A_device.reshape(-1) if A_device is not None else self._staging("A", A_host)
        dB = self._staging("B", B_host)
        dC = self._staging("C", C_host)
        b_flat, c_flat = B_host.reshape(-1), C_host.reshape(-1)
        a_flat = None if A_device is not None else A_host.reshape(-1)
        need_c = complex(beta) != 0
        es = B_host.element_size()
        h2d = ((a_flat.numel() if a_flat is not None else 0) + b_flat.numel() +
               (c_flat.numel() if need_c else 0)) * es
        d2h = c_flat.numel() * es
        blocks = self.column_blocks if (op_B == CUBLAS_OP_N and n >= 2 * self.column_blocks) else 1
        if blocks == 1:
            if a_flat is not None:
                dA.copy_(a_flat, non_blocking=True)
            elif A_ready is not None:
                torch.cuda.current_stream(self.device).wait_event(A_ready)
            dB.copy_(b_flat, non_blocking=True)
            if need_c:
                dC.copy_(c_flat, non_blocking=True)
            self.handle.gemm(op_A, op_B, m, n, k, alpha, dA, lda, dB, ldb, beta, dC, ldc, mode)
            c_flat.copy_(dC, non_blocking=True)
            return h2d, d2h

        if self._streams is None:
            self._streams = (torch.cuda.Stream(device=self.device),
                             torch.cuda.Stream(device=self.device),
                             torch.cuda.Stream(device=self.device))
        s_in, s_run, s_out = self._streams
        caller = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(caller)
        for st in (s_in, s_run, s_out):
            st.wait_event(start)
        self.handle.set_stream(s_run)
        if a_flat is not None:
            with torch.cuda.stream(s_in):
                dA.copy_(a_flat, non_blocking=True)
        elif A_ready is not None:
            s_run.wait_event(A_ready)
        per = -(-n // blocks)
        for j0 in range(0, n, per):
            j1 = min(n, j0 + per)
            bs, be = j0 * ldb, min(b_flat.numel(), j1 * ldb)
            cs, ce = j0 * ldc, min(c_flat.numel(), j1 * ldc)
            with torch.cuda.stream(s_in):
                dB[bs:be].copy_(b_flat[bs:be], non_blocking=True)
                if need_c:
                    dC[cs:ce].copy_(c_flat[cs:ce], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            s_run.wait_event(ready)
            self.handle.gemm(op_A, op_B, m, j1 - j0, k, alpha, dA, lda, dB[bs:], ldb, beta, dC[cs:],
                             ldc, mode)
            done = torch.cuda.Event()
            done.record(s_run)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                c_flat[cs:ce].copy_(dC[cs:ce], non_blocking=True)
        finished = torch.cuda.Event()
        finished.record(s_out)
        caller.wait_event(finished)
        self.handle.set_stream(caller)
        return h2d, d2h
