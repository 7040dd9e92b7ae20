"""numpy front end of the CPU oracle (``oracle.c``) and the seeded input generators.

TEST INFRASTRUCTURE ONLY.  Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import this
module; the product never does.

GEMM results of the emulation have no golden vectors in the reference
("parity unpinned" at bit level, see ``oracle.c``); the FP64 truth plus the
reference's own tolerance ``2^-23 * sqrt(K)`` (``test/main.cu:68-74``) is the
pinned criterion.  Statistics, decisions, flag words and scaling are restated
literally from the reference sources and are compared bit-exactly.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "liboracle.so"
REF_DIR = HERE / "_ref"

OP_N, OP_T, OP_C = 0, 1, 2
FP16TCEC, TF32TCEC, UNDEFINED, FP16TCEC_SCALING = 1, 2, 10, 11

_lib = None


class _Stats(C.Structure):
    _fields_ = [("max_exp", C.c_float), ("total", C.c_ulonglong), ("underflow", C.c_ulonglong),
                ("mode", C.c_int)]


def reference_tree():
    """Root of a checkout of the reference project, or None.  Taken from the environment
    variable CUMPSGEMM_REFERENCE_TREE; without it, a sibling directory `reference` of this
    repository is used when it exists."""
    env = os.environ.get("CUMPSGEMM_REFERENCE_TREE")
    cand = Path(env) if env else HERE.parent.parent / "reference"
    return cand if (cand / "src" / "exp_stats.cu").exists() else None


def build(with_ref: bool = False) -> None:
    """Compile liboracle.so (and, when asked and possible, the reference-derived objects)."""
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    ref = reference_tree()
    if with_ref and ref is not None:
        subprocess.run(["make", "-C", str(HERE), "ref", "ref_gpu", f"REF={ref}"], check=True,
                       capture_output=True)


def lib():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(LIB_PATH))
        _lib.oracle_residual.restype = C.c_double
        _lib.oracle_exp_max.restype = C.c_float
        _lib.oracle_flag_from_modes.restype = C.c_int
    return _lib


def set_num_threads(n: int) -> int:
    """Use `n` OpenMP threads in the oracle's loops (whatever OMP_NUM_THREADS says) and return
    the number the runtime then reports."""
    L = lib()
    L.oracle_set_num_threads(int(n))
    return int(L.oracle_get_max_threads())


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _as_f32(a: np.ndarray) -> np.ndarray:
    """Column-major arrays are passed as their flat storage; complex64 as interleaved floats."""
    a = np.ascontiguousarray(a) if not a.flags.f_contiguous and a.ndim == 1 else a
    if a.dtype == np.complex64:
        return a.view(np.float32)
    assert a.dtype == np.float32
    return a


# ------------------------------------------------------------------------ GEMM truth
def gemm_f64(op_a, op_b, m, n, k, alpha, a, lda, b, ldb, beta, c_in, ldc) -> np.ndarray:
    """FP64 result of alpha*op(A)op(B)+beta*C as an (m, n) Fortran-ordered array.

    a, b, c_in are flat storage arrays (float32 or complex64), column-major with the
    given leading dimensions.
    """
    L = lib()
    cplx = a.dtype == np.complex64
    if not cplx:
        out = np.empty(m * n, dtype=np.float64)
        L.oracle_gemm_f64(op_a, op_b, C.c_size_t(m), C.c_size_t(n), C.c_size_t(k),
                          C.c_double(alpha), _fp(a), C.c_size_t(lda), _fp(b), C.c_size_t(ldb),
                          C.c_double(beta), _fp(c_in) if c_in is not None else None,
                          C.c_size_t(ldc), _fp(out))
        return out.reshape((m, n), order="F")
    al, be = complex(alpha), complex(beta)
    out = np.empty(m * n, dtype=np.complex128)
    L.oracle_cgemm_f64(op_a, op_b, C.c_size_t(m), C.c_size_t(n), C.c_size_t(k),
                       C.c_double(al.real), C.c_double(al.imag), _fp(a), C.c_size_t(lda), _fp(b),
                       C.c_size_t(ldb), C.c_double(be.real), C.c_double(be.imag),
                       _fp(c_in) if c_in is not None else None, C.c_size_t(ldc), _fp(out))
    return out.reshape((m, n), order="F")


def residual(truth: np.ndarray, result: np.ndarray, ldr: int) -> float:
    """Relative Frobenius residual sqrt(sum|t-r|^2 / sum|t|^2) (reference: test/main.cu:196-228).

    truth: (m, n) Fortran array float64/complex128; result: flat float32/complex64 storage."""
    m, n = truth.shape
    fpe = 2 if np.iscomplexobj(truth) else 1
    t = np.asfortranarray(truth)
    return float(lib().oracle_residual(_fp(t), _fp(result), C.c_size_t(m), C.c_size_t(n),
                                       C.c_size_t(ldr), fpe))


def relative_errors(truth: np.ndarray, result: np.ndarray, ldr: int):
    """(max, mean) element-wise relative error against the FP64 truth (real matrices)."""
    m, n = truth.shape
    mx, mean = C.c_double(0), C.c_double(0)
    t = np.asfortranarray(truth)
    lib().oracle_relative_errors(_fp(t), _fp(result), C.c_size_t(m), C.c_size_t(n),
                                 C.c_size_t(ldr), C.byref(mx), C.byref(mean))
    return mx.value, mean.value


def error_threshold(mode_has_ec: bool, k: int) -> float:
    """The reference's pass criterion (test/main.cu:68-74)."""
    return (2.0 ** -23 if mode_has_ec else 2.0 ** -10) * np.sqrt(k)


# ------------------------------------------------------------------------ FP32 host GEMM
def gemm_f32(op_a, op_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc) -> None:
    """In-place FP32 host GEMM on flat column-major storage (the CPU baseline)."""
    L = lib()
    if a.dtype == np.complex64:
        al, be = complex(alpha), complex(beta)
        L.oracle_cgemm_f32(op_a, op_b, C.c_size_t(m), C.c_size_t(n), C.c_size_t(k),
                           C.c_float(al.real), C.c_float(al.imag), _fp(a), C.c_size_t(lda),
                           _fp(b), C.c_size_t(ldb), C.c_float(be.real), C.c_float(be.imag),
                           _fp(c), C.c_size_t(ldc))
    else:
        L.oracle_sgemm_f32(op_a, op_b, C.c_size_t(m), C.c_size_t(n), C.c_size_t(k),
                           C.c_float(alpha), _fp(a), C.c_size_t(lda), _fp(b), C.c_size_t(ldb),
                           C.c_float(beta), _fp(c), C.c_size_t(ldc))


def tiny_gemm_f32(long_is_m: bool, op_a, op_b, length, alpha, a, lda, b, ldb, beta, c, ldc,
                  stride_a=0, stride_b=0, stride_c=0, batch=1) -> None:
    """In-place FP32 GEMM with two-by-two inner problem on flat column-major storage, in the
    operation order of the device kernel (bit-exact comparison)."""
    cplx = a.dtype == np.complex64
    al, be = complex(alpha), complex(beta)
    lib().oracle_tiny_gemm_f32(1 if long_is_m else 0, op_a, op_b, C.c_size_t(length),
                               C.c_float(al.real), C.c_float(al.imag), _fp(a), C.c_size_t(lda),
                               C.c_size_t(stride_a), _fp(b), C.c_size_t(ldb),
                               C.c_size_t(stride_b), C.c_float(be.real), C.c_float(be.imag),
                               _fp(c), C.c_size_t(ldc), C.c_size_t(stride_c), C.c_size_t(batch),
                               2 if cplx else 1)


# ------------------------------------------------------------------------ TCEC model
def split(x: np.ndarray, kind: int):
    """(hi, lo) of every float32 value; kind 0 = FP16 (lo scaled by 2^11), 1 = TF32."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    hi = np.empty_like(x)
    lo = np.empty_like(x)
    lib().oracle_split(_fp(x), C.c_size_t(x.size), kind, _fp(hi), _fp(lo))
    return hi, lo


def tcec_model(kind, op_a, op_b, m, n, k, alpha, a, lda, b, ldb, beta, c_in, ldc,
               k_chunk=64) -> np.ndarray:
    out = np.empty(m * n, dtype=np.float32)
    lib().oracle_tcec_model(kind, op_a, op_b, C.c_size_t(m), C.c_size_t(n), C.c_size_t(k),
                            C.c_float(alpha), _fp(a), C.c_size_t(lda), _fp(b), C.c_size_t(ldb),
                            C.c_float(beta), _fp(c_in) if c_in is not None else None,
                            C.c_size_t(ldc), C.c_size_t(k_chunk), _fp(out))
    return out.reshape((m, n), order="F")


# ------------------------------------------------------------------------ statistics
def exp_stats(x: np.ndarray, m, n, ld, batch=1, stride=0, ignore_threshold=0.0,
              underflow_threshold=2.0 ** -15, tolerance=0.0, count_padding=False):
    """dict(max_exp, total, underflow, mode) exactly as the device pipeline leaves a slot."""
    fpe = 2 if x.dtype == np.complex64 else 1
    s = _Stats()
    lib().oracle_exp_stats(_fp(x), C.c_size_t(m), C.c_size_t(n), C.c_size_t(ld), C.c_size_t(batch),
                           C.c_size_t(stride), fpe, C.c_float(ignore_threshold),
                           C.c_float(underflow_threshold), C.c_float(tolerance),
                           1 if count_padding else 0, C.byref(s))
    return {"max_exp": float(s.max_exp), "total": int(s.total), "underflow": int(s.underflow),
            "mode": int(s.mode)}


def exp_max(x: np.ndarray, m, n, ld, batch=1, stride=0) -> float:
    fpe = 2 if x.dtype == np.complex64 else 1
    return float(lib().oracle_exp_max(_fp(x), C.c_size_t(m), C.c_size_t(n), C.c_size_t(ld),
                                      C.c_size_t(batch), C.c_size_t(stride), fpe))


def flag_from_modes(mode_a: int, mode_b: int) -> int:
    return int(lib().oracle_flag_from_modes(mode_a, mode_b))


SCALE_A, SCALE_B, SCALE_C, RESET_A, RESET_B = 0, 1, 2, 3, 4


def scale(what: int, x: np.ndarray, m, n, ld, batch, stride, flag, max_a: float,
          max_b: float = 0.0) -> None:
    """In-place scaling of flat storage `x` (float32 or complex64)."""
    fpe = 2 if x.dtype == np.complex64 else 1
    use_flag = 0 if flag is None else 1
    lib().oracle_scale(what, _fp(x), C.c_size_t(m), C.c_size_t(n), C.c_size_t(ld),
                       C.c_size_t(batch), C.c_size_t(stride), fpe, use_flag,
                       0 if flag is None else int(flag), C.c_float(max_a), C.c_float(max_b))


# ------------------------------------------------------------------------ seeded inputs
def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def gen_uniform(seed, count):
    """i.i.d. uniform(-1, 1) float32 (benchmark config: the reference's `sgemm` case)."""
    return rng(seed).uniform(-1.0, 1.0, size=count).astype(np.float32)


def gen_normal(seed, count):
    """i.i.d. N(0,1) float32 (the reference's own test inputs, test/main.cu:552-558)."""
    return rng(seed).standard_normal(size=count, dtype=np.float32)


def gen_uniform_exp(seed, count, lo=-8, hi=8):
    """uniform(-1,1) * 2^e with e uniform over the integers [lo, hi] per element."""
    g = rng(seed)
    u = g.uniform(-1.0, 1.0, size=count).astype(np.float32)
    e = g.integers(lo, hi + 1, size=count)
    return np.ldexp(u, e).astype(np.float32)


def gen_wide_exponent(seed, count, lo=-30, hi=10):
    """sign uniform, mantissa uniform in [1,2), exponent uniform over the integers [lo, hi]."""
    g = rng(seed)
    s = np.where(g.integers(0, 2, size=count) == 0, -1.0, 1.0)
    f = 1.0 + g.uniform(0.0, 1.0, size=count)
    e = g.integers(lo, hi + 1, size=count)
    return np.ldexp(s * f, e).astype(np.float32)


def gen_unit_frobenius_complex(seed, batch, rows, cols):
    """complex Gaussian matrices, each divided by its Frobenius norm; flat (batch*rows*cols)."""
    g = rng(seed)
    re = g.standard_normal(size=(batch, rows * cols), dtype=np.float32)
    im = g.standard_normal(size=(batch, rows * cols), dtype=np.float32)
    z = (re + 1j * im).astype(np.complex64)
    nrm = np.sqrt((np.abs(z.astype(np.complex128)) ** 2).sum(axis=1, keepdims=True))
    return (z / nrm).astype(np.complex64).ravel()


# ------------------------------------------------------------------------ the reference itself
class ReferenceStats:
    """The reference's own statistics / scaling / flag code running on the GPU.

    ``_ref/libref_stats.so`` is the reference's src/exp_stats.cu, src/dynamic_scaling.cu and
    src/dynamic_launch.cu compiled unmodified for sm_100a (``make ref_gpu``; only where the
    reference tree is available, the built library then travels with the repository).  Device
    buffers are passed as raw addresses; every getter synchronises.  Checker only.
    """

    PATH = REF_DIR / "libref_stats.so"

    @classmethod
    def available(cls) -> bool:
        return cls.PATH.exists()

    def __init__(self):
        L = C.CDLL(str(self.PATH))
        vp, u32 = C.c_void_p, C.c_uint
        L.ref_create.restype = vp
        L.ref_destroy.argtypes = [vp]
        L.ref_set_exp_stats_params.argtypes = [vp, C.c_float, C.c_float, C.c_float]
        for name in ("ref_exp_stats_ext_s", "ref_exp_stats_ext_c", "ref_exp_max_ext_s",
                     "ref_exp_max_ext_c"):
            fn = getattr(L, name)
            fn.restype = u32
            fn.argtypes = [vp, u32, u32, vp, u32, u32, u32]
        L.ref_get_exp_stats.argtypes = [vp, u32, C.POINTER(C.c_ulonglong),
                                        C.POINTER(C.c_ulonglong)]
        L.ref_get_max_exp.restype = C.c_float
        L.ref_get_max_exp.argtypes = [vp, u32]
        L.ref_get_compute_mode_level.restype = C.c_int
        L.ref_get_compute_mode_level.argtypes = [vp, u32]
        L.ref_next_flag_id.restype = u32
        L.ref_next_flag_id.argtypes = [vp]
        L.ref_set_flag_by_exp_stats.argtypes = [vp, u32, u32, u32]
        L.ref_get_flag.restype = C.c_int
        L.ref_get_flag.argtypes = [vp, u32]
        for name in ("ref_scale_s", "ref_scale_c"):
            getattr(L, name).argtypes = [vp, C.c_int, u32, u32, vp, u32, u32, u32, u32, u32, u32]
        self._L = L
        self._h = vp(L.ref_create())

    def close(self):
        if self._h:
            self._L.ref_destroy(self._h)
            self._h = None

    def set_exp_stats_params(self, ignore_threshold, underflow_threshold, tolerance):
        self._L.ref_set_exp_stats_params(self._h, ignore_threshold, underflow_threshold, tolerance)

    def exp_stats_ext(self, m, n, dev_ptr: int, ld, batch=1, stride=0, complex=False) -> int:
        fn = self._L.ref_exp_stats_ext_c if complex else self._L.ref_exp_stats_ext_s
        return fn(self._h, m, n, dev_ptr, ld, batch, stride)

    def exp_max_ext(self, m, n, dev_ptr: int, ld, batch=1, stride=0, complex=False) -> int:
        fn = self._L.ref_exp_max_ext_c if complex else self._L.ref_exp_max_ext_s
        return fn(self._h, m, n, dev_ptr, ld, batch, stride)

    def slot(self, sid: int) -> dict:
        uf, total = C.c_ulonglong(0), C.c_ulonglong(0)
        self._L.ref_get_exp_stats(self._h, sid, C.byref(uf), C.byref(total))
        return {"max_exp": float(self._L.ref_get_max_exp(self._h, sid)), "total": total.value,
                "underflow": uf.value, "mode": int(self._L.ref_get_compute_mode_level(self._h, sid))}

    def max_exp(self, sid: int) -> float:
        return float(self._L.ref_get_max_exp(self._h, sid))

    def flag_from_stats(self, sid_a: int, sid_b: int):
        """(flag id, flag word) after set_dynamic_launch_buffer_by_exp_stats on a fresh slot."""
        fid = self._L.ref_next_flag_id(self._h)
        self._L.ref_set_flag_by_exp_stats(self._h, fid, sid_a, sid_b)
        return fid, int(self._L.ref_get_flag(self._h, fid))

    def flag(self, fid: int) -> int:
        return int(self._L.ref_get_flag(self._h, fid))

    def scale(self, what: int, m, n, dev_ptr: int, ld, batch, stride, sid_a, sid_b, flag_id,
              complex=False):
        """what: SCALE_A, SCALE_B, SCALE_C, RESET_A, RESET_B (in place, on the device)."""
        fn = self._L.ref_scale_c if complex else self._L.ref_scale_s
        fn(self._h, what, m, n, dev_ptr, ld, batch, stride, sid_a, sid_b, flag_id)
