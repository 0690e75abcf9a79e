"""TEST INFRASTRUCTURE — Python face of the CPU oracle for the SGEMM path.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module.  It is the checker, never the product: nothing under the
shipped package imports it and there is no CPU fallback for the GPU path.

Parity is pinned: the restated arithmetic is checked against outputs of the
reference's own generator + GCN virtual machine (committed under
``tests/golden/``, produced by ``tests/golden/make_golden.py``) and against the
known-answer inputs the reference's tests use (test/test_vm.py:447-627).

Restated from the reference (paths relative to that project):

* ``runner/generator_runner.cpp:16-33``   cpuGemm arithmetic and indexing
* ``runner/generator_runner.cpp:133-148`` lda=M, ldb=K, ldc=ldd=M
* ``runner/Utils/Math.hpp:5-8``           |x-y| < delta comparison
* ``runner/generator_runner.cpp:75-83``   Gflops / "GiB/s" formulas
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "liboracle.so"
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_u32 = ctypes.c_uint32
_u64 = ctypes.c_uint64


def build(force: bool = False) -> Path:
    """Compile ``cpu_gemm.c`` with the Makefile beside it (gcc, OpenMP)."""
    src = _HERE / "cpu_gemm.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", str(_HERE), "-s", "-B"], check=True, env=env)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        gemm_args = [_f32p, _f32p, _f32p, _f32p, ctypes.c_float, ctypes.c_float,
                     _u32, _u32, _u32, _u32, _u32, _u32, _u32]
        L.oracle_gemm.argtypes = gemm_args
        L.oracle_gemm.restype = None
        L.oracle_gemm_ref_order.argtypes = gemm_args
        L.oracle_gemm_ref_order.restype = None
        L.oracle_gemm_f64.argtypes = [_f32p, _f32p, _f32p, _f64p, ctypes.c_float, ctypes.c_float,
                                      _u32, _u32, _u32, _u32, _u32, _u32, _u32]
        L.oracle_gemm_f64.restype = None
        L.oracle_abs_bound.argtypes = [_f32p, _f32p, _f64p, _u32, _u32, _u32, _u32, _u32, _u32]
        L.oracle_abs_bound.restype = None
        L.oracle_fill_uniform.argtypes = [_f32p, _u64, _u64, _u64]
        L.oracle_fill_uniform.restype = None
        L.oracle_count_mismatches.argtypes = [_f32p, _f32p, _u64, ctypes.c_float]
        L.oracle_count_mismatches.restype = _u64
        L.oracle_worst_ratio.argtypes = [_f32p, _f32p, _f64p, _u64, ctypes.c_double]
        L.oracle_worst_ratio.restype = ctypes.c_double
        L.oracle_set_num_threads.argtypes = [ctypes.c_int]
        L.oracle_set_num_threads.restype = None
        L.oracle_num_threads.argtypes = []
        L.oracle_num_threads.restype = ctypes.c_int
        L.oracle_gflops.argtypes = [_u32, _u32, _u32, ctypes.c_double]
        L.oracle_gflops.restype = ctypes.c_double
        L.oracle_mem_bw.argtypes = [_u64, _u64, _u64, ctypes.c_double]
        L.oracle_mem_bw.restype = ctypes.c_double
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Use every core this process may run on, whatever OMP_NUM_THREADS says (torchrun exports 1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(n)
    return num_threads()


def _p32(x: np.ndarray):
    assert x.dtype == np.float32 and x.flags.c_contiguous
    return x.ctypes.data_as(_f32p)


def _p64(x: np.ndarray):
    assert x.dtype == np.float64 and x.flags.c_contiguous
    return x.ctypes.data_as(_f64p)


# --------------------------------------------------------------------------
# seeded inputs: index-hash generator, uniform on [-1, 1) with 24-bit steps
# --------------------------------------------------------------------------
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def fill_uniform_numpy(count: int, stream: int, first_index: int = 0) -> np.ndarray:
    """NumPy restatement of ``oracle_fill_uniform`` (bit-identical)."""
    with np.errstate(over="ignore"):
        idx = np.arange(first_index, first_index + count, dtype=np.uint64)
        x = idx + np.uint64((0x9E3779B97F4A7C15 * (stream + 1)) & 0xFFFFFFFFFFFFFFFF)
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return ((x >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -23) - np.float32(1.0)).astype(np.float32)


def fill_uniform(count: int, stream: int, first_index: int = 0) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    lib().oracle_fill_uniform(_p32(out), count, first_index, stream)
    return out


def make_inputs(m: int, n: int, k: int, seed: int = 0, lda=None, ldb=None, ldc=None):
    """A (stream seed), B (seed+1), C (seed+2) as flat column-major buffers.

    Element (i, j) of a matrix with leading dimension ld lives at i + j*ld and
    takes the generator's value for *logical* index i + j*rows, so the data do
    not depend on the padding."""
    lda = lda or m
    ldb = ldb or k
    ldc = ldc or m

    def mat(rows, cols, ld, stream):
        dense = fill_uniform(rows * cols, stream)
        if ld == rows:
            return dense
        buf = np.zeros(ld * cols, dtype=np.float32)
        buf.reshape(cols, ld)[:, :rows] = dense.reshape(cols, rows)
        return buf

    return mat(m, k, lda, seed), mat(k, n, ldb, seed + 1), mat(m, n, ldc, seed + 2)


# --------------------------------------------------------------------------
# GEMM restatements
# --------------------------------------------------------------------------
def gemm(a, b, c, alpha, beta, m, n, k, lda=None, ldb=None, ldc=None, ldd=None, ref_order=False):
    """cpuGemm arithmetic on flat column-major FP32 buffers; returns flat D."""
    lda = lda or m
    ldb = ldb or k
    ldc = ldc or m
    ldd = ldd or m
    d = np.zeros(max(ldd * n, 1), dtype=np.float32)
    fn = lib().oracle_gemm_ref_order if ref_order else lib().oracle_gemm
    cp = _p32(c) if c is not None else ctypes.cast(None, _f32p)
    fn(_p32(a), _p32(b), cp, _p32(d), alpha, beta, m, n, k, lda, ldb, ldc, ldd)
    return d[: ldd * n]


def gemm_python(a, b, c, alpha, beta, m, n, k):
    """Pure-Python loop nest of cpuGemm with NumPy float32 scalars (tiny cases only)."""
    f = np.float32
    d = np.zeros(m * n, dtype=np.float32)
    alpha, beta = f(alpha), f(beta)
    for i in range(m):
        for j in range(n):
            acc = f(0.0)
            for l in range(k):
                acc = f(acc + f(a[i + l * m] * b[l + j * k]))
            d[i + j * m] = f(f(beta * c[i + j * m]) + f(alpha * acc))
    return d


def gemm_f64(a, b, c, alpha, beta, m, n, k, lda=None, ldb=None, ldc=None):
    lda = lda or m
    ldb = ldb or k
    ldc = ldc or m
    d = np.zeros(max(m * n, 1), dtype=np.float64)
    cp = _p32(c) if c is not None else ctypes.cast(None, _f32p)
    lib().oracle_gemm_f64(_p32(a), _p32(b), cp, _p64(d), alpha, beta, m, n, k, lda, ldb, ldc, m)
    return d[: m * n]


def abs_bound(a, b, m, n, k, lda=None, ldb=None):
    """S[i + j*m] = sum_l |a_il| |b_lj| (FP64) — the scale of the parity tolerance."""
    lda = lda or m
    ldb = ldb or k
    s = np.zeros(max(m * n, 1), dtype=np.float64)
    lib().oracle_abs_bound(_p32(a), _p32(b), _p64(s), m, n, k, lda, ldb, m)
    return s[: m * n]


REL_TOL = 1e-5  # max|D - D_ref| <= REL_TOL * sum_l |a_il||b_lj| per element


def worst_ratio(x, ref, s, rel=REL_TOL) -> float:
    """max over elements of |x-ref| / (rel*S); parity holds iff the result is <= 1."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    ref = np.ascontiguousarray(ref, dtype=np.float32)
    s = np.ascontiguousarray(s, dtype=np.float64)
    assert x.size == ref.size == s.size
    return float(lib().oracle_worst_ratio(_p32(x), _p32(ref), _p64(s), x.size, rel))


def strip_ld(flat, rows, cols, ld):
    """Dense rows x cols (flat, column-major) view of a buffer with leading dimension ld."""
    if ld == rows:
        return np.ascontiguousarray(flat[: rows * cols])
    return np.ascontiguousarray(flat[: ld * cols].reshape(cols, ld)[:, :rows]).reshape(-1)


def count_mismatches(x, y, delta=1e-3) -> int:
    """The reference runner's own validation rule (abs diff, default 1e-3)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.ascontiguousarray(y, dtype=np.float32)
    return int(lib().oracle_count_mismatches(_p32(x), _p32(y), x.size, delta))


def gflops(m, n, k, ms):
    return float(lib().oracle_gflops(m, n, k, ms))


def mem_bw(m, n, k, ms):
    return float(lib().oracle_mem_bw(m, n, k, ms))
