"""ctypes binding of libsgemm_runner.so (the C ABI declared in include/sgemm_runner.h).

This is the Python face of the runner: the calls the reference makes inside its C++ runner program
(runner/generator_runner.cpp:69-190 — load the code object, read the TOML, pack arguments, launch) are
reachable from Python here, so tests and the benchmark drive exactly the path a C caller would.

There is no CPU implementation behind this module: when the shared library has not been built, or no
CUDA driver / device is present, the calls raise ``SgemmError``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path
from typing import Optional, Tuple

PKG_DIR = Path(__file__).resolve().parent.parent
LIB_PATH = PKG_DIR / "build" / "libsgemm_runner.so"
RUNNER_PATH = PKG_DIR / "build" / "GeneratorRunner"

_f32p = ctypes.POINTER(ctypes.c_float)
_u32 = ctypes.c_uint32
_u64 = ctypes.c_uint64
_vp = ctypes.c_void_p


class SgemmConfig(ctypes.Structure):
    """Mirror of ``struct sgemm_config``."""
    _fields_ = [
        ("a_type", ctypes.c_int32), ("b_type", ctypes.c_int32), ("cd_type", ctypes.c_int32), ("scalar_type", ctypes.c_int32),
        ("mfma", ctypes.c_int32 * 4), ("wave_group", ctypes.c_int32 * 2), ("wave_tiling", ctypes.c_int32 * 2),
        ("depth_k", ctypes.c_int32), ("vmem_stage", ctypes.c_int32), ("wavefront_size", ctypes.c_int32),
        ("lds_usage_bytes", ctypes.c_int32), ("trans_a", ctypes.c_int32), ("trans_b", ctypes.c_int32),
        ("variant", ctypes.c_int32), ("num_threads", ctypes.c_int32), ("dynamic_smem_bytes", ctypes.c_int32),
        ("stages", ctypes.c_int32), ("a_kmajor", ctypes.c_int32), ("split_inkernel", ctypes.c_int32),
        ("fallback_tile", ctypes.c_int32 * 3),
        ("fallback_threads", ctypes.c_int32), ("entry", ctypes.c_char * 64), ("fallback_entry", ctypes.c_char * 64),
        ("skinny_tile", ctypes.c_int32 * 3), ("skinny_threads", ctypes.c_int32), ("skinny_smem_bytes", ctypes.c_int32),
        ("skinny_entry", ctypes.c_char * 64), ("acc_chain", ctypes.c_int32), ("skinny_acc_chain", ctypes.c_int32),
        ("wholek_entry", ctypes.c_char * 64),
        ("thin_tile", ctypes.c_int32 * 3), ("thin_threads", ctypes.c_int32), ("thin_smem_bytes", ctypes.c_int32),
        ("thin_acc_chain", ctypes.c_int32), ("thin_entry", ctypes.c_char * 64),
        ("feed_tma", ctypes.c_int32),
    ]


class SgemmError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str):
        super().__init__(f"{what}: {detail} [code {code}]")
        self.code = code


# every symbol include/sgemm_runner.h declares: name -> (restype, argtypes)
_GEMM_ARGS = [_vp, _vp, _vp, _vp, _vp, ctypes.c_float, ctypes.c_float, _u32, _u32, _u32, _u32, _u32, _u32, _u32]
ABI = {
    "sgemm_config_parse": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(SgemmConfig)]),
    "sgemm_config_tile": (ctypes.c_int, [ctypes.POINTER(SgemmConfig), ctypes.POINTER(_u32), ctypes.POINTER(_u32)]),
    "sgemm_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(_vp)]),
    "sgemm_close": (ctypes.c_int, [_vp]),
    "sgemm_launch": (ctypes.c_int, _GEMM_ARGS + [_vp]),
    "sgemm_launch_noalloc": (ctypes.c_int, _GEMM_ARGS + [_vp]),
    "sgemm_noalloc_scratch_bytes": (ctypes.c_size_t, []),
    "sgemm_run_host": (ctypes.c_int, _GEMM_ARGS),
    "sgemm_run_host_sharded": (ctypes.c_int, _GEMM_ARGS),
    "sgemm_shard_columns": (ctypes.c_int, [_u32, _u32, _u32, _u32, ctypes.POINTER(_u32), ctypes.POINTER(_u32)]),
    "sgemm_comm_unique_id": (ctypes.c_int, [ctypes.c_char_p]),
    "sgemm_comm_init": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]),
    "sgemm_comm_init_all": (ctypes.c_int, [ctypes.POINTER(_vp), ctypes.c_int]),
    "sgemm_comm_destroy": (ctypes.c_int, [_vp]),
    "sgemm_allgather_columns": (ctypes.c_int, [_vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "sgemm_bench": (ctypes.c_int, _GEMM_ARGS + [_u32, _u32, _vp, ctypes.POINTER(ctypes.c_float)]),
    "sgemm_last_status": (ctypes.c_int, [_vp, ctypes.POINTER(_u32 * 8)]),
    "sgemm_wait_selftest": (ctypes.c_int, [_vp, _u32, _u32]),
    "sgemm_set_option": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_int64]),
    "sgemm_get_info": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int64)]),
    "sgemm_workspace_bytes": (ctypes.c_int, [_vp, _u32, _u32, _u32, _u32, _u32, ctypes.POINTER(ctypes.c_size_t)]),
    "sgemm_workspace_bytes_for": (ctypes.c_int, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, ctypes.POINTER(ctypes.c_size_t)]),
    "sgemm_set_workspace": (ctypes.c_int, [_vp, _vp, ctypes.c_size_t]),
    "sgemm_fill_uniform": (ctypes.c_int, [_vp, _vp, _u64, _u64, _u64, _vp]),
    "sgemm_narrow16": (ctypes.c_int, [_vp, _vp, _vp, _u64, _vp]),
    "sgemm_tile_map": (ctypes.c_int, [_vp, ctypes.POINTER(ctypes.c_int32), _u32, _u32]),
    "sgemm_dev_alloc": (ctypes.c_int, [_vp, ctypes.c_size_t, ctypes.POINTER(_vp)]),
    "sgemm_dev_free": (ctypes.c_int, [_vp, _vp]),
    "sgemm_dev_upload": (ctypes.c_int, [_vp, _vp, _vp, ctypes.c_size_t]),
    "sgemm_dev_download": (ctypes.c_int, [_vp, _vp, _vp, ctypes.c_size_t]),
    "sgemm_dev_memset": (ctypes.c_int, [_vp, _vp, ctypes.c_int, ctypes.c_size_t]),
    "sgemm_dev_sync": (ctypes.c_int, [_vp]),
    "sgemm_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "sgemm_last_error": (ctypes.c_char_p, [_vp]),
    "sgemm_device_count": (ctypes.c_int, []),
}

_lib: Optional[ctypes.CDLL] = None


def build_library(force: bool = False) -> Path:
    """Run the Makefile beside this file (g++ and nvcc; needs the CUDA toolkit headers, not a GPU)."""
    if force or not LIB_PATH.exists() or not RUNNER_PATH.exists():
        env = dict(os.environ)
        env.pop("CXX", None)
        subprocess.run(["make", "-C", str(Path(__file__).resolve().parent), "-s"] + (["-B"] if force else []),
                       check=True, env=env)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise SgemmError(-5, "libsgemm_runner.so", f"{LIB_PATH} is not built; run __graft_entry__.build() "
                                                        f"or make -C {PKG_DIR / 'runner'}")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in ABI.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def parse_config(toml_path: str) -> SgemmConfig:
    cfg = SgemmConfig()
    rc = lib().sgemm_config_parse(str(toml_path).encode(), ctypes.byref(cfg))
    if rc:
        raise SgemmError(rc, "sgemm_config_parse", lib().sgemm_last_error(None).decode())
    return cfg


def config_tile(cfg: SgemmConfig) -> Tuple[int, int]:
    tm, tn = _u32(), _u32()
    lib().sgemm_config_tile(ctypes.byref(cfg), ctypes.byref(tm), ctypes.byref(tn))
    return tm.value, tn.value


def _ptr(x) -> int:
    """Device/host address of a torch tensor, a NumPy array, an int, or None."""
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)}")


class SgemmRunner:
    """One loaded kernel on one device (wraps ``sgemm_handle``)."""

    AUTO, TENSOR, SIMT, TENSOR_SKINNY = 0, 1, 2, 3

    def __init__(self, cubin_path: str, toml_path: str, device: int = 0):
        self._L = lib()
        self._h = _vp()
        rc = self._L.sgemm_open(str(cubin_path).encode(), str(toml_path).encode(), device, ctypes.byref(self._h))
        if rc:
            self._h = None
            raise SgemmError(rc, "sgemm_open", self._L.sgemm_last_error(None).decode())
        self.device = device

    # ---------------------------------------------------------------------------------- plumbing
    def _check(self, rc: int, what: str):
        if rc:
            raise SgemmError(rc, what, self._L.sgemm_last_error(self._h).decode())

    def close(self):
        if self._h:
            self._L.sgemm_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _lds(m, n, k, lda, ldb, ldc, ldd):
        return (lda or max(m, 1), ldb or max(k, 1), ldc or max(m, 1), ldd or max(m, 1))

    # ----------------------------------------------------------------------------------- compute
    def launch(self, a, b, c, d, m, n, k, alpha=1.0, beta=0.0, lda=0, ldb=0, ldc=0, ldd=0, stream=0):
        """Asynchronous D = alpha*A*B + beta*C on device buffers (tensors, arrays' addresses or ints)."""
        lda, ldb, ldc, ldd = self._lds(m, n, k, lda, ldb, ldc, ldd)
        self._check(self._L.sgemm_launch(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), alpha, beta, m, n, k,
                                         lda, ldb, ldc, ldd, stream), "sgemm_launch")

    def launch_noalloc(self, a, b, c, d, m, n, k, alpha=1.0, beta=0.0, lda=0, ldb=0, ldc=0, ldd=0, stream=0):
        """``launch`` for callers that must not allocate device memory: the scratch comes from the library's
        fixed array (``noalloc_scratch_bytes()``); larger problems raise ``SgemmError`` with code -9."""
        lda, ldb, ldc, ldd = self._lds(m, n, k, lda, ldb, ldc, ldd)
        self._check(self._L.sgemm_launch_noalloc(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), alpha, beta, m, n, k,
                                                 lda, ldb, ldc, ldd, stream), "sgemm_launch_noalloc")

    def run_host(self, a, b, c, d, m, n, k, alpha=1.0, beta=0.0, lda=0, ldb=0, ldc=0, ldd=0):
        """The same with HOST buffers (upload, launch, download, synchronise)."""
        lda, ldb, ldc, ldd = self._lds(m, n, k, lda, ldb, ldc, ldd)
        self._check(self._L.sgemm_run_host(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), alpha, beta, m, n, k,
                                           lda, ldb, ldc, ldd), "sgemm_run_host")

    def run_host_sharded(self, a, b, c, d, m, n_local, k, alpha=1.0, beta=0.0, lda=0, ldb=0, ldc=0, ldd=0):
        """``run_host`` for one rank of a column-sharded call: ``a`` is the whole replicated A in host memory (only this
        rank's slice is uploaded, the ranks complete each other's copies over NVLink), ``b``, ``c``, ``d`` are this
        rank's column shards.  Collective over the handle's communicator (``comm_init``)."""
        lda, ldb, ldc, ldd = self._lds(m, n_local, k, lda, ldb, ldc, ldd)
        self._check(self._L.sgemm_run_host_sharded(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), alpha, beta, m, n_local, k,
                                                   lda, ldb, ldc, ldd), "sgemm_run_host_sharded")

    # ------------------------------------------------------------------------------- multi-GPU
    def comm_init(self, comm_id: bytes, rank: int, world: int):
        """Join the communicator ``comm_id`` (from ``comm_unique_id()`` on one rank) as ``rank`` of ``world``."""
        self._check(self._L.sgemm_comm_init(self._h, comm_id, rank, world), "sgemm_comm_init")

    def comm_destroy(self):
        self._check(self._L.sgemm_comm_destroy(self._h), "sgemm_comm_destroy")

    def allgather_columns(self, d_full, m, n, ldd=0, tile_n=0, stream=0):
        """In-place all-gather of D's column shards (this rank's shard already lies at its place in ``d_full``)."""
        self._check(self._L.sgemm_allgather_columns(self._h, _ptr(d_full), m, n, ldd or max(m, 1), tile_n or self.info("tile_n"),
                                                    stream), "sgemm_allgather_columns")

    def bench(self, a, b, c, d, m, n, k, alpha=1.0, beta=0.0, warmup=5, runs=50, stream=0) -> float:
        """Mean milliseconds of ``runs`` back-to-back launches after ``warmup`` (CUDA events)."""
        ms = ctypes.c_float()
        lda, ldb, ldc, ldd = self._lds(m, n, k, 0, 0, 0, 0)
        self._check(self._L.sgemm_bench(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), alpha, beta, m, n, k,
                                        lda, ldb, ldc, ldd, warmup, runs, stream, ctypes.byref(ms)), "sgemm_bench")
        return ms.value

    def last_status(self):
        st = (_u32 * 8)()
        self._check(self._L.sgemm_last_status(self._h, ctypes.byref(st)), "sgemm_last_status")
        return list(st)

    def wait_selftest(self, timeout_ms: int = 20, tag: int = 0x7E57):
        """Launch the bounded-wait self-test kernel (see ``sgemm_wait_selftest``); read the outcome with ``last_status``."""
        self._check(self._L.sgemm_wait_selftest(self._h, timeout_ms, tag), "sgemm_wait_selftest")

    # ------------------------------------------------------------------------- options and facts
    def set_option(self, key: str, value: int):
        self._check(self._L.sgemm_set_option(self._h, key.encode(), value), "sgemm_set_option")

    def info(self, key: str) -> int:
        v = ctypes.c_int64()
        self._check(self._L.sgemm_get_info(self._h, key.encode(), ctypes.byref(v)), "sgemm_get_info")
        return v.value

    def workspace_bytes(self, m, n, k, lda=0, ldb=0, a=None, b=None) -> int:
        """Scratch bytes a launch of this problem needs; with `a` / `b` (device addresses) the need of these very
        operands, aligned copies of unaligned ones included."""
        out = ctypes.c_size_t()
        self._check(self._L.sgemm_workspace_bytes_for(self._h, _ptr(a), _ptr(b), m, n, k, lda or m, ldb or k,
                                                      ctypes.byref(out)), "sgemm_workspace_bytes_for")
        if a is None and b is None:
            plain = ctypes.c_size_t()
            self._check(self._L.sgemm_workspace_bytes(self._h, m, n, k, lda or m, ldb or k, ctypes.byref(plain)),
                        "sgemm_workspace_bytes")
            assert plain.value == out.value
        return out.value

    def set_workspace(self, dptr, nbytes: int):
        self._check(self._L.sgemm_set_workspace(self._h, _ptr(dptr), nbytes), "sgemm_set_workspace")

    # --------------------------------------------------------------------------------- utilities
    def fill_uniform(self, dptr, count: int, stream_id: int, first_index: int = 0, stream=0):
        self._check(self._L.sgemm_fill_uniform(self._h, _ptr(dptr), count, first_index, stream_id, stream),
                    "sgemm_fill_uniform")

    def narrow16(self, dsrc, ddst, count: int, stream=0):
        """FP32 -> the cubin's 16-bit operand type (FP16 / BF16), on the device."""
        self._check(self._L.sgemm_narrow16(self._h, _ptr(dsrc), _ptr(ddst), count, stream), "sgemm_narrow16")

    def tile_map(self, nx: int, ny: int):
        buf = (ctypes.c_int32 * (2 * nx * ny))()
        self._check(self._L.sgemm_tile_map(self._h, buf, nx, ny), "sgemm_tile_map")
        return [(buf[2 * i], buf[2 * i + 1]) for i in range(nx * ny)]

    def dev_alloc(self, nbytes: int) -> int:
        p = _vp()
        self._check(self._L.sgemm_dev_alloc(self._h, nbytes, ctypes.byref(p)), "sgemm_dev_alloc")
        return p.value or 0

    def dev_free(self, dptr: int):
        self._check(self._L.sgemm_dev_free(self._h, dptr), "sgemm_dev_free")

    def upload(self, dptr: int, host_array):
        self._check(self._L.sgemm_dev_upload(self._h, dptr, _ptr(host_array), host_array.nbytes), "sgemm_dev_upload")

    def download(self, host_array, dptr: int):
        self._check(self._L.sgemm_dev_download(self._h, _ptr(host_array), dptr, host_array.nbytes), "sgemm_dev_download")

    def memset(self, dptr: int, value: int, nbytes: int):
        self._check(self._L.sgemm_dev_memset(self._h, dptr, value, nbytes), "sgemm_dev_memset")

    def sync(self):
        self._check(self._L.sgemm_dev_sync(self._h), "sgemm_dev_sync")


def shard_columns(n: int, world: int, rank: int, tile_n: int = 1) -> Tuple[int, int]:
    """The library's column-shard rule (``sgemm_shard_columns``); ``runner.shard.shard_columns`` restates it in Python."""
    n0, n1 = _u32(), _u32()
    rc = lib().sgemm_shard_columns(n, world, rank, tile_n, ctypes.byref(n0), ctypes.byref(n1))
    if rc:
        raise SgemmError(rc, "sgemm_shard_columns", "bad shard request")
    return n0.value, n1.value


def comm_unique_id() -> bytes:
    """Id of a new communicator (128 bytes): one rank makes it, the host program hands it to all ranks."""
    buf = ctypes.create_string_buffer(128)
    rc = lib().sgemm_comm_unique_id(buf)
    if rc:
        raise SgemmError(rc, "sgemm_comm_unique_id", lib().sgemm_last_error(None).decode())
    return buf.raw


def comm_init_all(runners) -> None:
    """One process, several ``SgemmRunner`` on distinct GPUs: one communicator over them, runner i = rank i."""
    arr = (_vp * len(runners))(*[r._h for r in runners])
    rc = lib().sgemm_comm_init_all(arr, len(runners))
    if rc:
        raise SgemmError(rc, "sgemm_comm_init_all", lib().sgemm_last_error(runners[0]._h).decode())


def noalloc_scratch_bytes() -> int:
    return int(lib().sgemm_noalloc_scratch_bytes())


def device_count() -> int:
    return int(lib().sgemm_device_count())
