"""Kernel generator for the sm_100a SGEMM backend.

Drop-in for the reference's ``generator/generator.py`` on the generate -> compile leg of its
pipeline: same public names, same positional signatures, same TOML contract — but ``gemm()`` emits
CUDA C++ (hand-written tcgen05 / FFMA kernels specialised by ``#define``s) instead of GCN assembly and
``compile()`` runs ``nvcc -gencode arch=compute_100a,code=sm_100a -cubin`` instead of ROCm clang++.

Reference interface mirrored here (paths relative to the reference project):

* ``DataType``                 generator/generator.py:816-824
* ``GemmOptimizations``        generator/generator.py:827-854   (level, wgm, plr, gw, map_k_idx)
* ``GemmSolutionConfig``       generator/generator.py:857-1055  (tile = mfma * wave_group * wave_tiling,
                               shared-memory budget check raising ``RuntimeError``, ``to_dict``)
* ``FunctionArgument``         generator/generator.py:94-101    (the 15-argument kernel ABI)
* ``gemm``                     generator/generator.py:1056-2532 (returns the kernel source text)
* ``compile``                  generator/generator.py:2534-2569 (source -> code object + TOML, returns rc)
* CLI                          generator/generator.py:2571-2623

How the reference's knobs are read on sm_100a
---------------------------------------------
``mfma = (M, N, B, K)`` is the MMA atom.  ``(128, N, 1, 8)`` selects the tensor-core variant
(tcgen05 ``kind::tf32``, one CTA issues 128 x N x 8; with FP16 / BF16 operands the atom is
``(128, N, 1, 16)``, tcgen05 ``kind::f16``); ``(1, 1, 1, 1)`` selects the FFMA SIMT variant.
The GCN shapes ``(16,16,1,4)`` / ``(32,32,1,2)`` of the reference's tuner are still accepted: they have
no tensor-core counterpart for FP32 operands, so they map to the SIMT variant with the same block tile.
``wave_group`` is the cluster shape for the tensor variant and the thread grid of a block for SIMT;
``wave_tiling`` is atoms per CTA tile resp. the per-thread register tile.  ``tile_size`` keeps the
reference's product rule, so a runner that only knows the legacy keys still derives the right grid.
``depth_k`` is K per shared-memory stage, ``vmem_stage + 1`` the number of stages (the reference
allocates ``vmem_stage + 1`` LDS buffers the same way).  ``lds_usage_bytes`` is the shared memory one
CTA needs (dynamic for the tensor variant, static for SIMT) and is checked against the sm_100a limit.

Keyword-only additions of the tensor variant: ``a_major`` ("mn" / "k": read A where it lies or from a packed
K-major copy), ``terms`` (3 = 3xTF32, 1 = one MMA per k-slice), ``split`` ("prepass" / "inkernel": where the lo terms
are made), ``epilogue_warps`` (4 / 8), ``companion`` (emit the 128 x 128 companion kernel for low-intensity shapes)
and ``acc_chain`` (k accumulated inside the tensor core before the partial sum is added, in FP32, to a running sum in
registers; 0 = all of K in one chain).
"""
from __future__ import annotations

import argparse
import os
import re
import shutil
import subprocess
from enum import IntEnum
from io import StringIO
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import tomli_w

CSRC_DIR = Path(__file__).resolve().parent.parent / "csrc"

DEFAULT_NVCC_PATH = os.environ.get("SGEMM_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
SUPPORTED_ARCHS = ("sm_100a",)
MAX_LDS_NUM_BYTES = 232448          # 227 KiB: dynamic shared memory one sm_100a CTA can opt in to
MAX_STATIC_LDS_NUM_BYTES = 49152    # static shared memory limit (SIMT variant)
MAX_TMEM_COLUMNS = 512

VARIANT_TENSOR = "tcgen05_3xtf32"
VARIANT_SIMT = "simt_ffma"
KERNEL_ENTRY = "generated_gemm"     # the entry name the runner and the tuner hard-code
SIMT_FALLBACK_ENTRY = "generated_gemm_simt"
WHOLEK_ENTRY = "generated_gemm_wholek"   # twin of the main tcgen05 kernel that accumulates all of K in one chain
SKINNY_ENTRY = "generated_gemm_skinny"   # companion tcgen05 kernel for low-intensity shapes (tensor cubins)
THIN_ENTRY = "generated_gemm_thin"       # the companion with 32-column tiles, for N of a few columns

# The 15 arguments of the kernel ABI in order: (typename, name, bytes).
KERNEL_ABI = (
    ("global_buffer", "a", 8), ("global_buffer", "b", 8), ("global_buffer", "c", 8), ("global_buffer", "d", 8),
    ("by_value", "m", 4), ("by_value", "n", 4), ("by_value", "k", 4),
    ("by_value", "lda", 4), ("by_value", "ldb", 4), ("by_value", "ldc", 4), ("by_value", "ldd", 4),
    ("by_value", "alpha", 4), ("by_value", "beta", 4),
    ("by_value", "numWorkgroupX", 4), ("by_value", "numWorkgroupY", 4),
)


class FunctionArgument:
    def __init__(self, typename: str, name: str, offset: Optional[int], num_bytes: int):
        self.typename = typename
        self.name = name
        self.offset = offset
        self.num_bytes = num_bytes
        self.address_space = "global" if typename == "global_buffer" else None


FunctionArgumentList = List[FunctionArgument]


def default_arguments() -> FunctionArgumentList:
    return [FunctionArgument(t, n, None, s) for (t, n, s) in KERNEL_ABI]


class GpuContext:
    """Holder for the emitted source (the reference's context accumulates GCN instructions; there is
    no instruction DSL here, ``gemm`` writes the whole translation unit into ``content``)."""

    def __init__(self):
        self.content = StringIO()
        self.instructions: list = []

    def materialize(self) -> str:
        return self.content.getvalue()


def gpu_function(func):
    def wrapper(context, *args, **kwargs):
        if context is None:
            context = GpuContext()
        return func(context, *args, **kwargs)

    return wrapper


class DataType(IntEnum):
    """Element types.  The reference has FP32 only (generator/generator.py:816-824) and plumbs ``a_type`` ...
    ``scalar_type`` to its TOML as these integers; FP16 and BF16 are additions for the A and B operands of the
    tensor variant (C, D and the scalars stay FP32)."""
    FP32 = 0
    FP16 = 1
    BF16 = 2


def datatype_size(dtype: DataType) -> int:
    if dtype == DataType.FP32:
        return 4
    if dtype in (DataType.FP16, DataType.BF16):
        return 2
    raise RuntimeError(f"unrecognized type {dtype}")


class GemmOptimizations:
    """Optimisation knobs with the reference's names.

    level      0 = plain schedule (SIMT: fragments read just in time), >=1 = prefetching schedule
    wgm        tile rasterisation width (launch units are walked in groups of ``wgm`` tiles along M)
    plr        SIMT: shared-memory fragment prefetch depth (0/1); ignored by the tensor variant
    gw         epilogue strategy; both variants store straight from registers, accepted for parity
    map_k_idx  per-tile K-start stagger; it would change the summation order per tile and with it
               bit-reproducibility, so only 0 is implemented and other values are rejected by ``gemm``
    """

    def __init__(self, level: int, wgm: int | None = None, plr: int | None = None,
                 gw: int | None = None, map_k_idx: int | None = None):
        self.level = level
        self.wgm = 1
        self.plr = 0
        self.gw = 0
        self.map_k_idx = 0
        self._setup_optimizations()
        if wgm is not None:
            self.wgm = wgm
        if plr is not None:
            self.plr = plr
        if gw is not None:
            self.gw = gw
        if map_k_idx is not None:
            self.map_k_idx = map_k_idx

    def _setup_optimizations(self):
        if self.level != 0:
            self.plr = 1
            self.gw = 1


def _is_pow2(x: int) -> bool:
    return x > 0 and (x & (x - 1)) == 0


class GemmSolutionConfig:
    def __init__(self, a_type: DataType, b_type: DataType, cd_type: DataType, scalar_type: DataType,
                 mfma: Tuple[int, int, int, int], wave_group: Tuple[int, int], wave_tiling: Tuple[int, int],
                 depth_k: int, trans_a: bool, trans_b: bool, vmem_stage: int = 1, *,
                 a_major: str = "mn", terms: int = 3, split: str = "prepass",
                 epilogue_warps: Optional[int] = None, companion: bool = True, acc_chain: Optional[int] = None,
                 feed: str = "ldg"):
        self.a_type = a_type
        self.b_type = b_type
        self.cd_type = cd_type
        self.scalar_type = scalar_type
        self.wave_group = tuple(wave_group)
        self.trans_a = trans_a
        self.trans_b = trans_b
        self.mfma = tuple(mfma)
        self.wave_tiling = tuple(wave_tiling)
        self.depth_k = depth_k
        self.vmem_stage = vmem_stage
        self.wavefront_size = 32
        self.name = None
        self.a_major = a_major      # tensor variant: "mn" = TMA straight from column-major A, "k" = packed copy
        self.terms = terms          # tensor variant: 3 = 3xTF32 (FP32-accurate), 1 = plain TF32 (bring-up only)
        # tensor variant: warps that drain the accumulator; 8 (two per TMEM lane quarter, half the columns each)
        # keeps twice as many loads/stores in flight as 4 and is the default whenever tile N allows it
        self.epilogue_warps = epilogue_warps
        # tensor variant: also emit the companion kernel (128 x 128 x 32, one CTA per tile, lo terms made in the kernel)
        # that the runner uses for problems of low arithmetic intensity, where a pre-pass over the operands would
        # cost as much as the GEMM itself
        self.companion = companion
        # tensor variant: how many k a product is accumulated inside the tensor core before the partial sum is added,
        # in FP32 with round-to-nearest, to a running sum in the epilogue warps' registers.  The tensor core adds with
        # truncation, so an unbroken chain drifts toward zero in proportion to its length (for same-signed data the
        # error of a K = 8192 chain is 16 times the parity bound; a chain of 128 stays at a quarter of it for any K).
        # None: 128 when the running sum fits the register file, else 0; 0: all of K in one chain
        self.acc_chain = acc_chain
        self.split = split          # tensor variant: where lo = x - trunc_tf32(x) is made: "prepass" (a kernel writes
                                    # A_lo, B_lo to global memory once per call), "inkernel" (transform warps make the
                                    # lo tiles in shared memory from the TMA-landed raw tiles) or "hybrid" (A_lo by the
                                    # pre-pass, B's lo tile by the transform warps)

        # FFMA variant: how operand tiles reach shared memory.  "ldg": every thread loads 16-byte vectors into registers
        # and stores them (two buffers, any base and leading dimension); "tma": a producer warp issues TMA box copies
        # into a ring of vmem_stage + 1 stages and the other warps only multiply (operands TMA can describe; the
        # register-fed fallback kernel of the tensor-variant cubins is emitted beside it for the rest)
        self.feed = feed

        for t in (a_type, b_type, cd_type, scalar_type):
            datatype_size(t)
        if cd_type != DataType.FP32 or scalar_type != DataType.FP32:
            raise RuntimeError("C, D, alpha and beta are FP32")
        if a_type != b_type:
            raise RuntimeError("A and B have the same element type")
        self.elem_bytes = datatype_size(a_type)
        self.trans_a, self.trans_b = bool(trans_a), bool(trans_b)
        if not all(_is_pow2(g) for g in self.wave_group):
            raise RuntimeError(f"Invalid wave group: {wave_group}")
        if len(self.mfma) != 4 or len(self.wave_group) != 2 or len(self.wave_tiling) != 2:
            raise RuntimeError("mfma takes 4 ints, wave_group and wave_tiling 2 each")
        if min(self.mfma + self.wave_group + self.wave_tiling) < 1 or depth_k < 1 or vmem_stage < 1:
            raise RuntimeError("tiling parameters must be positive")

        m0 = self.mfma[0]
        if m0 == 128 and self.mfma[3] == (8 if self.elem_bytes == 4 else 16):
            self.variant = VARIANT_TENSOR
            self._check_tensor()
        elif self.mfma == (1, 1, 1, 1) or self.mfma in ((16, 16, 1, 4), (32, 32, 1, 2)):
            self.variant = VARIANT_SIMT
            self._check_simt()
        else:
            raise RuntimeError(f"unsupported MMA atom {self.mfma}: use (128, N, 1, 8) for tcgen05 tf32 (FP32 operands), "
                               f"(128, N, 1, 16) for tcgen05 f16/bf16, "
                               f"(1, 1, 1, 1) for FFMA, or a legacy (16,16,1,4)/(32,32,1,2) shape")

        if self.variant == VARIANT_TENSOR and self.feed != "ldg":
            raise RuntimeError("feed is a knob of the FFMA variant (the tensor variant is always fed by TMA)")
        limit = MAX_LDS_NUM_BYTES if (self.variant == VARIANT_TENSOR or self.feed == "tma") else MAX_STATIC_LDS_NUM_BYTES
        if self.lds_usage_bytes > limit:
            raise RuntimeError(f"LDS usage exceeds {limit}: {self.lds_usage_bytes}")

    # ------------------------------------------------------------------ variant-specific checks
    def _check_tensor(self):
        if self.elem_bytes == 2:
            # FP16 / BF16 operands: one kind::f16 MMA per 16 k (no split).  Every operand is read where it lies: stored
            # K-contiguous (A transposed, B untransposed) as a K-major tile, stored M- or N-contiguous as an MN-major
            # tile in chunks of 64 rows (128 bytes); a_major="k" instead reads an untransposed A through a packed
            # K-major copy made by a pre-pass (the first implementation, kept for comparison)
            if self.split != "prepass":
                raise RuntimeError("16-bit operands have no lo terms: split='inkernel' does not apply")
            if self.depth_k != 32 and self.depth_k % 64:
                raise RuntimeError(f"depth_k = {self.depth_k} must be 32 (one 64-byte span of 16-bit elements) or a "
                                   f"multiple of 64 (whole 128-byte spans)")
            self.terms = 1
            self.companion = False
        if self.wave_group not in ((1, 1), (2, 1)):
            raise RuntimeError(f"cluster shape {self.wave_group} is not implemented for the tensor variant "
                               f"(1x1: one CTA per tile, 2x1: a CTA pair on a 256-row tile)")
        if self.wave_tiling[0] != 1:
            raise RuntimeError("the tensor variant holds one 128-row atom per CTA (wave_tiling[0] must be 1)")
        bn = self.tile_size[1]
        if bn % 16 or bn < 32 or bn > 256:
            raise RuntimeError(f"tile N = {bn} must be a multiple of 16 in [32, 256] (UMMA N for M = 128)")
        if bn % 32:
            raise RuntimeError(f"tile N = {bn} must be a multiple of 32 (epilogue reads 32 TMEM columns at a time)")
        if self.wave_group[0] == 2 and bn % 64:
            raise RuntimeError(f"tile N = {bn} must be a multiple of 64 for a CTA pair (each CTA stages N/2 columns)")
        if self.elem_bytes == 4 and self.depth_k != 16 and self.depth_k % 32:
            raise RuntimeError(f"depth_k = {self.depth_k} must be 16 (one 64-byte swizzle span of FP32) or a "
                               f"multiple of 32 (whole 128-byte spans)")
        if 2 * bn > MAX_TMEM_COLUMNS:
            raise RuntimeError("two accumulator buffers exceed the 512 TMEM columns")
        if self.a_major not in ("mn", "k"):
            raise RuntimeError("a_major is 'mn' or 'k'")
        if self.terms not in (1, 3):
            raise RuntimeError("terms is 3 (3xTF32) or 1 (plain TF32)")
        if self.epilogue_warps is None:
            self.epilogue_warps = 8 if bn % 64 == 0 else 4
        if self.epilogue_warps not in (4, 8) or (self.epilogue_warps == 8 and bn % 64):
            raise RuntimeError("epilogue_warps is 4, or 8 when tile N is a multiple of 64")
        if self.split not in ("prepass", "inkernel", "hybrid"):
            raise RuntimeError("split is 'prepass', 'inkernel' or 'hybrid'")
        if self.trans_a and self.a_major == "k":
            raise RuntimeError("a transposed A is K-major already: a_major='k' (packed copy) does not apply")
        if self.trans_b and (bn // self.wave_group[0]) % (128 // self.elem_bytes):
            raise RuntimeError(f"a transposed B is staged in chunks of {128 // self.elem_bytes} columns (128 bytes): tile N per "
                               f"CTA must be a multiple of that")
        if self.split != "prepass" and self.a_major == "k":
            raise RuntimeError("the K-major packed copy of A is made by a pre-pass that also writes both lo copies; it "
                               "excludes split='inkernel' and 'hybrid'")
        # the running sum of chunked accumulation: tile N / (epilogue warps per lane quarter) registers per epilogue
        # thread, next to about 72 others, for every thread of the block (one register allocation per kernel)
        threads = 128 + 32 * self.epilogue_warps + (128 if self.split != "prepass" else 0)
        sum_regs = bn // (self.epilogue_warps // 4)
        # registers an epilogue thread can have: an even share of its scheduler partition's 512 per lane, or, with
        # 8 epilogue warps, what is left when the other warp groups shrink to 56 (the kernel's register hand-over)
        per_partition = threads // 128
        epi_regs = (512 - (per_partition - 2) * 56) // 2 if self.epilogue_warps == 8 else min(255, 512 // per_partition)
        fits = sum_regs + 72 <= min(epi_regs // 8 * 8, 232)
        self._acc_chain_requested = self.acc_chain
        if self.acc_chain is None:
            # 3xTF32 adds to the accumulator three times per 8 k, 16-bit operands once per 16 k: a sixth of the
            # truncating adds per k, so their chain can be that much longer for the same drift
            self.acc_chain = (max(128, self.depth_k) if self.elem_bytes == 4 else 1024) if fits else 0
        if self.acc_chain < 0 or self.acc_chain % self.depth_k:
            raise RuntimeError(f"acc_chain = {self.acc_chain} must be 0 or a multiple of depth_k = {self.depth_k}")
        if self.acc_chain and not fits:
            raise RuntimeError(f"acc_chain: a running sum of {sum_regs} registers per thread does not "
                               f"fit a block of {threads} threads")
        if self.stages * 24 + 40 > 256:
            raise RuntimeError(f"{self.stages} stages exceed the barrier block of the kernel")
        if self.stages < 2:
            raise RuntimeError("the TMA ring needs at least 2 stages")

    def _check_simt(self):
        if self.elem_bytes != 4:
            raise RuntimeError("the FFMA variant computes on FP32 operands only")
        bm, bn = self.tile_size
        tm, tn = self.simt_thread_tile
        if bm % tm or bn % tn:
            raise RuntimeError(f"block tile {bm}x{bn} is not a multiple of the thread tile {tm}x{tn}")
        threads = (bm // tm) * (bn // tn)
        if threads < 1 or threads > 1024:
            raise RuntimeError(f"a block of {threads} threads is not launchable")
        if self.depth_k % 4:
            raise RuntimeError("depth_k must be a multiple of 4 (16-byte loads along K)")
        if tm * tn > 128:
            raise RuntimeError(f"thread tile {tm}x{tn} does not fit the register file")
        if self.feed not in ("ldg", "tma"):
            raise RuntimeError("feed is 'ldg' or 'tma'")
        if self.feed == "tma":
            if self.trans_a:
                raise RuntimeError("the TMA-fed FFMA kernel reads an untransposed A (a K-contiguous A tile would be read "
                                   "with shared-memory bank conflicts): use feed='ldg'")
            if threads % 128 or threads > 512:
                raise RuntimeError(f"{threads} multiplying threads: registers are handed over in groups of four warps "
                                   f"(128, 256, 384 or 512 threads)")
            if max(bm, bn, self.depth_k) > 256:
                raise RuntimeError("a TMA box has at most 256 elements per dimension")
            if not self.trans_b and (bn % 32 or (self.depth_k // 4) & (self.depth_k // 4 - 1)):
                raise RuntimeError("an untransposed B is transposed in shared memory 32 columns and a power-of-two number "
                                   "of k-quads at a time: tile N must be a multiple of 32, depth_k / 4 a power of two")
            if self.stages < 2 or self.stages > 12:
                raise RuntimeError(f"{self.stages} stages: the TMA ring has 2 to 12")

    # ------------------------------------------------------------------------------- geometry
    @property
    def tile_size(self) -> Tuple[int, int]:
        return (self.mfma[0] * self.wave_group[0] * self.wave_tiling[0],
                self.mfma[1] * self.wave_group[1] * self.wave_tiling[1])

    @property
    def stages(self) -> int:
        return self.vmem_stage + 1

    @property
    def simt_thread_tile(self) -> Tuple[int, int]:
        """Per-thread register tile of the SIMT variant (multiples of 4 in both directions)."""
        if self.mfma == (1, 1, 1, 1):
            return self.wave_tiling
        bm, bn = self.tile_size  # legacy MFMA shape: largest square thread tile that leaves >= 64 threads
        for t in (8, 4):
            if bm % t == 0 and bn % t == 0 and (bm // t) * (bn // t) >= 64:
                return t, t
        return 4, 4

    @property
    def num_workitems(self) -> int:
        if self.variant == VARIANT_TENSOR:
            # first group of four warps (TMA, MMA, two spare) + epilogue warps (+ four transform warps for the in-kernel split)
            return 128 + 32 * self.epilogue_warps + (128 if self.split != "prepass" else 0)
        bm, bn = self.tile_size
        tm, tn = self.simt_thread_tile
        return (bm // tm) * (bn // tn) + (128 if self.feed == "tma" else 0)   # + the producer's group of four warps

    @property
    def num_bytes_per_buffer_load(self) -> Tuple[int, int]:
        """Bytes one global->shared transfer moves per operand: a 16-byte vector per thread for SIMT (the
        reference's tuner keeps only configurations where this is (16, 16)), a whole TMA box for tcgen05."""
        if self.variant == VARIANT_TENSOR:
            return 32 * self.depth_k * 4, min(self.depth_k, 32) * (self.tile_size[1] // self.wave_group[0]) * 4
        return 16, 16

    @property
    def tmem_columns(self) -> int:
        if self.variant != VARIANT_TENSOR:
            return 0
        need, cols = 2 * self.tile_size[1], 32
        while cols < need:
            cols *= 2
        return cols

    def _ring_bytes(self) -> int:
        bn_cta = self.tile_size[1] // self.wave_group[0]                         # a CTA pair splits B's columns
        tiles = 2 if self.terms == 3 else 1                                      # A_hi, A_lo, B_hi, B_lo or A, B
        stage = tiles * (128 + bn_cta) * self.depth_k * self.elem_bytes
        return self.stages * stage + 1024 + 256                                  # + alignment slack + barriers

    @property
    def lds_usage_bytes(self) -> int:
        bm, bn = self.tile_size
        if self.variant == VARIANT_TENSOR:
            return self._ring_bytes()
        if self.feed == "tma":
            # A tile, B tile and, for an untransposed B, the raw buffer TMA fills before the tile is transposed
            raw = 0 if self.trans_b else bn
            return self.stages * self.depth_k * (bm + bn + raw) * 4 + 128 + 512   # ring + alignment slack + barriers
        return 2 * self.depth_k * (bm + 4 + bn + 4) * 4                          # double-buffered, padded A and B

    @property
    def num_unrolled_iters(self) -> int:
        return self.depth_k // max(self.mfma[3], 1)

    def companion_config(self) -> Optional["GemmSolutionConfig"]:
        """Configuration of the companion kernel emitted next to a tensor-variant kernel (None: no companion)."""
        if self.variant != VARIANT_TENSOR or not self.companion or self.terms != 3:
            return None   # (the companion makes lo tiles in the kernel: it belongs to the 3xTF32 scheme)
        return GemmSolutionConfig(self.a_type, self.b_type, self.cd_type, self.scalar_type, (128, 128, 1, 8), (1, 1), (1, 1),
                                  32, self.trans_a, self.trans_b, vmem_stage=2, split="inkernel", terms=self.terms,
                                  companion=False, acc_chain=0 if self._acc_chain_requested == 0 else None)

    def thin_config(self) -> Optional["GemmSolutionConfig"]:
        """The companion kernel's narrow sibling (128 x 32 x 32, 5 stages, lo terms made in the kernel): with N of a
        few columns the 128-column companion would spend its tensor-pipe time on padding."""
        if self.companion_config() is None:
            return None
        return GemmSolutionConfig(self.a_type, self.b_type, self.cd_type, self.scalar_type, (128, 32, 1, 8), (1, 1), (1, 1),
                                  32, self.trans_a, self.trans_b, vmem_stage=4, split="inkernel", terms=self.terms,
                                  companion=False, acc_chain=0 if self._acc_chain_requested == 0 else None)

    def to_dict(self) -> Dict:
        d = {
            # ---- the reference's 14 keys (generator/generator.py:1001-1017), same order and types ----
            "a_type": int(self.a_type),
            "b_type": int(self.b_type),
            "cd_type": int(self.cd_type),
            "scalar_type": int(self.scalar_type),
            "wave_group": list(self.wave_group),
            "trans_a": self.trans_a,
            "trans_b": self.trans_b,
            "mfma": list(self.mfma),
            "wave_tiling": list(self.wave_tiling),
            "depth_k": self.depth_k,
            "vmem_stage": self.vmem_stage,
            "wavefront_size": self.wavefront_size,
            "lds_usage_bytes": self.lds_usage_bytes,
            "name": self.name if self.name else "",
            # ---- sm_100a additions read by the CUDA runner ----
            "variant": self.variant,
            "block_tile": [self.tile_size[0], self.tile_size[1], self.depth_k],
            "cluster": list(self.wave_group) if self.variant == VARIANT_TENSOR else [1, 1],
            "stages": self.stages,
            "num_threads": self.num_workitems,
            "dynamic_smem_bytes": self.lds_usage_bytes if (self.variant == VARIANT_TENSOR or self.feed == "tma") else 0,
            "tmem_columns": self.tmem_columns,
            "entry": KERNEL_ENTRY,
            # optimisation knobs of the reference that are accepted for compatibility and change nothing in these
            # kernels (so that a tuner log does not suggest they were searched): the epilogue register strategy and the
            # schedule level only set defaults, the K-start stagger is refused because it changes the summation order
            "knobs_without_effect": "gw level map_k_idx",
        }
        if self.variant == VARIANT_TENSOR:
            fb = simt_fallback_config(self.trans_a, self.trans_b)
            d.update({
                "a_major": self.a_major,
                "terms": self.terms,
                "split": self.split,
                "epilogue_warps": self.epilogue_warps,
                "acc_chain": self.acc_chain,
                "wholek_entry": WHOLEK_ENTRY if self.acc_chain else "",
                "fallback_entry": SIMT_FALLBACK_ENTRY,
                "fallback_tile": [fb.tile_size[0], fb.tile_size[1], fb.depth_k],
                "fallback_threads": fb.num_workitems,
            })
            sk = self.companion_config()
            if sk is not None:
                d.update({
                    "skinny_entry": SKINNY_ENTRY,
                    "skinny_tile": [sk.tile_size[0], sk.tile_size[1], sk.depth_k],
                    "skinny_threads": sk.num_workitems,
                    "skinny_smem_bytes": sk.lds_usage_bytes,
                    "skinny_acc_chain": sk.acc_chain,
                })
            th = self.thin_config()
            if th is not None:
                d.update({
                    "thin_entry": THIN_ENTRY,
                    "thin_tile": [th.tile_size[0], th.tile_size[1], th.depth_k],
                    "thin_threads": th.num_workitems,
                    "thin_smem_bytes": th.lds_usage_bytes,
                    "thin_acc_chain": th.acc_chain,
                })
        elif self.feed == "tma":
            # the register-fed kernel for operands TMA cannot describe
            fb = simt_fallback_config(self.trans_a, self.trans_b)
            d.update({
                "feed": "tma",
                "fallback_entry": SIMT_FALLBACK_ENTRY,
                "fallback_tile": [fb.tile_size[0], fb.tile_size[1], fb.depth_k],
                "fallback_threads": fb.num_workitems,
            })
        return d


def simt_fallback_config(trans_a: bool = False, trans_b: bool = False) -> GemmSolutionConfig:
    """The FFMA kernel compiled into every tensor-variant cubin for shapes TMA cannot describe
    (leading dimensions that are not multiples of 4, unaligned bases) and for tiny problems."""
    return GemmSolutionConfig(DataType.FP32, DataType.FP32, DataType.FP32, DataType.FP32,
                              (1, 1, 1, 1), (16, 16), (8, 8), 16, trans_a, trans_b)


# --------------------------------------------------------------------------------------------------
# source emission
# --------------------------------------------------------------------------------------------------
def _read(name: str) -> str:
    return (CSRC_DIR / name).read_text()


def _defines(pairs) -> str:
    return "".join(f"#define {k} {v}\n" for k, v in pairs)


def _check_arguments(arguments: FunctionArgumentList):
    got = [(a.typename, a.name, a.num_bytes) for a in arguments]
    if got != list(KERNEL_ABI):
        raise RuntimeError("kernel arguments must be the 15-entry SGEMM ABI "
                           "(a, b, c, d, m, n, k, lda, ldb, ldc, ldd, alpha, beta, numWorkgroupX, numWorkgroupY)")
    offset = 0
    for a in arguments:  # natural alignment, as the reference's kernarg segment (generator.py:127-147)
        offset = (offset + a.num_bytes - 1) // a.num_bytes * a.num_bytes
        a.offset = offset
        offset += a.num_bytes


def _simt_defines(cfg: GemmSolutionConfig, opt: GemmOptimizations, entry: str):
    bm, bn = cfg.tile_size
    tm, tn = cfg.simt_thread_tile
    return [("SIMT_ENTRY", entry), ("SIMT_BM", bm), ("SIMT_BN", bn), ("SIMT_BK", cfg.depth_k),
            ("SIMT_TM", tm), ("SIMT_TN", tn), ("SIMT_PLR", 1 if opt.plr else 0)]


def _tensor_defines(config: GemmSolutionConfig):
    return [("TC_BN", config.tile_size[1]), ("TC_BK", config.depth_k), ("TC_STAGES", config.stages),
            ("TC_CTA_GROUP", config.wave_group[0]), ("TC_SPLIT_INKERNEL", 1 if config.split != "prepass" else 0),
            ("TC_SPLIT_HYBRID", 1 if config.split == "hybrid" else 0),
            ("TC_EPI_WARPS", config.epilogue_warps),
            ("TC_A_KMAJOR", 1 if (config.a_major == "k" or config.trans_a) else 0),
            ("TC_B_MNMAJOR", 1 if config.trans_b else 0), ("TC_TERMS", config.terms),
            ("TC_ELEM_BYTES", config.elem_bytes),
            ("TC_AB_FORMAT", {DataType.FP32: "2u", DataType.FP16: "0u", DataType.BF16: "1u"}[config.a_type]),
            ("TC_ACC_CHUNK", config.acc_chain // config.depth_k)]


def _trans_defines(cfg: GemmSolutionConfig):
    return [("GEMM_TRANS_A", 1 if cfg.trans_a else 0), ("GEMM_TRANS_B", 1 if cfg.trans_b else 0)]


@gpu_function
def gemm(context: GpuContext, name: str, arch: str, config: GemmSolutionConfig, opt: GemmOptimizations,
         arguments: FunctionArgumentList) -> str:
    """Emit the CUDA translation unit for ``config``/``opt``; returns the source text.

    ``name`` is recorded in the header only: the ``__global__`` entry is always ``generated_gemm``
    because the runner and the tuner look it up under that name (runner/generator_runner.cpp:197,
    tuner/sgemm_tuner.py:67).  Infeasible knob combinations raise ``RuntimeError`` — the tuner's skip
    mechanism (tuner/sgemm_tuner.py:92)."""
    _check_arguments(arguments)
    if not _is_pow2(opt.wgm):
        raise RuntimeError(f"wgm must be a power of two, got {opt.wgm}")
    if opt.map_k_idx:
        raise RuntimeError("map_k_idx != 0 (per-tile K stagger) is not offered: it changes the summation "
                           "order per tile and would break run-to-run and tile-to-tile reproducibility")
    if arch is not None and arch not in SUPPORTED_ARCHS:
        raise RuntimeError(f"unsupported arch {arch!r}; this generator targets {SUPPORTED_ARCHS}")

    out = StringIO()
    out.write(f"// generated by generator.py: kernel '{name}', variant {config.variant}, "
              f"tile {config.tile_size[0]}x{config.tile_size[1]}x{config.depth_k}, stages {config.stages}, "
              f"wgm {opt.wgm}, plr {opt.plr}, gw {opt.gw}\n")
    out.write(_defines([("OPT_WGM", opt.wgm)] + _trans_defines(config)))
    out.write(_read("sgemm_common.cuh"))
    if config.variant == VARIANT_SIMT and config.feed == "tma":
        # the register-fed kernel under the fallback name (as in a tensor-variant cubin), the TMA-fed one as the entry
        out.write(_defines(_simt_defines(simt_fallback_config(config.trans_a, config.trans_b), opt, SIMT_FALLBACK_ENTRY)))
        out.write(_read("sgemm_simt.cuh"))
        bm, bn = config.tile_size
        tm, tn = config.simt_thread_tile
        out.write(_defines([("FT_ENTRY", KERNEL_ENTRY), ("FT_BM", bm), ("FT_BN", bn), ("FT_BK", config.depth_k),
                            ("FT_TM", tm), ("FT_TN", tn), ("FT_STAGES", config.stages)]))
        out.write(_read("sgemm_ffma_tma.cuh"))
    elif config.variant == VARIANT_SIMT:
        out.write(_defines(_simt_defines(config, opt, KERNEL_ENTRY)))
        out.write(_read("sgemm_simt.cuh"))
    else:
        out.write(_defines(_simt_defines(simt_fallback_config(config.trans_a, config.trans_b), opt, SIMT_FALLBACK_ENTRY)))
        out.write(_read("sgemm_simt.cuh"))
        template = _read("sgemm_tcgen05.cuh")
        out.write(_defines(_tensor_defines(config)))
        out.write(template)
        if config.acc_chain:
            # twin of the main kernel without the running sum (all of K in one tensor-core chain, accumulator written
            # out straight from TMEM): what the runner launches when a tile has a single accumulation chunk anyway
            # (K up to two chains) or the caller turns chunking off
            body = template.split("// ==== end of the per-kernel section")[0]
            body = re.sub(r"\bTC_", "TCW_", body)
            body = re.sub(r"\btc_", "tcw_", body)
            body = re.sub(r"\bTc(?=[A-Z])", "Tcw", body)
            body = re.sub(r"\b%s\b" % KERNEL_ENTRY, WHOLEK_ENTRY, body)
            out.write("\n// ---- twin of the main kernel: whole-K accumulation, epilogue straight from TMEM ----\n")
            out.write(_defines([(k.replace("TC_", "TCW_", 1), 0 if k == "TC_ACC_CHUNK" else v) for k, v in _tensor_defines(config)]))
            out.write(body)
        companion = config.companion_config()
        if companion is not None:
            # second instance of the per-kernel part of the template under its own names: macros TC_* -> TCS_*,
            # functions tc_* -> tcs_*, types Tc* -> Tcs*, entry generated_gemm -> generated_gemm_skinny
            body = template.split("// ==== end of the per-kernel section")[0]
            body = re.sub(r"\bTC_", "TCS_", body)
            body = re.sub(r"\btc_", "tcs_", body)
            body = re.sub(r"\bTc(?=[A-Z])", "Tcs", body)
            body = re.sub(r"\b%s\b" % KERNEL_ENTRY, SKINNY_ENTRY, body)
            out.write("\n// ---- companion kernel for low-intensity shapes: 128 x 128 x 32, one CTA per tile, in-kernel split ----\n")
            out.write(_defines([(k.replace("TC_", "TCS_", 1), v) for k, v in _tensor_defines(companion)]))
            out.write(body)
            thin = config.thin_config()
            body = template.split("// ==== end of the per-kernel section")[0]
            body = re.sub(r"\bTC_", "TCT_", body)
            body = re.sub(r"\btc_", "tct_", body)
            body = re.sub(r"\bTc(?=[A-Z])", "Tct", body)
            body = re.sub(r"\b%s\b" % KERNEL_ENTRY, THIN_ENTRY, body)
            out.write("\n// ---- the companion's narrow sibling: 128 x 32 x 32, 5 stages, in-kernel split, for N of a few columns ----\n")
            out.write(_defines([(k.replace("TC_", "TCT_", 1), v) for k, v in _tensor_defines(thin)]))
            out.write(body)
    src = out.getvalue()
    context.content.write(src)
    return src


def nvcc_command(src: str, out: str, extra: Optional[List[str]] = None) -> List[str]:
    return [DEFAULT_NVCC_PATH, "-gencode", "arch=compute_100a,code=sm_100a", "-cubin", "-O3", "-std=c++17",
            "-lineinfo", "-ccbin", os.environ.get("SGEMM_HOST_CXX", "g++"), *(extra or []), "-o", out, src]


def compile(kern_name: str, kern_str: str, arch: str, output_folder: str, gemm_config: GemmSolutionConfig) -> int:
    """Write ``<kern_name>.cu``, compile it to ``<kern_name>.cubin`` and write ``<kern_name>.toml``.
    Returns nvcc's return code (0 = success).

    The three files appear together or not at all: everything is built in a scratch directory inside
    ``output_folder`` and moved into place (``os.replace``, atomic within a file system) only after nvcc has
    succeeded — cubin and TOML first, the source last.  A failed or interrupted build therefore leaves the previous
    kernel intact AND leaves its old source beside it, so that a freshness check that compares the emitted source with
    the ``.cu`` on disk (``kernels.ensure``) keeps reporting the kernel as stale, and no reader ever opens a
    half-written cubin.  (The reference writes ``.s`` first and ignores the assembler's return code,
    generator/generator.py:2535-2555.)"""
    import shutil
    import tempfile

    os.makedirs(output_folder, exist_ok=True)
    scratch = tempfile.mkdtemp(prefix=".build-", dir=output_folder)
    try:
        src = f"{scratch}/{kern_name}.cu"
        with open(src, "w") as f:
            f.write(kern_str)
        ret = subprocess.run(nvcc_command(src, f"{scratch}/{kern_name}.cubin"),
                             stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if ret.returncode:
            print(ret.stdout)
            return ret.returncode
        with open(f"{scratch}/{kern_name}.toml", "wb") as f:
            tomli_w.dump(gemm_config.to_dict(), f)
        for suffix in ("cubin", "toml", "cu"):
            os.replace(f"{scratch}/{kern_name}.{suffix}", f"{output_folder}/{kern_name}.{suffix}")
        return 0
    finally:
        shutil.rmtree(scratch, ignore_errors=True)


def tensor_config(bn: int = 256, bk: int = 32, stages: int = 2, cluster: int = 1, trans_a: bool = False,
                  trans_b: bool = False, ab_type: DataType = DataType.FP32, **kw) -> GemmSolutionConfig:
    """Shorthand for a tensor-variant configuration with tile (128 * cluster) x bn x bk; ``ab_type`` is the element
    type of A and B (FP32: 3xTF32 with atom K = 8; FP16 / BF16: one MMA per 16 k)."""
    atom_k = 8 if ab_type == DataType.FP32 else 16
    return GemmSolutionConfig(ab_type, ab_type, DataType.FP32, DataType.FP32,
                              (128, bn, 1, atom_k), (cluster, 1), (1, 1), bk, trans_a, trans_b, vmem_stage=stages - 1, **kw)


def simt_config(bm: int = 128, bn: int = 128, bk: int = 16, tm: int = 8, tn: int = 8, trans_a: bool = False,
                trans_b: bool = False, feed: str = "ldg", stages: int = 2) -> GemmSolutionConfig:
    """Shorthand for an FFMA configuration: block tile bm x bn x bk, thread tile tm x tn; ``feed="tma"`` selects the
    TMA-fed, warp-specialised kernel with a ring of ``stages`` stages."""
    return GemmSolutionConfig(DataType.FP32, DataType.FP32, DataType.FP32, DataType.FP32,
                              (1, 1, 1, 1), (bm // tm, bn // tn), (tm, tn), bk, trans_a, trans_b,
                              vmem_stage=stages - 1, feed=feed)


def build_kernel(output_folder: str, config: GemmSolutionConfig, opt: Optional[GemmOptimizations] = None,
                 kern_name: str = KERNEL_ENTRY, arch: str = "sm_100a") -> Tuple[str, str]:
    """generate + compile in one call; returns (cubin path, toml path) or raises RuntimeError."""
    opt = opt or GemmOptimizations(1, wgm=8)
    src = gemm(None, kern_name, arch, config, opt, default_arguments())
    if compile(kern_name, src, arch, output_folder, config):
        raise RuntimeError(f"nvcc failed for {kern_name} in {output_folder}")
    return f"{output_folder}/{kern_name}.cubin", f"{output_folder}/{kern_name}.toml"


def tile_raster(z: int, nx: int, ny: int, wgm: int) -> Tuple[int, int]:
    """Host model of the kernels' launch-unit -> tile mapping (``sgemm_tile_raster`` in csrc/sgemm_common.cuh).
    For ``nx`` a multiple of ``wgm`` this is the reference's workgroup remap (generator/generator.py:1437-1464,
    checked by test/test_vm.py:735-740): x' = (z % wgm) + (z // wgm // ny) * wgm, y' = (z // wgm) % ny."""
    if wgm <= 1:
        return z % nx, z // nx
    group = z // (wgm * ny)
    first_x = group * wgm
    width = min(wgm, nx - first_x)
    r = z - group * wgm * ny
    return first_x + r % width, r // width


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument(dest="output_folder", action="store", type=str, help="Output folder")
    ap.add_argument("--arch", dest="arch", action="store", choices=list(SUPPORTED_ARCHS), default="sm_100a")
    ap.add_argument("--variant", choices=["tensor", "simt"], default="tensor")
    args = ap.parse_args()
    gemm_config = tensor_config() if args.variant == "tensor" else simt_config()
    opt = GemmOptimizations(1, wgm=8)
    src_str = gemm(None, KERNEL_ENTRY, args.arch, gemm_config, opt, default_arguments())
    raise SystemExit(compile(KERNEL_ENTRY, src_str, args.arch, args.output_folder, gemm_config))

