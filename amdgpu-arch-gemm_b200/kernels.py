"""Named kernel configurations that are generated and compiled ahead of time (by ``build_all``) so that the
tests, the smoke check and the benchmark find ready cubins; ``ensure`` compiles one on demand."""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Tuple

from generator.generator import (KERNEL_ENTRY, GemmOptimizations, GemmSolutionConfig, DataType, build_kernel,
                                 default_arguments, gemm, simt_config, tensor_config)

GENERATED_DIR = Path(__file__).resolve().parent / "_generated"
F = DataType.FP32


def _legacy(mfma, wg, wt, dk):
    return GemmSolutionConfig(F, F, F, F, mfma, wg, wt, dk, False, False)


# name -> (config factory, optimisation knobs)
REGISTRY = {
    # tensor-core 3xTF32 kernels: tile 128 x BN x BK, S stages
    "tc_128x256x32_s2": (lambda: tensor_config(256, 32, 2), dict(wgm=8)),
    "tc_128x128x32_s3": (lambda: tensor_config(128, 32, 3), dict(wgm=8)),
    "tc_128x64x32_s4": (lambda: tensor_config(64, 32, 4), dict(wgm=8)),
    "tc2_256x256x32_s3_e4": (lambda: tensor_config(256, 32, 3, cluster=2, epilogue_warps=4), dict(wgm=8)),
    "tc_128x64x64_s2": (lambda: tensor_config(64, 64, 2), dict(wgm=4)),
    "tc_128x256x16_s4": (lambda: tensor_config(256, 16, 4), dict(wgm=8)),
    "tc_128x128x16_s7": (lambda: tensor_config(128, 16, 7), dict(wgm=8)),
    # CTA pairs (cluster 2x1, tcgen05 cta_group::2): tile 256 x BN x BK
    "tc2_256x256x32_s3": (lambda: tensor_config(256, 32, 3, cluster=2), dict(wgm=8)),
    "tc2_256x256x16_s6": (lambda: tensor_config(256, 16, 6, cluster=2), dict(wgm=4)),
    "tc2_256x128x32_s4": (lambda: tensor_config(128, 32, 4, cluster=2), dict(wgm=4)),
    # lo tiles made inside the kernel by transform warps (no pre-pass, no lo copies in global memory)
    "tc2i_256x256x32_s3": (lambda: tensor_config(256, 32, 3, cluster=2, split="inkernel"), dict(wgm=8)),
    "tc2h_256x256x32_s3": (lambda: tensor_config(256, 32, 3, cluster=2, split="hybrid"), dict(wgm=8)),   # A_lo by the pre-pass, B's lo tile in the kernel
    "tc2i_256x256x16_s6": (lambda: tensor_config(256, 16, 6, cluster=2, split="inkernel"), dict(wgm=8)),
    "tci_128x256x32_s2": (lambda: tensor_config(256, 32, 2, split="inkernel"), dict(wgm=8)),
    "tci_128x128x32_s3": (lambda: tensor_config(128, 32, 3, split="inkernel"), dict(wgm=8)),
    # the same tile reading A from K-major packed copies, and a plain-TF32 build (bring-up aids)
    "tc_128x128x32_s3_ak": (lambda: tensor_config(128, 32, 3, a_major="k"), dict(wgm=8)),
    "tc_128x128x16_s6_ak": (lambda: tensor_config(128, 16, 6, a_major="k"), dict(wgm=8)),
    # whole-K accumulation inside the tensor core (no chunking): the kernels the recorded device arithmetic is pinned with
    "tc_128x128x32_s3_1x": (lambda: tensor_config(128, 32, 3, terms=1, acc_chain=0), dict(wgm=8)),
    # one MMA per k-slice on the raw FP32 words (plain TF32, a third of the tensor work, NOT FP32-accurate): the bench
    # uses it as a probe of the TF32 tensor rate this pipeline reaches on the box at hand
    "tc2_256x256x32_s6_1x": (lambda: tensor_config(256, 32, 6, cluster=2, terms=1, acc_chain=0), dict(wgm=8)),
    "tc2_256x256x32_s3_c0": (lambda: tensor_config(256, 32, 3, cluster=2, acc_chain=0), dict(wgm=8)),
    # transposed operands (TN: A stored K x M, NT: B stored N x K, TT: both)
    "tc2_256x256x32_s3_tn": (lambda: tensor_config(256, 32, 3, cluster=2, trans_a=True), dict(wgm=8)),
    "tc2_256x256x32_s3_nt": (lambda: tensor_config(256, 32, 3, cluster=2, trans_b=True), dict(wgm=8)),
    "tc2_256x256x32_s3_tt": (lambda: tensor_config(256, 32, 3, cluster=2, trans_a=True, trans_b=True), dict(wgm=8)),
    "tc_128x128x32_s3_tt": (lambda: tensor_config(128, 32, 3, trans_a=True, trans_b=True), dict(wgm=8)),
    "tc2i_256x256x32_s3_tt": (lambda: tensor_config(256, 32, 3, cluster=2, split="inkernel", trans_a=True, trans_b=True), dict(wgm=8)),
    "simt_128x128x16_tn": (lambda: simt_config(128, 128, 16, 8, 8, trans_a=True), dict(wgm=8)),
    "simt_128x128x16_nt": (lambda: simt_config(128, 128, 16, 8, 8, trans_b=True), dict(wgm=8)),
    "simt_64x64x16_tt": (lambda: simt_config(64, 64, 16, 4, 4, trans_a=True, trans_b=True), dict(wgm=4)),
    # FFMA SIMT kernels
    # FP16 / BF16 operands (FP32 accumulate, C and D FP32), every operand read where it lies in all four layouts;
    # "_ak": an untransposed A through a packed K-major copy instead (the first implementation, kept for comparison)
    "bf16_tc2_256x256x64_s6": (lambda: tensor_config(256, 64, 6, cluster=2, ab_type=DataType.BF16), dict(wgm=8)),
    "bf16_tc2_256x256x128_s3": (lambda: tensor_config(256, 128, 3, cluster=2, ab_type=DataType.BF16), dict(wgm=16)),   # the tuner's best at 8192^3
    "fp16_tc2_256x256x128_s3": (lambda: tensor_config(256, 128, 3, cluster=2, ab_type=DataType.FP16), dict(wgm=16)),
    "bf16_tc2_256x256x64_s6_ak": (lambda: tensor_config(256, 64, 6, cluster=2, ab_type=DataType.BF16, a_major="k"), dict(wgm=8)),
    "fp16_tc_128x128x64_s4": (lambda: tensor_config(128, 64, 4, ab_type=DataType.FP16), dict(wgm=8)),
    "bf16_tc_128x256x32_s4_tn": (lambda: tensor_config(256, 32, 4, trans_a=True, ab_type=DataType.BF16), dict(wgm=8)),
    "fp16_tc2_256x128x64_s4_tn": (lambda: tensor_config(128, 64, 4, cluster=2, trans_a=True, ab_type=DataType.FP16), dict(wgm=8)),
    "bf16_tc2_256x256x64_s6_tt": (lambda: tensor_config(256, 64, 6, cluster=2, trans_a=True, trans_b=True, ab_type=DataType.BF16), dict(wgm=8)),
    "fp16_tc_128x128x64_s4_nt": (lambda: tensor_config(128, 64, 4, trans_b=True, ab_type=DataType.FP16), dict(wgm=8)),
    "simt_128x128x16": (lambda: simt_config(128, 128, 16, 8, 8), dict(wgm=8)),
    "simt_128x128x16_t16x8": (lambda: simt_config(128, 128, 16, 16, 8), dict(wgm=8)),   # best of the FFMA sweep at 4096^3
    "simt_64x64x16": (lambda: simt_config(64, 64, 16, 4, 4), dict(wgm=4)),
    # FFMA kernels fed by TMA (a producer thread, mbarrier ring, consumers that only multiply)
    "ffma_tma_256x128x32_s3": (lambda: simt_config(256, 128, 32, 16, 8, feed="tma", stages=3), dict(wgm=8)),   # best of the staged FFMA search at 8192^3
    "ffma_tma_256x128x16_s4": (lambda: simt_config(256, 128, 16, 16, 8, feed="tma", stages=4), dict(wgm=8)),
    "ffma_tma_128x256x16_s4": (lambda: simt_config(128, 256, 16, 8, 16, feed="tma", stages=4), dict(wgm=8)),
    "ffma_tma_128x128x16_s4": (lambda: simt_config(128, 128, 16, 8, 8, feed="tma", stages=4), dict(wgm=8)),
    "ffma_tma_128x128x16_t16x8_s6": (lambda: simt_config(128, 128, 16, 16, 8, feed="tma", stages=6), dict(wgm=8)),
    "ffma_tma_256x128x16_s4_nt": (lambda: simt_config(256, 128, 16, 16, 8, trans_b=True, feed="tma", stages=4), dict(wgm=8)),
    "simt_128x64x8_plr0": (lambda: simt_config(128, 64, 8, 8, 4), dict(wgm=1, plr=0)),
    # configurations written the reference's way (GCN MFMA shapes): served by the SIMT kernel
    "legacy_32x32x2_1wave": (lambda: _legacy((32, 32, 1, 2), (1, 1), (1, 1), 16), dict(wgm=1)),
    "legacy_16x16x4_2x2x2x2": (lambda: _legacy((16, 16, 1, 4), (2, 2), (2, 2), 16), dict(wgm=4)),
}

DEFAULT_TENSOR = "tc2_256x256x32_s3"
DEFAULT_SIMT = "simt_128x128x16"


def paths(name: str) -> Tuple[str, str]:
    d = GENERATED_DIR / name
    return str(d / "generated_gemm.cubin"), str(d / "generated_gemm.toml")


_fresh = set()   # kernels whose in-tree files were checked (or built) by this process


def ensure(name: str, force: bool = False) -> Tuple[str, str]:
    """Return (cubin, toml) of a registered kernel, generating and compiling it if it is not there or if the source
    the generator emits today differs from the one the cubin was compiled from (a changed knob or kernel template).

    Check and build run under an exclusive file lock per kernel, so that several processes asking for the same
    kernel at once (one rank per GPU under torchrun) build it once, one after the other finds it fresh, and none
    loads files that another is still writing."""
    cubin, toml = paths(name)
    if name in _fresh and not force:
        return cubin, toml
    import fcntl

    factory, opt_kwargs = REGISTRY[name]
    config, opt = factory(), GemmOptimizations(1, **opt_kwargs)
    folder = GENERATED_DIR / name
    folder.mkdir(parents=True, exist_ok=True)
    with open(folder / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            stale = force or not (Path(cubin).exists() and Path(toml).exists())
            if not stale:
                import tomllib
                source = Path(cubin).with_suffix(".cu")
                stale = not source.exists() or source.read_text() != gemm(None, KERNEL_ENTRY, "sm_100a", config, opt, default_arguments())
                with open(toml, "rb") as f:
                    stale = stale or tomllib.load(f) != config.to_dict()
            if stale:
                build_kernel(str(folder), config, opt)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    _fresh.add(name)
    return cubin, toml


def build_all(force: bool = True, jobs: int = 0) -> Dict[str, Tuple[str, str]]:
    """Generate and compile every registered kernel (nvcc runs as a subprocess, so threads give real parallelism)."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    jobs = jobs or min(8, os.cpu_count() or 1)
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        results = list(pool.map(lambda name: ensure(name, force=force), REGISTRY))
    return dict(zip(REGISTRY, results))


TUNED_TABLE = Path(__file__).resolve().parent / "tuner" / "tuned.json"


def _registered_like(entry) -> str | None:
    """Registered NN kernel with the structure of a tuner-table entry (tile, k per stage, stages, cluster, split
    placement, operand type); the rasterisation width may differ."""
    want_type = {"fp32": DataType.FP32, "fp16": DataType.FP16, "bf16": DataType.BF16}[entry["operands"]]
    for name, (factory, _) in REGISTRY.items():
        try:
            cfg = factory()
        except RuntimeError:
            continue
        if cfg.trans_a or cfg.trans_b or cfg.a_type != want_type or cfg.variant != entry["variant"]:
            continue
        if (list(cfg.tile_size), cfg.depth_k, list(cfg.wave_group)) != (entry["tile"], entry["depth_k"], entry["cluster"]):
            continue
        if cfg.variant == "simt_ffma" and (getattr(cfg, "feed", "ldg") != entry.get("feed", "ldg")
                                           or (cfg.feed == "tma" and cfg.stages != entry["stages"])):
            continue
        if cfg.variant == "tcgen05_3xtf32" and (cfg.stages != entry["stages"] or getattr(cfg, "split", "prepass") != entry["split"]
                                                or getattr(cfg, "a_major", "mn") == "k" or getattr(cfg, "terms", 3) != (3 if want_type == DataType.FP32 else 1)
                                                or getattr(cfg, "epilogue_warps", 8) != 8):
            continue
        return name
    return None


DEFAULT_SIMT_LARGE = "ffma_tma_256x128x32_s3"   # strict FP32 on problems of many 256 x 128 tiles


def recommend(m: int, n: int, k: int, operands: str = "fp32", strict_fp32: bool = False) -> str:
    """Registered kernel to use for a problem of this shape on a B200 (NN layout).

    ``strict_fp32`` asks for the FFMA variant (every product and sum in IEEE FP32, what ``force_variant`` 2 runs): the
    tuner table's FFMA entry nearest to the problem if a registered kernel has its structure, else the TMA-fed kernel
    when the problem has at least two waves of its 256 x 128 tiles, else the register-fed default.

    A handle serves one cubin, so choosing between configurations is the caller's (or the tuner's) job, as in the
    reference where the tuner picks one configuration per problem size.  Two sources, in this order:

      * shapes the runner handles inside the default cubin get the default cubin — tiny problems (its FFMA kernel),
        few flops per byte of A and B or fewer than 2^33 flop (its companion kernels: no pre-pass launch);
      * otherwise the tuner's table (``tuner/tuned.json``, written by ``sgemm_tuner.py --summarise`` from measured
        sweeps): the entry of the same operand type whose problem is nearest in log2 distance, within a factor of two
        in every dimension, if a registered kernel has its structure;
      * otherwise rules condensed from the sweeps: fewer than half a wave of 256 x 256 tiles -> 128 x 128 tiles so
        that more SMs get work; everything else -> CTA pairs on 256 x 256 tiles with the split pre-pass.
    """
    import json
    import math

    flops = 2.0 * m * n * k
    if strict_fp32:
        if operands != "fp32":
            raise ValueError("the FFMA variant computes on FP32 operands only")
        try:
            entries = json.loads(TUNED_TABLE.read_text())["entries"]
        except (OSError, ValueError, KeyError):
            entries = []
        near = None
        for e in entries:
            if e["operands"] != "fp32" or e["variant"] != "simt_ffma":
                continue
            steps = [abs(math.log2(x / y)) for x, y in ((m, e["m"]), (n, e["n"]), (k, e["k"]))]
            if max(steps) <= 1.0 and (near is None or sum(steps) < near[0]):
                near = (sum(steps), e)
        name = _registered_like(near[1]) if near is not None else None
        if name is not None:
            return name
        return DEFAULT_SIMT_LARGE if -(-m // 256) * -(-n // 128) >= 2 * 148 else DEFAULT_SIMT
    if operands == "fp32":
        if flops < 2 ** 27:
            return DEFAULT_SIMT
        if flops / (4.0 * (m * k + k * n)) < 200.0:
            return DEFAULT_TENSOR if min(m, n) < 256 else "tc2i_256x256x32_s3"
        if flops < 2 ** 33:
            return DEFAULT_TENSOR
    try:
        entries = json.loads(TUNED_TABLE.read_text())["entries"]
    except (OSError, ValueError, KeyError):
        entries = []
    nearest = None
    for e in entries:
        if e["operands"] != operands or e["variant"] != "tcgen05_3xtf32":
            continue
        steps = [abs(math.log2(x / y)) for x, y in ((m, e["m"]), (n, e["n"]), (k, e["k"]))]
        if max(steps) <= 1.0 and (nearest is None or sum(steps) < nearest[0]):
            nearest = (sum(steps), e)
    if nearest is not None:
        name = _registered_like(nearest[1])
        if name is not None:
            return name
    if operands != "fp32":
        return "bf16_tc2_256x256x128_s3" if operands == "bf16" else "fp16_tc2_256x256x128_s3"
    if -(-m // 256) * -(-n // 256) < 37:
        return "tc_128x128x32_s3"
    return DEFAULT_TENSOR
