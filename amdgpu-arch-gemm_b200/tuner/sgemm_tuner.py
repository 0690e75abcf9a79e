"""Grid-search tuner for the sm_100a SGEMM kernels.

Same workflow and CLI as the reference's tuner (tuner/sgemm_tuner.py:24-128): for every knob combination build a
``GemmSolutionConfig`` (infeasible ones raise ``RuntimeError`` and are skipped), generate, filter, compile, run the
runner program as ``<bench> <out>/generated_gemm.cubin <out>/generated_gemm.toml m n k 5 50 0``, read the measured
``Gflops`` from the third line from the end of its stdout, keep the best.

    python tuner/sgemm_tuner.py --m 8192 --n 8192 --k 8192 --bench build/GeneratorRunner --output-folder out

What differs: the search lists are the sm_100a knobs (MMA atom / variant, cluster shape, tile N, k per stage,
pipeline stages, rasterisation width) instead of wave tilings and MFMA shapes; every measured configuration is
appended to ``<out>/tuner_results.jsonl`` and skipped on the next run (the reference keeps its best only in
memory and loses everything on a crash); a runner that exits non-zero is recorded and skipped instead of ending
the search with ``assert False``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from itertools import product
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from generator.generator import (  # noqa: E402
    compile,
    gemm,
    GemmSolutionConfig,
    GemmOptimizations,
    DataType,
    FunctionArgument,
)

# tensor-core variant: (cluster M, tile N, k per stage, stages)
SUPPORTED_CLUSTERS = [(1, 1), (2, 1)]
SUPPORTED_TILE_N = [128, 256]
SUPPORTED_DEPTH_K = [16, 32, 64]
SUPPORTED_DEPTH_K_16BIT = [32, 64, 128]   # 16-bit operands: 64-byte rows, or whole 128-byte rows of 64 k
SUPPORTED_STAGES = [2, 3, 4, 5, 6, 7]
SUPPORTED_SPLIT = ["prepass", "inkernel"]   # where the 3xTF32 lo terms are made
# FFMA variant: (thread grid, per-thread tile, k per stage)
SUPPORTED_SIMT = [((16, 16), (8, 8), 16), ((16, 16), (8, 8), 8), ((16, 8), (8, 8), 16), ((8, 16), (8, 8), 16),
                  ((16, 16), (8, 4), 16), ((16, 16), (4, 8), 16), ((32, 8), (4, 8), 16), ((16, 16), (4, 4), 16),
                  ((16, 8), (8, 8), 8), ((32, 16), (4, 8), 16), ((16, 16), (8, 16), 16), ((16, 16), (16, 8), 16),
                  ((8, 16), (16, 8), 16), ((16, 16), (8, 8), 32)]
SUPPORTED_WGM = [1, 4, 8, 16]
SUPPORTED_PLR = [0, 1]
VERBOSE = False
KERNEL_NAME = "generated_gemm"
ARCH = "sm_100a"


def kernel_arguments():
    names = [("global_buffer", n, 8) for n in "abcd"]
    names += [("by_value", n, 4) for n in ("m", "n", "k", "lda", "ldb", "ldc", "ldd", "alpha", "beta",
                                            "numWorkgroupX", "numWorkgroupY")]
    return [FunctionArgument(t, n, None, s) for t, n, s in names]


def candidates(include_simt: bool = True, include_tensor: bool = True, ab_type: DataType = DataType.FP32):
    """Yield (key, config factory, optimisation factory) for every point of the search space.  ``ab_type`` FP16 or
    BF16 searches the tensor variant for 16-bit operands (atom K = 16, no split placement, no FFMA variant)."""
    F = DataType.FP32
    half = ab_type != DataType.FP32
    depth_ks = SUPPORTED_DEPTH_K_16BIT if half else SUPPORTED_DEPTH_K
    splits = ["prepass"] if half else SUPPORTED_SPLIT
    tensor_space = product(SUPPORTED_CLUSTERS, SUPPORTED_TILE_N, depth_ks, SUPPORTED_STAGES, splits,
                           SUPPORTED_WGM) if include_tensor else ()
    for cluster, bn, dk, stages, split, wgm in tensor_space:
        key = f"tensor{'' if not half else ' ' + ab_type.name.lower()} c{cluster[0]}x{cluster[1]} n{bn} k{dk} s{stages} {split} wgm{wgm}"
        yield (key,
               lambda cluster=cluster, bn=bn, dk=dk, stages=stages, split=split: GemmSolutionConfig(
                   ab_type, ab_type, F, F, (128, bn, 1, 16 if half else 8), cluster, (1, 1), dk, False, False,
                   vmem_stage=stages - 1, split=split),
               lambda wgm=wgm: GemmOptimizations(1, wgm=wgm))
    if include_simt and not half:
        for (wg, wt, dk), wgm, plr in product(SUPPORTED_SIMT, SUPPORTED_WGM, SUPPORTED_PLR):
            key = f"simt g{wg[0]}x{wg[1]} t{wt[0]}x{wt[1]} k{dk} wgm{wgm} plr{plr}"
            yield (key,
                   lambda wg=wg, wt=wt, dk=dk: GemmSolutionConfig(F, F, F, F, (1, 1, 1, 1), wg, wt, dk, False, False),
                   lambda wgm=wgm, plr=plr: GemmOptimizations(1, wgm=wgm, plr=plr))


def parse_gflops(stdout: str) -> float:
    """The measured block's ``Gflops:`` line is the third line from the end (tuner/sgemm_tuner.py:115)."""
    return float(stdout.split("\n")[-3].split(":")[-1])


def load_done(path: Path):
    done = {}
    if path.exists():
        for line in path.read_text().splitlines():
            try:
                rec = json.loads(line)
                done[rec["key"]] = rec
            except (ValueError, KeyError):
                continue
    return done


def tune(m: int, n: int, k: int, bench: str, output_folder: str, include_simt: bool = True, allow_ragged: bool = False,
         limit: int | None = None, include_tensor: bool = True, ab_type: DataType = DataType.FP32):
    os.makedirs(output_folder, exist_ok=True)
    log_path = Path(output_folder) / "tuner_results.jsonl"
    done = load_done(log_path)
    best = None
    measured = 0
    for key, make_config, make_opt in candidates(include_simt, include_tensor, ab_type):
        problem_key = f"{m}x{n}x{k} {key}"
        if problem_key in done:
            rec = done[problem_key]
        else:
            try:
                config = make_config()
                opt = make_opt()
                src = gemm(None, KERNEL_NAME, ARCH, config, opt, kernel_arguments())
            except RuntimeError as e:
                if VERBOSE:
                    print(e)
                continue
            if not allow_ragged and ((m % config.tile_size[0]) or (n % config.tile_size[1]) or (k % config.depth_k)):
                if VERBOSE:
                    print(f"{m}, {n}, {k} were not divisible by {config.tile_size[0]}, {config.tile_size[1]}, {config.depth_k}")
                continue
            if config.num_bytes_per_buffer_load[0] % 16 or config.num_bytes_per_buffer_load[1] % 16:
                continue
            if limit is not None and measured >= limit:
                break
            if compile(KERNEL_NAME, src, ARCH, output_folder, config):
                if VERBOSE:
                    print("compile error")
                continue
            ret = subprocess.run([bench, f"{output_folder}/{KERNEL_NAME}.cubin", f"{output_folder}/{KERNEL_NAME}.toml",
                                  str(m), str(n), str(k), "5", "50", "0"], stdout=subprocess.PIPE, stderr=subprocess.PIPE)
            measured += 1
            rec = {"key": problem_key, "returncode": ret.returncode, "tile": list(config.tile_size), "depth_k": config.depth_k,
                   "stages": config.stages, "cluster": list(config.wave_group), "variant": config.variant, "wgm": opt.wgm,
                   "plr": opt.plr, "split": getattr(config, "split", "")}
            if not ret.returncode:
                rec["gflops"] = parse_gflops(ret.stdout.decode())
            else:
                rec["stderr"] = ret.stderr.decode()[-300:]
            with open(log_path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        if rec.get("returncode"):
            print(f"runner failed for {rec['key']} (exit {rec['returncode']})")
            continue
        print(f"Gflops: {rec['gflops']}, MT: {tuple(rec['tile'])}, DK: {rec['depth_k']}, wgm: {rec['wgm']}, plr: {rec['plr']}, "
              f"stages: {rec['stages']}, cluster: {tuple(rec['cluster'])}, variant: {rec['variant']} {rec.get('split', '')}")
        if best is None or rec["gflops"] > best["gflops"]:
            best = rec
    if best is not None:
        print(f"Best: {best['gflops']} Gflops, MT: {tuple(best['tile'])}, DK: {best['depth_k']}, wgm: {best['wgm']}, "
              f"plr: {best['plr']}, stages: {best['stages']}, cluster: {tuple(best['cluster'])}, variant: {best['variant']} "
              f"{best.get('split', '')}")
    else:
        print("No valid configurations found.")
    return best


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", dest="m", type=int, required=True, action="store")
    ap.add_argument("--n", dest="n", type=int, required=True, action="store")
    ap.add_argument("--k", dest="k", type=int, required=True, action="store")
    ap.add_argument("--bench", dest="bench", type=str, required=True, action="store")
    ap.add_argument("--output-folder", dest="output_folder", type=str, required=True, action="store")
    ap.add_argument("--no-simt", action="store_true", help="search the tensor-core variant only")
    ap.add_argument("--no-tensor", action="store_true", help="search the FFMA variant only")
    ap.add_argument("--allow-ragged", action="store_true", help="keep tilings that do not divide M, N, K")
    ap.add_argument("--limit", type=int, default=None, help="stop after this many new measurements")
    ap.add_argument("--ab-type", choices=["fp32", "fp16", "bf16"], default="fp32",
                    help="element type of A and B (fp16 / bf16: tensor variant only; the reference has fp32 only)")
    args = ap.parse_args()
    tune(args.m, args.n, args.k, args.bench, args.output_folder, include_simt=not args.no_simt,
         allow_ragged=args.allow_ragged, limit=args.limit, include_tensor=not args.no_tensor,
         ab_type=DataType[args.ab_type.upper()])
