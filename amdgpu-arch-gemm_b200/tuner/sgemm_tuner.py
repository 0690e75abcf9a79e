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

The default search is STAGED instead of the reference's exhaustive product (tuner/sgemm_tuner.py:41-51), which
here would be several hundred compile-and-run points:

  1. every structural configuration (everything but the rasterisation width and the FFMA prefetch depth) gets an
     analytic score — waves the tiles make on the device, shared-memory bytes per tensor-pipe clock, k in flight in
     the stage ring (``predict_efficiency``) — and only the best-scoring ``--shortlist`` of them are ever compiled;
  2. successive halving: the shortlist is measured with few timed runs, its best quarter again with the full count;
  3. the two best are then swept over the knob left out of step 1 (the rasterisation width).

``--exhaustive`` restores the full product.  ``--summarise`` turns result files into the table
``kernels.recommend`` reads (best configuration per problem and variant).
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
SUPPORTED_SPLIT = ["prepass", "inkernel", "hybrid"]   # where the 3xTF32 lo terms are made (hybrid: A's by the pre-pass, B's in the kernel)
# FFMA variant: (thread grid, per-thread tile, k per stage)
SUPPORTED_SIMT = [((16, 16), (8, 8), 16), ((16, 16), (8, 8), 8), ((16, 8), (8, 8), 16), ((8, 16), (8, 8), 16),
                  ((16, 16), (8, 4), 16), ((16, 16), (4, 8), 16), ((32, 8), (4, 8), 16), ((16, 16), (4, 4), 16),
                  ((16, 8), (8, 8), 8), ((32, 16), (4, 8), 16), ((16, 16), (8, 16), 16), ((16, 16), (16, 8), 16),
                  ((8, 16), (16, 8), 16), ((16, 16), (8, 8), 32)]
# FFMA variant fed by TMA (producer thread + mbarrier ring, one block per SM): (thread grid of the consumers,
# per-thread tile, k per stage, stages)
SUPPORTED_SIMT_TMA = [((16, 16), (16, 8), 16, 4), ((16, 16), (16, 8), 16, 3), ((16, 16), (16, 8), 16, 6),
                      ((16, 16), (16, 8), 8, 6), ((16, 16), (16, 8), 32, 3), ((16, 16), (8, 16), 16, 4),
                      ((16, 16), (8, 8), 16, 4), ((32, 16), (8, 8), 16, 4), ((16, 8), (16, 8), 16, 6)]
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
        for (wg, wt, dk, stages), wgm in product(SUPPORTED_SIMT_TMA, SUPPORTED_WGM):
            key = f"simt tma g{wg[0]}x{wg[1]} t{wt[0]}x{wt[1]} k{dk} s{stages} wgm{wgm}"
            yield (key,
                   lambda wg=wg, wt=wt, dk=dk, stages=stages: GemmSolutionConfig(
                       F, F, F, F, (1, 1, 1, 1), wg, wt, dk, False, False, vmem_stage=stages - 1, feed="tma"),
                   lambda wgm=wgm: GemmOptimizations(1, wgm=wgm))


# ------------------------------------------------------------------------------------------ analytic pruning
SM_COUNT = 148                 # B200; only the ranking matters, not the absolute score
SMEM_BYTES_PER_CLK = 118.0     # shared-memory bandwidth of one SM that mixed TMA / tensor-core / warp traffic gets out of the nominal 128
STAGE_ISSUE_CLKS = 520.0       # what issuing one ring stage costs (a dozen TMA copies, its MMAs, two barrier hand-overs)


def predict_time_us(config: GemmSolutionConfig, m: int, n: int, k: int, sm_count: int = SM_COUNT, ghz: float = 1.5) -> float:
    """Microseconds one SGEMM call can be expected to take with this configuration — a coarse model, good enough to
    rank candidates before anything is compiled.  It follows what the runner will do with the kernel:

      launch units   tiles x the split-K factor the runner would choose (too few tiles for the device: K is cut),
                     run in waves of one unit per SM (per SM pair for a CTA pair);
      main loop      per k-slice the tensor pipe needs 2*128*N*mma_k flops / (4096 or, 16-bit, 8192 per clock) for each
                     of the 3 (1) MMAs; the tensor core reads A (128 rows) and B (N / cluster columns) of the slice
                     from shared memory for every MMA — 8192/N + 64/cluster bytes per clock for FP32 — and TMA (with
                     the in-kernel split also the transform warps) writes 2/3 (all) of that again: beyond about 118 of the nominal 128 B/clk the
                     stage ring sets the pace, a ring holding less than about 96 k of FP32 operands in flight
                     cannot cover a TMA round trip, and no stage is faster than its copies and MMAs can be issued;
      around it      ring fill at the start of a unit, the write-out of the last tile, and per dependent launch (split
                     pre-pass, split-K reduction) its latency plus the bytes it moves at HBM speed.
    The FFMA variant is scored on waves of two blocks per SM, FMAs per shared-memory word (per-thread tile) and k
    per stage."""
    tm, tn = config.tile_size
    tiles = -(-m // tm) * -(-n // tn)
    hbm_bytes_per_us = 6.5e6
    launch_us = 2.5
    if config.variant != "tcgen05_3xtf32":
        tma_fed = getattr(config, "feed", "ldg") == "tma"                  # one block per SM on all of its lanes
        slots = sm_count if tma_fed else 2 * sm_count
        kb_total = -(-k // config.depth_k)
        split = min(slots // tiles, kb_total // 8, 32) if tiles * 2 <= slots and kb_total >= 16 else 1
        split = max(split, 1)
        waves = -(-tiles * split // slots)
        ttm, ttn = config.simt_thread_tile
        reuse = min(1.0, 0.4 + 0.6 * (ttm * ttn) / (ttm + ttn) / 4.0)      # FMAs per shared-memory word loaded, 8 x 8 -> 1
        depth = min(1.0, 0.7 + 0.3 * config.depth_k / 16.0)
        k_unit = -(-kb_total // split) * config.depth_k
        # one block computes tm x tn x k_unit FMAs on half an SM's 128 lanes (all of them when fed by TMA, whose
        # multiplying warps issue nothing but fragment loads and FMAs: measured 5 % above the register-fed kernel)
        clks = tm * tn * k_unit / (128.0 if tma_fed else 64.0) / (0.8 * reuse * depth * (1.05 if tma_fed else 1.0))
        extra = (launch_us + (split + 1) * m * n * 4 / hbm_bytes_per_us) if split > 1 else 0.0
        return waves * clks / (ghz * 1e3) + launch_us + extra
    cluster = config.wave_group[0]
    slots = max(1, sm_count // cluster)
    elem = 4 if config.a_type == DataType.FP32 else 2
    terms, mma_k, rate = (3, 8, 4096.0) if elem == 4 else (1, 16, 8192.0)
    kb_total = -(-k // config.depth_k)
    split = min(slots // tiles, kb_total // 8, 32) if tiles * 2 <= slots and kb_total >= 16 else 1
    split = max(split, 1)
    waves = -(-tiles * split // slots)
    k_unit = -(-kb_total // split) * config.depth_k
    clks_per_slice = terms * 2.0 * 128 * tn * mma_k / rate
    reads = terms * (128 + tn / cluster) * mma_k * elem / clks_per_slice          # bytes per clock the tensor core reads
    placement = getattr(config, "split", "prepass")
    inkernel = placement != "prepass"
    # TMA (+ transform warps) into the ring: four tiles by TMA; two by TMA and two read + written by the warps; three + one
    writes = reads * ({"prepass": 2.0 / 3.0, "inkernel": 1.0, "hybrid": 5.0 / 6.0}[placement] if terms == 3 else 1.0)
    smem_eff = min(1.0, SMEM_BYTES_PER_CLK / (reads + writes))
    k_in_flight = (config.stages - 1) * config.depth_k * elem / 4.0
    depth_eff = min(1.0, 0.55 + 0.45 * k_in_flight / 96.0)
    # per ring stage one thread issues the TMA copies and one the MMAs and commits: a stage cannot take less than that
    stage_clks = max(config.depth_k / mma_k * clks_per_slice / (smem_eff * depth_eff), STAGE_ISSUE_CLKS)
    main_clks = k_unit / config.depth_k * stage_clks
    fill_clks = 1800.0 + (400.0 if inkernel else 0.0)
    store_clks = 128.0 * tn * 4 / 48.0                                            # the last tile's write-out, not overlapped
    t = (waves * main_clks + fill_clks + store_clks) / (ghz * 1e3) + launch_us
    if cluster > 1:
        t += 4.0   # a cluster launch is scheduled pair by pair and synchronises cluster-wide at set-up and teardown
    if terms == 3 and placement != "inkernel":
        prepass_elems = (m * k + k * n) if placement == "prepass" else m * k        # the split pre-pass reads and writes A and B (hybrid: A)
        t += launch_us + 2.0 * prepass_elems * 4 / hbm_bytes_per_us
    if split > 1:
        t += launch_us + (split + 1) * m * n * 4 / hbm_bytes_per_us               # partial sums out and in again
    return t


def predict_efficiency(config: GemmSolutionConfig, m: int, n: int, k: int, sm_count: int = SM_COUNT) -> float:
    """Ranking score: the problem's flops over the predicted time, as a fraction of the variant's pipe peak at the
    model's clock (higher is better; only the order matters)."""
    ghz = 1.5
    if config.variant == "tcgen05_3xtf32":
        rate = (4096.0 / 3.0) if config.a_type == DataType.FP32 else 8192.0
    else:
        rate = 256.0
    peak_flops_per_us = rate * sm_count * ghz * 1e3
    return 2.0 * m * n * k / predict_time_us(config, m, n, k, sm_count, ghz) / peak_flops_per_us


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


def structural_candidates(include_simt: bool = True, include_tensor: bool = True, ab_type: DataType = DataType.FP32):
    """The search space without the knob that does not change the kernel's structure (the rasterisation width): yields
    (structural key, config factory, variations) where ``variations`` lists the (key suffix, optimisation factory)
    pairs of that structure, the default one (rasterisation width 8) first."""
    F = DataType.FP32
    half = ab_type != DataType.FP32
    depth_ks = SUPPORTED_DEPTH_K_16BIT if half else SUPPORTED_DEPTH_K
    splits = ["prepass"] if half else SUPPORTED_SPLIT
    default_wgm = 8 if 8 in SUPPORTED_WGM else SUPPORTED_WGM[0]
    wgms = [default_wgm] + [w for w in SUPPORTED_WGM if w != default_wgm]
    if include_tensor:
        for cluster, bn, dk, stages, split in product(SUPPORTED_CLUSTERS, SUPPORTED_TILE_N, depth_ks, SUPPORTED_STAGES, splits):
            key = f"tensor{'' if not half else ' ' + ab_type.name.lower()} c{cluster[0]}x{cluster[1]} n{bn} k{dk} s{stages} {split}"
            yield (key,
                   lambda cluster=cluster, bn=bn, dk=dk, stages=stages, split=split: GemmSolutionConfig(
                       ab_type, ab_type, F, F, (128, bn, 1, 16 if half else 8), cluster, (1, 1), dk, False, False,
                       vmem_stage=stages - 1, split=split),
                   [(f" wgm{w}", lambda w=w: GemmOptimizations(1, wgm=w)) for w in wgms])
    if include_simt and not half:
        # (the FFMA kernel's prefetch depth changes its register pipeline, and which depth wins depends on the tile: it
        # is part of the structure, not a knob to sweep afterwards)
        for (wg, wt, dk), plr in product(SUPPORTED_SIMT, SUPPORTED_PLR):
            key = f"simt g{wg[0]}x{wg[1]} t{wt[0]}x{wt[1]} k{dk} plr{plr}"
            yield (key,
                   lambda wg=wg, wt=wt, dk=dk: GemmSolutionConfig(F, F, F, F, (1, 1, 1, 1), wg, wt, dk, False, False),
                   [(f" wgm{w}", lambda w=w, plr=plr: GemmOptimizations(1, wgm=w, plr=plr)) for w in wgms])
        for wg, wt, dk, stages in SUPPORTED_SIMT_TMA:
            key = f"simt tma g{wg[0]}x{wg[1]} t{wt[0]}x{wt[1]} k{dk} s{stages}"
            yield (key,
                   lambda wg=wg, wt=wt, dk=dk, stages=stages: GemmSolutionConfig(
                       F, F, F, F, (1, 1, 1, 1), wg, wt, dk, False, False, vmem_stage=stages - 1, feed="tma"),
                   [(f" wgm{w}", lambda w=w: GemmOptimizations(1, wgm=w)) for w in wgms])


class Measurer:
    """Generates, compiles and runs one configuration through the runner program and keeps the JSONL log; a point that
    is already in the log is not run again (resume).  ``runs`` is the number of timed launches asked of the runner;
    a logged measurement with at least as many runs is reused."""

    def __init__(self, m: int, n: int, k: int, bench: str, output_folder: str, allow_ragged: bool = False,
                 limit: int | None = None):
        self.m, self.n, self.k, self.bench, self.out = m, n, k, bench, output_folder
        self.allow_ragged, self.limit = allow_ragged, limit
        os.makedirs(output_folder, exist_ok=True)
        self.log_path = Path(output_folder) / "tuner_results.jsonl"
        self.done = load_done(self.log_path)
        self.measured = 0

    def admissible(self, config: GemmSolutionConfig) -> bool:
        """The reference's filters (tuner/sgemm_tuner.py:97,102): tile divisibility and 16-byte loads."""
        m, n, k = self.m, self.n, self.k
        if not self.allow_ragged and ((m % config.tile_size[0]) or (n % config.tile_size[1]) or (k % config.depth_k)):
            if VERBOSE:
                print(f"{m}, {n}, {k} were not divisible by {config.tile_size[0]}, {config.tile_size[1]}, {config.depth_k}")
            return False
        return not (config.num_bytes_per_buffer_load[0] % 16 or config.num_bytes_per_buffer_load[1] % 16)

    def __call__(self, key: str, config: GemmSolutionConfig, opt: GemmOptimizations, runs: int = 50):
        """Record of the point (from the log, or measured now), or None when it was skipped."""
        problem_key = f"{self.m}x{self.n}x{self.k} {key}"
        rec = self.done.get(problem_key)
        if rec is not None and (rec.get("returncode") or rec.get("runs", 50) >= runs):
            return rec
        if self.limit is not None and self.measured >= self.limit:
            return None
        src = gemm(None, KERNEL_NAME, ARCH, config, opt, kernel_arguments())
        if compile(KERNEL_NAME, src, ARCH, self.out, config):
            if VERBOSE:
                print("compile error")
            return None
        ret = subprocess.run([self.bench, f"{self.out}/{KERNEL_NAME}.cubin", f"{self.out}/{KERNEL_NAME}.toml",
                              str(self.m), str(self.n), str(self.k), "5", str(runs), "0"], stdout=subprocess.PIPE, stderr=subprocess.PIPE)
        self.measured += 1
        rec = {"key": problem_key, "returncode": ret.returncode, "tile": list(config.tile_size), "depth_k": config.depth_k,
               "stages": config.stages, "cluster": list(config.wave_group), "variant": config.variant, "wgm": opt.wgm,
               "plr": opt.plr, "split": getattr(config, "split", ""), "feed": getattr(config, "feed", "ldg"), "runs": runs}
        if not ret.returncode:
            rec["gflops"] = parse_gflops(ret.stdout.decode())
        else:
            rec["stderr"] = ret.stderr.decode()[-300:]
        with open(self.log_path, "a") as f:
            f.write(json.dumps(rec) + "\n")
        self.done[problem_key] = rec
        return rec


def describe(rec) -> str:
    """The variant of a record and what distinguishes kernels within it: where the lo terms are made (tensor variant),
    how the tiles reach shared memory (FFMA variant)."""
    if rec["variant"] == "simt_ffma":
        return f"simt_ffma {'tma' if rec.get('feed') == 'tma' or ' tma ' in rec.get('key', '') else 'ldg'}-fed"
    return f"{rec['variant']} {rec.get('split', '')}"


def report(rec) -> None:
    print(f"Gflops: {rec['gflops']}, MT: {tuple(rec['tile'])}, DK: {rec['depth_k']}, wgm: {rec['wgm']}, plr: {rec['plr']}, "
          f"stages: {rec['stages']}, cluster: {tuple(rec['cluster'])}, variant: {describe(rec)}")


def staged_search(points, measure, m: int, n: int, k: int, shortlist: int = 40, short_runs: int = 5, long_runs: int = 50,
                  sweep_best: int = 2, sweep_budget: int = 8):
    """The pruned search over ``points`` = [(structural key, config, variations)] with ``measure(key, config, opt, runs)``
    -> record or None.  Returns (best record, number of ``measure`` calls made)."""
    scored = sorted(points, key=lambda p: -predict_efficiency(p[1], m, n, k))
    calls = 0

    def run(point, variation, runs):
        nonlocal calls
        key, config, variations = point
        suffix, make_opt = variations[variation]
        calls += 1
        rec = measure(key + suffix, config, make_opt(), runs)
        if rec is None or rec.get("returncode"):
            if rec is not None:
                print(f"runner failed for {rec['key']} (exit {rec['returncode']})")
            return None
        report(rec)
        return rec

    # 1 + 2a: the analytic shortlist, measured briefly in its default variation
    first = [(p, run(p, 0, short_runs)) for p in scored[:shortlist]]
    first = sorted([(p, r) for p, r in first if r is not None], key=lambda pr: -pr[1]["gflops"])
    # 2b: the best quarter again, with the full number of runs
    second = [(p, run(p, 0, long_runs)) for p, _ in first[:max(sweep_best, (len(first) + 3) // 4)]]
    second = sorted([(p, r) for p, r in second if r is not None], key=lambda pr: -pr[1]["gflops"])
    results = [r for _, r in second]
    # 3: the knobs left out so far, on the best few structures (best first, at most `sweep_budget` measurements)
    for p, _ in second[:sweep_best]:
        for variation in range(1, len(p[2])):
            if sweep_budget <= 0:
                break
            sweep_budget -= 1
            rec = run(p, variation, long_runs)
            if rec is not None:
                results.append(rec)
    best = max(results, key=lambda r: r["gflops"]) if results else None
    return best, calls


def tune(m: int, n: int, k: int, bench: str, output_folder: str, include_simt: bool = True, allow_ragged: bool = False,
         limit: int | None = None, include_tensor: bool = True, ab_type: DataType = DataType.FP32,
         exhaustive: bool = False, shortlist: int = 40):
    measure = Measurer(m, n, k, bench, output_folder, allow_ragged, limit)
    points = []
    for key, make_config, variations in structural_candidates(include_simt, include_tensor, ab_type):
        try:
            config = make_config()
            gemm(None, KERNEL_NAME, ARCH, config, variations[0][1](), kernel_arguments())   # infeasible points raise here
        except RuntimeError as e:
            if VERBOSE:
                print(e)
            continue
        if measure.admissible(config):
            points.append((key, config, variations))
    best = None
    if exhaustive:
        for key, config, variations in points:
            for suffix, make_opt in variations:
                rec = measure(key + suffix, config, make_opt())
                if rec is None:
                    continue
                if rec.get("returncode"):
                    print(f"runner failed for {rec['key']} (exit {rec['returncode']})")
                    continue
                report(rec)
                if best is None or rec["gflops"] > best["gflops"]:
                    best = rec
    else:
        best, calls = staged_search(points, measure, m, n, k, shortlist=shortlist)
        total = sum(len(v) for _, _, v in points)
        print(f"staged search: {calls} measurements asked for ({measure.measured} new) of {total} points in the full product")
    if best is not None:
        print(f"Best: {best['gflops']} Gflops, MT: {tuple(best['tile'])}, DK: {best['depth_k']}, wgm: {best['wgm']}, "
              f"plr: {best['plr']}, stages: {best['stages']}, cluster: {tuple(best['cluster'])}, variant: {describe(best)}")
    else:
        print("No valid configurations found.")
    return best


def summarise(paths, table_path: str, merge: bool = True) -> dict:
    """Best measured configuration per (problem, variant, operand type) over result files -> the JSON table
    ``kernels.recommend`` consults (``tuner/tuned.json``).  With ``merge`` the entries of an existing table are kept
    unless a result file holds a faster configuration for the same slot (sweeps come from different sessions)."""
    best = {}
    if merge and Path(table_path).exists():
        try:
            for e in json.loads(Path(table_path).read_text())["entries"]:
                best[f"{e['m']}x{e['n']}x{e['k']} {e['variant']} {e['operands']}"] = e
        except (ValueError, KeyError):
            best = {}
    for path in paths:
        for rec in load_done(Path(path)).values():
            if rec.get("returncode") or "gflops" not in rec:
                continue
            if rec.get("runs", 50) < 20:
                continue   # a first-round measurement of the staged search: a few launches at burst clocks, not comparable
            problem, _, rest = rec["key"].partition(" ")
            words = rest.split()
            operand = words[1] if len(words) > 1 and words[1] in ("bf16", "fp16") else "fp32"
            slot = f"{problem} {rec['variant'] if words[0] == 'tensor' else 'simt_ffma'} {operand}"
            if slot not in best or rec["gflops"] > best[slot]["gflops"]:
                m, n, k = (int(x) for x in problem.split("x"))
                best[slot] = {"m": m, "n": n, "k": k, "operands": operand, "variant": rec["variant"], "gflops": rec["gflops"],
                              "tile": rec["tile"], "depth_k": rec["depth_k"], "stages": rec["stages"], "cluster": rec["cluster"],
                              "wgm": rec["wgm"], "plr": rec["plr"], "split": rec.get("split") or "prepass",
                              "feed": "tma" if rec.get("feed") == "tma" or " tma " in rec["key"] else "ldg", "key": rec["key"]}
    table = {"entries": sorted(best.values(), key=lambda e: (e["operands"], e["variant"], e["m"] * e["n"] * e["k"]))}
    Path(table_path).write_text(json.dumps(table, indent=1) + "\n")
    return table


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    summarising = "--summarise" in sys.argv
    ap.add_argument("--m", dest="m", type=int, required=not summarising, action="store")
    ap.add_argument("--n", dest="n", type=int, required=not summarising, action="store")
    ap.add_argument("--k", dest="k", type=int, required=not summarising, action="store")
    ap.add_argument("--bench", dest="bench", type=str, required=not summarising, action="store")
    ap.add_argument("--output-folder", dest="output_folder", type=str, required=not summarising, action="store")
    ap.add_argument("--no-simt", action="store_true", help="search the tensor-core variant only")
    ap.add_argument("--no-tensor", action="store_true", help="search the FFMA variant only")
    ap.add_argument("--allow-ragged", action="store_true", help="keep tilings that do not divide M, N, K")
    ap.add_argument("--limit", type=int, default=None, help="stop after this many new measurements")
    ap.add_argument("--ab-type", choices=["fp32", "fp16", "bf16"], default="fp32",
                    help="element type of A and B (fp16 / bf16: tensor variant only; the reference has fp32 only)")
    ap.add_argument("--exhaustive", action="store_true", help="measure the full product like the reference instead of the staged search")
    ap.add_argument("--shortlist", type=int, default=40, help="structural configurations kept by the analytic ranking")
    ap.add_argument("--summarise", nargs="+", metavar="JSONL", default=None,
                    help="write the best-per-problem table from these result files to --table and exit")
    ap.add_argument("--table", default=str(Path(__file__).resolve().parent / "tuned.json"))
    args = ap.parse_args()
    if args.summarise:
        print(f"{len(summarise(args.summarise, args.table)['entries'])} entries -> {args.table}")
        raise SystemExit(0)
    tune(args.m, args.n, args.k, args.bench, args.output_folder, include_simt=not args.no_simt,
         allow_ragged=args.allow_ragged, limit=args.limit, include_tensor=not args.no_tensor,
         ab_type=DataType[args.ab_type.upper()], exhaustive=args.exhaustive, shortlist=args.shortlist)
