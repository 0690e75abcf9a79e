#!/usr/bin/env python
"""SGEMM benchmark: FP32-accurate TFLOPS of the column-major NN SGEMM at M = N = K = 8192 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--kernel NAME]

One process per GPU (N > 1: launched by torch.distributed.run, one rank per GPU).  A "step" is one SGEMM
D = A*B (alpha = 1, beta = 0) through the C ABI of libsgemm_runner.so; with N ranks the problem is
M = K = 8192, N_total = 8192 * N, column-block sharded: A replicated, B and D column-partitioned, no collective
on the compute path (weak scaling: fixed work per GPU).  Inputs are seeded uniform[-1, 1) FP32 filled on the
device by global element index, so every N sees the same matrices.

What one JSON line carries:
  value / ms_per_step   K steps between CUDA events on the launching stream, bracketed by barrier + synchronise, max
                        over ranks; algorithmic flops 2*M*N*K only (the 3x tensor work of the split is not counted),
                        the split pre-pass that is part of every call included.
  roofline              the main kernel alone (event pairs around each of its launches inside the same timed region)
                        against the tensor ceiling for FP32-accurate flops; the ceiling is the burst figure of the
                        measured peaks for a timed region shorter than a second, the sustained one otherwise.
  sustained             the same step repeated for at least three seconds with the SM clock sampled throughout.
  parity                after the timed regions every rank checks sampled columns of its own shard of D against the CPU
                        oracle (the checker; never inside a timed region).
  c5                    the fixed M = N = 32768, K = 8192 problem column-sharded over the N ranks (strong scaling),
                        at least two seconds of timed steps, with its own parity check.
  e2e                   the measurement through the host-buffer entry points with pinned HOST buffers, uploads and
                        downloads inside the timed region; with N ranks every rank uploads 1/N of the replicated A and
                        the ranks complete it with an all-gather over NVLink (sgemm_run_host_sharded).
  ffma_path             the same problem on the FFMA kernel (strict FP32), with the FP32 FMA peak at the sampled clock.
  cpu_baseline          the reference's CPU GEMM (oracle restatement) on the box's host cores, N = 1 only.

--impl reference times the reference's CPU GEMM (restated in oracle/, its native runner needs HIP and cannot be
built here) on all host cores, on a column block of the same 8192^3 problem.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N_PER_GPU = K = 8192
METRIC = "sgemm_fp32_accurate_tflops_8192"
UNIT = "TFLOP/s"
C5_M, C5_N, C5_K = 32768, 32768, 8192
TRAFFIC_FILE = ROOT / "profiles" / "dram_traffic.json"
# flops per clock and SM of the tensor pipe on TF32 operands (the ncu counter sm__ops_path_tensor_op_utchmma_src_tf32
# saturates at this value); a third of it is the ceiling of the 3xTF32 scheme at a given clock
TF32_FLOPS_PER_CLK_SM = 4096


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def ncu_traffic(kernel: str, cubin: str, shape):
    """DRAM bytes one launch of the dominant kernel moved in an ncu capture, from the tracked record beside the
    profile summaries — valid only for the very source the capture ran: the record carries a hash of the emitted .cu,
    and a kernel that has changed since gets null instead of a stale figure."""
    try:
        rec = json.loads(TRAFFIC_FILE.read_text()).get(kernel)
        src = Path(cubin).with_suffix(".cu").read_bytes()
    except (OSError, ValueError):
        return None, "no record"
    if not rec or list(rec.get("shape", [])) != list(shape):
        return None, "no record for this kernel and shape"
    if rec.get("source_sha256") != hashlib.sha256(src).hexdigest():
        return None, "kernel source changed since the capture"
    return rec.get("dram_bytes_per_launch"), rec.get("capture")


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read (never set) every few milliseconds through NVML in a
    thread of this process while a timed region runs; falls back to an `nvidia-smi -lms 100` child when the NVML
    binding is not importable.  A region with fewer than five samples is reported as `valid: false`."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_uuid: str | None, gpu_index: int, period_s: float = 0.004):
        self.uuid, self.gpu_index, self.period_s = gpu_uuid, gpu_index, period_s
        self.samples = []            # (sm_mhz, power_w, reasons bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._proc = None
        self._lines = []
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._dev = (pynvml.nvmlDeviceGetHandleByUUID(gpu_uuid.encode() if isinstance(gpu_uuid, str) else gpu_uuid)
                         if gpu_uuid else pynvml.nvmlDeviceGetHandleByIndex(gpu_index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._dev, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _loop(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._dev, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._dev)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._dev)
                try:
                    power = nv.nvmlDeviceGetPowerUsage(self._dev) / 1000.0
                except Exception:
                    power = None
                self.samples.append((float(mhz), power, int(mask)))
            except Exception:
                pass
            self._stop.wait(self.period_s)

    def start(self):
        self.samples, self._lines = [], []
        self._stop.clear()
        if self._nvml:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
            return
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                           "-lms", "100", "-i", str(self.gpu_index)],
                                          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=lambda: [self._lines.append(l) for l in self._proc.stdout], daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None

    def stop(self):
        self._stop.set()
        if self._nvml:
            if self._thread:
                self._thread.join(timeout=2)
            nv = self._nvml
            names = (("hw_slowdown", nv.nvmlClocksThrottleReasonHwSlowdown),
                     ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown),
                     ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap))
            sm = [s[0] for s in self.samples]
            power = [s[1] for s in self.samples if s[1] is not None]
            reasons = sorted({name for name, bit in names for s in self.samples if s[2] & bit})
            source = "nvml"
        elif self._proc:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            sm, smax, power, found = [], [], [], set()
            for line in self._lines:
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        found.add(name)
            self.max_mhz = max(smax) if smax else None
            reasons = sorted(found)
            source = "nvidia-smi"
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "valid": False, "reasons": ["no clock source available"]}
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_mhz_min": min(sm) if sm else None,
                "sm_max_mhz": self.max_mhz, "power_w_max": max(power) if power else None, "samples": len(sm),
                "valid": len(sm) >= 5, "reasons": reasons, "source": source}


def cpu_reference_tflops(oracle, budget_s: float = 12.0, cols: int | None = None):
    """The reference's CPU GEMM (oracle restatement, all host threads) on a column block of the 8192^3 problem.
    Without `cols` the block is grown until one product takes about `budget_s` / 3 seconds or more.
    Returns (tflops, columns used, seconds, threads)."""
    oracle.use_all_cores()
    a = oracle.fill_uniform(M * K, 0)
    fixed = cols is not None
    cols = cols or 64
    while True:
        b = oracle.fill_uniform(K * cols, 1)
        t0 = time.perf_counter()
        oracle.gemm(a, b, None, 1.0, 0.0, M, cols, K)
        dt = time.perf_counter() - t0
        if fixed or dt >= budget_s / 3 or cols >= N_PER_GPU:
            break
        cols = min(N_PER_GPU, max(cols * 2, int(cols * (budget_s * 0.6) / max(dt, 1e-3)) // 64 * 64))
    return 2.0 * M * cols * K / dt * 1e-12, cols, dt, oracle.num_threads()


def cpu_reference_order(oracle):
    """The reference's loop nest as written (i, j, l; one thread; runner/generator_runner.cpp:21-32) timed at 32^3 and
    1024^3 — the reference's own CPU path, next to the reordered all-core figure."""
    out = {}
    for size, repeats in ((32, 200), (1024, 1)):
        a, b, c = oracle.make_inputs(size, size, size, seed=0)
        oracle.gemm(a[: 32 * 32], b[: 32 * 32], None, 1.0, 0.0, 32, 32, 32, ref_order=True)   # page the code in
        t0 = time.perf_counter()
        for _ in range(repeats):
            oracle.gemm(a, b, c, 1.0, 0.0, size, size, size, ref_order=True)
        dt = (time.perf_counter() - t0) / repeats
        out[f"{size}^3"] = {"seconds": dt, "gflops": 2.0 * size ** 3 / dt * 1e-9}
    out["8192^3"] = {"seconds": out["1024^3"]["seconds"] * 512, "extrapolated": "1024^3 time x 512"}
    return out


def run_reference(args, rank):
    if rank != 0:
        return
    from oracle import oracle
    # one step = the CPU GEMM on a fixed column block of the problem, sized in a calibration pass so that the whole
    # run (warm-up + steps) takes about two minutes at most, and at least 64 columns per step
    _, c0, t0, threads = cpu_reference_tflops(oracle, cols=64)
    per_step_s = min(8.0, max(0.2, 110.0 / max(args.warmup + args.steps, 1)))
    cols = int(min(N_PER_GPU, max(64, (64 * per_step_s / max(t0, 1e-3)) // 64 * 64)))
    times = []
    for i in range(args.warmup + args.steps):
        tf, cols, dt, threads = cpu_reference_tflops(oracle, cols=cols)
        if i >= args.warmup:
            times.append((tf, dt))
    tf = statistics.mean(t for t, _ in times)
    sample = f"column block of {cols} of 8192 columns of the 8192^3 problem per step (all {M} rows, full K)"
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": statistics.mean(d for _, d in times) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "column-major NN SGEMM M=N=K=8192, alpha=1, beta=0, seeded uniform[-1,1)",
                   "arm": "reference CPU GEMM (runner/generator_runner.cpp cpuGemm arithmetic, OpenMP over columns)"},
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class Job:
    """One rank's view of a column-sharded SGEMM workload on its GPU: buffers, workspace, step, timing, parity."""

    def __init__(self, torch, dist, api_runner, dev, world, rank, m, n_total, k, stream):
        from runner.shard import fill_shard_inputs, shard_columns
        self.torch, self.dist, self.r, self.dev, self.world, self.rank = torch, dist, api_runner, dev, world, rank
        self.m, self.n_total, self.k, self.stream = m, n_total, k, stream
        self.tile_n = self.r.info("tile_n")
        self.n0, self.n1 = shard_columns(n_total, world, rank, self.tile_n)
        self.n_local = self.n1 - self.n0
        self.a = torch.empty(m * k, dtype=torch.float32, device=dev)
        self.b = torch.empty(max(k * self.n_local, 1), dtype=torch.float32, device=dev)
        self.d = torch.zeros(max(m * self.n_local, 1), dtype=torch.float32, device=dev)
        self.last_device_mhz = None
        fill_shard_inputs(self.r, self.a, self.b, m, k, self.n0, self.n1, seed=0, stream=stream)
        ws_bytes = self.r.workspace_bytes(m, max(self.n_local, 1), k)
        self.ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        self.r.set_workspace(self.ws, ws_bytes)
        torch.cuda.synchronize()

    def step(self):
        if self.n_local:
            self.r.launch(self.a, self.b, None, self.d, self.m, self.n_local, self.k, alpha=1.0, beta=0.0, stream=self.stream)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        from runner.shard import max_over_ranks
        return max_over_ranks(self.dist, x, self.dev) if self.world > 1 else x

    def timed(self, steps: int, sampler=None):
        """`steps` steps between two events, barrier + synchronise on both sides; returns (ms per step as the max over
        ranks, clock record or None, main-kernel ns per launch on this rank, launches counted by the library)."""
        torch = self.torch
        self.barrier()
        self.r.set_option("profile", 1)
        self.r.info("sm_khz_effective")       # clears the device-side stopwatch
        launches0 = self.r.info("launches")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.start()
        self.barrier()
        e0.record()
        for _ in range(steps):
            self.step()
        e1.record()
        self.barrier()
        clocks = sampler.stop() if sampler else None
        ms = e0.elapsed_time(e1)
        launches = self.r.info("launches") - launches0
        count = self.r.info("profile_count")
        main_ns = self.r.info("profile_main_ns")
        self.r.set_option("profile", 0)
        # SM clock the GEMM kernels of this region really ran at: SM cycles / nanoseconds counted on the device
        self.last_device_mhz = self.r.info("sm_khz_effective") * 1e-3 or None
        return self.max_over_ranks(ms) / steps, clocks, (main_ns / count if count else None), launches

    def parity(self, columns: int):
        """Sampled columns of this rank's shard of D against the CPU oracle, max over ranks (outside any timed region)."""
        from oracle import oracle, shard_check
        oracle.use_all_cores()
        ratio, count = 0.0, 0
        if self.n_local:
            cols = shard_check.sample_columns(self.n0, self.n1, self.tile_n, columns, seed=17)
            import numpy as np
            idx = self.torch.from_numpy((cols - self.n0).astype(np.int64)).to(self.dev)
            sampled = self.d[: self.m * self.n_local].view(self.n_local, self.m).index_select(0, idx).cpu().numpy()
            ratio = shard_check.worst_ratio_of_columns(sampled, cols, self.m, self.k)
            count = len(cols)
            if not math.isfinite(ratio):
                ratio = float("inf")
        worst = self.max_over_ranks(ratio if math.isfinite(ratio) else 1e30)
        return {"worst_ratio": worst, "columns_per_rank": count, "ranks": self.world,
                "rule": "max |D - D_oracle| / (1e-5 * sum|a||b|) <= 1 (oracle = the reference's cpuGemm arithmetic)",
                "ok": bool(worst <= 1.0)}

    def free(self):
        self.r.set_workspace(None, 0)
        del self.a, self.b, self.d, self.ws
        self.torch.cuda.empty_cache()


def gather_list(dist, world, value):
    if world == 1:
        return [value]
    out = [None] * world
    dist.all_gather_object(out, value)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--kernel", default=None, help="registered kernel name (default: the tensor-core default)")
    ap.add_argument("--size", type=int, default=8192, help="M = N_per_gpu = K (profiling runs use a smaller case)")
    ap.add_argument("--workload", choices=["c3", "c5"], default="c3",
                    help="c3: M = K = N per GPU = --size, N grows with the GPU count (weak scaling, the default headline); "
                         "c5: make the fixed M = N = 32768, K = 8192 problem (strong scaling) the headline instead")
    ap.add_argument("--allgather", action="store_true",
                    help="also time the optional NCCL all-gather of D's column shards (reported apart from the GEMM)")
    ap.add_argument("--acc-chain", type=int, default=-1,
                    help="k per tensor-core accumulation chain: -1 = as the kernel was generated (128), 0 = all of K in "
                         "one chain (faster, drifts toward zero for same-signed inputs)")
    ap.add_argument("--sustained-seconds", type=float, default=3.0, help="length of the clock-sampled sustained loop (0: skip)")
    ap.add_argument("--c5-seconds", type=float, default=2.5, help="timed length of the 32768 x 32768 x 8192 record (0: skip)")
    ap.add_argument("--parity-columns", type=int, default=16, help="columns of D every rank checks against the oracle (0: skip)")
    ap.add_argument("--no-tf32-probe", dest="tf32_probe", action="store_false", help="skip the plain-TF32 probe of the tensor rate")
    ap.add_argument("--no-ffma", dest="ffma", action="store_false", help="skip the FFMA-path record of the same problem")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    global M, N_PER_GPU, K
    M = N_PER_GPU = K = args.size

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    importlib.import_module("amdgpu-arch-gemm_b200")
    from runner import api
    import kernels

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    kernel = args.kernel or kernels.DEFAULT_TENSOR
    cubin, toml = kernels.ensure(kernel)
    r = api.SgemmRunner(cubin, toml, local_rank)
    r.set_option("acc_chain", args.acc_chain)
    if world > 1:
        from runner.shard import make_communicator
        make_communicator(dist, r, rank, world)     # the library's own NCCL communicator: sharded host call, all-gather of D
    stream = torch.cuda.current_stream().cuda_stream
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        uuid = None
    sampler = ClockSampler(uuid, local_rank)
    peaks, peak_src = measured_peaks()
    sm_count = r.info("sm_count")

    def record_of(job, steps, with_clocks=True):
        ms_step, clocks, main_ns, launches = job.timed(steps, sampler if with_clocks else None)
        flops_all = 2.0 * job.m * job.n_total * job.k
        rec = {"value": flops_all / (ms_step * 1e-3) * 1e-12, "ms_per_step": ms_step, "steps": steps,
               "seconds": ms_step * steps * 1e-3, "launches": launches}
        rec["per_gpu_tflops"] = rec["value"] / world
        main_ms = gather_list(dist, world, main_ns * 1e-6 if main_ns else None)
        rec["main_kernel_ms_per_rank"] = main_ms
        all_clocks = gather_list(dist, world, clocks)
        rec["clocks"] = all_clocks[0]
        device_mhz = gather_list(dist, world, job.last_device_mhz)
        rec["sm_mhz_counted_on_device"] = device_mhz[0]
        if rec["clocks"] is not None:
            rec["clocks"]["sm_mhz_counted_on_device"] = device_mhz[0]
        if world > 1:
            rec["sm_mhz_median_per_rank"] = [c and c.get("sm_mhz") for c in all_clocks]
            rec["sm_mhz_counted_on_device_per_rank"] = device_mhz
        # cycles the main kernel took: its time x the clock it ran at (the device's own count when there is one)
        mhz = job.last_device_mhz or (clocks and clocks.get("valid") and clocks.get("sm_mhz"))
        if main_ns and mhz:
            rec["main_kernel_ms_x_sm_mhz"] = main_ns * 1e-6 * mhz
            rec["value_per_ghz"] = rec["per_gpu_tflops"] / (mhz * 1e-3)
        return rec, main_ns

    # ------------------------------------------------------------------ the headline: 8192 columns per GPU (weak)
    if args.workload == "c5":
        job = Job(torch, dist, r, dev, world, rank, C5_M, C5_N, C5_K, stream)
    else:
        job = Job(torch, dist, r, dev, world, rank, M, N_PER_GPU * world, K, stream)
    for _ in range(args.warmup):
        job.step()
    head, main_ns = record_of(job, args.steps)
    status = r.last_status()
    n_local = job.n_local

    # TF32 probe (outside every reported figure; taken right after the headline region, in the same thermal state): the
    # same pipeline issuing ONE plain-TF32 MMA per k-slice instead of the three of the split — the TF32 tensor rate this
    # code reaches on this box, measured with the bench's own harness next to the peak derived from the BF16 figure.
    # It is a yardstick, not a ceiling: plain TF32 needs three times the operand bytes per pipe clock (the split reuses
    # each staged tile in two MMAs), which puts its stage ring at the shared-memory bandwidth limit, so the 3xTF32
    # kernel keeps the pipe busier than a third of the probe would suggest.
    probe = None
    if args.tf32_probe and args.workload == "c3":
        try:
            pc, pt = kernels.ensure("tc2_256x256x32_s6_1x")
            pr = api.SgemmRunner(pc, pt, local_rank)
            pr.set_workspace(job.ws, job.ws.numel())
            for _ in range(3):
                pr.launch(job.a, job.b, None, job.d, job.m, n_local, job.k, alpha=1.0, beta=0.0, stream=stream)
            job.barrier()
            pr.set_option("profile", 1)
            pr.info("sm_khz_effective")
            for _ in range(max(args.steps, 10)):
                pr.launch(job.a, job.b, None, job.d, job.m, n_local, job.k, alpha=1.0, beta=0.0, stream=stream)
            torch.cuda.synchronize()
            cnt, ns = pr.info("profile_count"), pr.info("profile_main_ns")
            mhz = pr.info("sm_khz_effective") * 1e-3
            pr.close()
            rate = 2.0 * job.m * n_local * job.k / (ns / cnt * 1e-9) * 1e-12
            probe = {"kernel": "tc2_256x256x32_s6_1x (one kind::tf32 MMA per k-slice, same tile and CTA pairs)", "launches": cnt,
                     "tf32_tflops": rate, "third": rate / 3.0, "sm_mhz_counted_on_device": mhz or None,
                     "frac_of_pipe_at_kernel_clock": (rate / (TF32_FLOPS_PER_CLK_SM * sm_count * mhz * 1e6 * 1e-12)) if mhz else None,
                     "note": "plain TF32 stages 3x the operand bytes per pipe clock and is shared-memory bound: a third of "
                             "its rate is a yardstick for the 3xTF32 kernel, not a ceiling"}
            job.step()          # D holds the probe's plain-TF32 product: recompute it before anything reads it
            torch.cuda.synchronize()
        except Exception as exc:   # noqa: BLE001 - the probe is informational
            probe = {"error": str(exc)[:200]}

    # The FFMA path on the same problem (strict FP32: the other arm of the 8192^3 comparison), on the kernel
    # kernels.recommend names for it; outside every other figure.  Its roof is the FP32 FMA pipe, 128 lanes per SM and
    # clock, at the clock NVML samples during the launches.
    ffma = None
    if args.ffma and args.workload == "c3" and args.kernel is None and args.size == 8192:   # (the headline run only)
        try:
            fname = kernels.recommend(job.m, n_local, job.k, strict_fp32=True)
            fr = api.SgemmRunner(*kernels.ensure(fname), local_rank)
            fr.set_option("force_variant", 2)
            fr.set_workspace(job.ws, job.ws.numel())
            for _ in range(3):
                fr.launch(job.a, job.b, None, job.d, job.m, n_local, job.k, alpha=1.0, beta=0.0, stream=stream)
            job.barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            runs = 10
            sampler.start()
            f0.record()
            for _ in range(runs):
                fr.launch(job.a, job.b, None, job.d, job.m, n_local, job.k, alpha=1.0, beta=0.0, stream=stream)
            f1.record()
            torch.cuda.synchronize()
            fclk = sampler.stop()
            fms = f0.elapsed_time(f1) / runs
            frate = 2.0 * job.m * n_local * job.k / (fms * 1e-3) * 1e-12
            fmhz = fclk.get("sm_mhz") if fclk and fclk.get("valid") else None
            fpeak = sm_count * 128 * 2 * fmhz * 1e6 * 1e-12 if fmhz else None
            ffma = {"kernel": fname, "fed_by_tma": bool(fr.info("last_feed_tma")), "launches": runs, "ms_per_launch": fms,
                    "tflops": frate, "sm_mhz": fmhz, "fp32_peak_tflops_at_that_clock": fpeak,
                    "frac": frate / fpeak if fpeak else None, "device_status": fr.last_status()[0]}
            fr.close()
            job.step()          # D holds the FFMA product: recompute the tensor-path one before anything reads it
            torch.cuda.synchronize()
        except Exception as exc:   # noqa: BLE001 - informational
            ffma = {"error": str(exc)[:200]}

    # sustained: the same step for a few seconds, clock-sampled, so that the power-capped rate is on record
    sustained = None
    if args.sustained_seconds > 0:
        steps = max(args.steps, int(math.ceil(args.sustained_seconds * 1e3 / head["ms_per_step"])))
        sustained, sus_main_ns = record_of(job, steps)
        sustained["main_kernel_tflops"] = (2.0 * job.m * n_local * job.k) / (sus_main_ns * 1e-9) * 1e-12 if sus_main_ns else None
    parity = job.parity(args.parity_columns) if args.parity_columns > 0 else None

    # ---- optional: all-gather of the column shards of D over NVLink (NCCL, in place in a full-size D on every GPU:
    # sgemm_allgather_columns); never part of `value`
    allgather = None
    if args.allgather and world > 1:
        full_d = torch.empty(job.m * job.n_total, dtype=torch.float32, device=dev)
        mine = full_d[job.m * job.n0: job.m * job.n1]
        mine.copy_(job.d[: job.m * n_local])
        r.allgather_columns(full_d, job.m, job.n_total, stream=stream)      # warm-up (NCCL channel set-up)
        job.barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        r.allgather_columns(full_d, job.m, job.n_total, stream=stream)
        g1.record()
        job.barrier()
        ag_ms = job.max_over_ranks(g0.elapsed_time(g1))
        recv_bytes = (full_d.numel() - job.m * n_local) * 4
        # what arrived must be what the owners computed: this rank's neighbour's first column against the oracle
        check = None
        if args.parity_columns > 0:
            from oracle import shard_check
            other = (rank + 1) % world
            from runner.shard import shard_columns
            o0, o1 = shard_columns(job.n_total, world, other, job.tile_n)
            if o1 > o0:
                col = full_d[job.m * o0: job.m * (o0 + 1)].cpu().numpy()
                check = job.max_over_ranks(shard_check.worst_ratio_of_columns(col, [o0], job.m, job.k))
        allgather = {"ms": ag_ms, "bytes_received_per_gpu": recv_bytes, "gb_per_s_per_gpu": recv_bytes / ag_ms * 1e-6,
                     "full_d_elements": full_d.numel(), "path": "sgemm_allgather_columns (in place, ncclAllGather)",
                     "received_column_worst_ratio": check}
        del full_d, mine

    # ---- end to end through the host-buffer entry point (pinned host memory, copies inside the timed region)
    e2e = None
    if not args.no_e2e and args.workload == "c3":   # (the c5 problem would need 6 GiB of pinned host memory per rank)
        ha = torch.empty(M * K, dtype=torch.float32).pin_memory()
        hb = torch.empty(K * n_local, dtype=torch.float32).pin_memory()
        hd = torch.empty(M * n_local, dtype=torch.float32).pin_memory()
        ha.copy_(job.a)
        hb.copy_(job.b)
        r.set_workspace(None, 0)     # the host entry point sizes its own scratch (A's copies are shared by the chunks)
        e2e_steps = max(1, min(args.steps, 5))
        # one rank: the host-buffer call; several: its sharded form — every rank uploads 1/world of the replicated A
        # and its own columns of B, the ranks complete A over NVLink, every rank downloads its columns of D
        host_call = r.run_host_sharded if world > 1 else r.run_host
        host_call(ha, hb, None, hd, M, n_local, K, alpha=1.0, beta=0.0)   # warm-up: allocates the staging buffers
        job.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_call(ha, hb, None, hd, M, n_local, K, alpha=1.0, beta=0.0)   # synchronises before returning
        dt = job.max_over_ranks(time.perf_counter() - t0)
        # the result the host now holds must be the one the device path computed
        same = bool(torch.equal(hd, job.d.cpu()))
        same = bool(job.max_over_ranks(0.0 if same else 1.0) == 0.0)
        # what the host side of the box sustains: the bytes every rank moved over its link per second, their sum, and —
        # measured on rank 0 alone with all host cores while the GPUs are idle — a plain copy in host memory (read +
        # write bytes), the ceiling all ranks' transfers share when the GPUs hang off one NUMA node
        step_s = dt / e2e_steps
        link_rank = ((M * K // world + K * n_local) * 4 + M * n_local * 4) / step_s * 1e-9
        host_copy = None
        job.barrier()
        if rank == 0:
            cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
            before = torch.get_num_threads()
            torch.set_num_threads(cores)
            src = torch.ones(1 << 28, dtype=torch.float32)
            dst = torch.empty_like(src)
            dst.copy_(src)
            t1 = time.perf_counter()
            for _ in range(3):
                dst.copy_(src)
            host_copy = 3 * 2 * src.numel() * 4 / (time.perf_counter() - t1) * 1e-9
            torch.set_num_threads(before)
            del src, dst
        job.barrier()
        e2e = {"value": 2.0 * job.m * job.n_total * job.k / (dt / e2e_steps) * 1e-12, "unit": UNIT,
               "host_link_gb_per_s_per_rank": link_rank, "host_link_gb_per_s_all_ranks": link_rank * world,
               "host_memory_copy_gb_per_s": host_copy,
               "h2d_bytes_per_step": (M * K // world + K * n_local) * 4, "d2h_bytes_per_step": M * n_local * 4,
               "bytes_are": "per rank", "steps": e2e_steps, "host_result_equals_device_result": same,
               "path": ("sgemm_run_host_sharded (A uploaded in 1/N slices and completed by an all-gather over NVLink; "
                        if world > 1 else "sgemm_run_host (") + "pinned host buffers, column chunks pipelined over three streams)"}
        del ha, hb, hd
    head_shape = (job.m, n_local, job.k)
    head_total = job.n_total
    job.free()

    # ------------------------------------------------- strong scaling: 32768 x 32768 x 8192 sharded over the ranks
    c5 = None
    if args.c5_seconds > 0 and args.workload == "c3" and args.size == 8192:
        big = Job(torch, dist, r, dev, world, rank, C5_M, C5_N, C5_K, stream)
        for _ in range(3):
            big.step()
        est_ms, _, _, _ = big.timed(2)
        steps = max(3, int(math.ceil(args.c5_seconds * 1e3 / est_ms)))
        c5, _ = record_of(big, steps)
        c5["scaling"] = "strong"
        c5["workload"] = f"M={C5_M} N={C5_N} K={C5_K}, columns sharded over {world} GPU(s) ({big.n_local} on rank 0), A replicated"
        if args.parity_columns > 0:
            c5["parity"] = big.parity(args.parity_columns)
        big.free()
    status2 = r.last_status()
    failed = False

    if rank == 0:
        # roofline of the dominant kernel (generated_gemm): algorithmic flops of one launch / its mean duration.
        # Ceiling: the tensor pipe runs TF32 at half the BF16 rate and the split issues 3 MMAs per product, so
        # FP32-accurate flops top out at BF16 / 6.  A timed region shorter than a second never reaches the power cap:
        # the burst figure applies; a longer one is held to the sustained figure.
        timed_s = head["seconds"]
        key = "bf16_tflops" if timed_s < 1.0 else "bf16_tflops_sustained"
        peak = peaks.get(key, peaks["bf16_tflops"]) / 6.0
        achieved = (2.0 * head_shape[0] * head_shape[1] * head_shape[2]) / (main_ns * 1e-9) * 1e-12 if main_ns else None
        traffic, traffic_src = ncu_traffic(kernel, cubin, head_shape)
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": (achieved / peak) if achieved else None, "traffic": traffic, "traffic_source": traffic_src,
                    "kernel": "generated_gemm", "launches_timed": args.steps,
                    "peak_source": f"{peak_src} {key} / 6 (TF32 = 1/2 BF16 rate, 3 MMAs per product); timed region "
                                   f"{timed_s:.3f} s -> {'burst' if timed_s < 1.0 else 'sustained'} figure"}
        clk = head["clocks"]
        head_mhz = head.get("sm_mhz_counted_on_device") or (clk and clk.get("valid") and clk.get("sm_mhz"))
        if achieved and head_mhz:
            pipe = TF32_FLOPS_PER_CLK_SM * sm_count * head_mhz * 1e6 / 3.0 * 1e-12
            roofline["pipe_peak_at_kernel_clock"] = pipe
            roofline["frac_of_pipe_at_kernel_clock"] = achieved / pipe
            roofline["kernel_clock_mhz"] = head_mhz
        if probe and probe.get("third") and achieved:
            probe["frac_of_third"] = achieved / probe["third"]
        roofline["tf32_probe"] = probe
        if sustained and sustained.get("main_kernel_tflops"):
            sus_peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) / 6.0
            sustained["frac_of_sustained_peak"] = sustained["main_kernel_tflops"] / sus_peak
            sustained["peak"] = sus_peak
            sclk = sustained["clocks"]
            sus_mhz = sustained.get("sm_mhz_counted_on_device") or (sclk and sclk.get("valid") and sclk.get("sm_mhz"))
            if sus_mhz:
                pipe = TF32_FLOPS_PER_CLK_SM * sm_count * sus_mhz * 1e6 / 3.0 * 1e-12
                sustained["frac_of_pipe_at_kernel_clock"] = sustained["main_kernel_tflops"] / pipe
        line = {
            "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong" if args.workload == "c5" else "weak",
            "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"column-major NN SGEMM M={head_shape[0]} N={head_total} K={head_shape[2]} (N={head_shape[1]} on rank 0), alpha=1, beta=0, "
                                   "seeded uniform[-1,1); 3xTF32 tcgen05 path", "kernel": kernel,
                       "acc_chain": r.info("last_acc_chain"),
                       "parallelism": f"column-block shards x{world}, A replicated, no collective",
                       "l2": f"inputs (A + B = {(head_shape[0] * head_shape[2] + head_shape[2] * head_shape[1]) * 4 >> 20} MiB per GPU) exceed the 126 MB L2, no flush needed"},
            "roofline": roofline, "e2e": e2e, "gpu_launches": head["launches"], "clocks": head["clocks"],
            "main_kernel_ms_per_rank": head["main_kernel_ms_per_rank"],
            "sustained": sustained, "parity": parity, "c5": c5,
            "device_status": max(status[0], status2[0]), "allgather": allgather, "ffma_path": ffma,
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle
            tf, cols, dt, threads = cpu_reference_tflops(oracle)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{cols} of 8192 columns of the same problem, {dt:.1f} s of CPU work",
                                    "reference_loop_order_one_thread": cpu_reference_order(oracle)}
        print(json.dumps(line), flush=True)
        # a number next to a wrong result is worth nothing: the line is printed for the record, the run fails
        wrong = [name for name, bad in (("parity", parity is not None and not parity["ok"]),
                                        ("c5 parity", bool(c5 and c5.get("parity")) and not c5["parity"]["ok"]),
                                        ("e2e result differs from the device result", bool(e2e) and not e2e["host_result_equals_device_result"]),
                                        ("device status", max(status[0], status2[0]) != 0)) if bad]
        if wrong:
            print("bench.py: FAILED checks: " + ", ".join(wrong), file=sys.stderr, flush=True)
            failed = True
    r.close()
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit(3)


if __name__ == "__main__":
    main()
