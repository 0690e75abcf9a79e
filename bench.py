#!/usr/bin/env python
"""SGEMM benchmark: FP32-accurate TFLOPS of the column-major NN SGEMM at M = N = K = 8192 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--kernel NAME]

One process per GPU (N > 1: launched by torch.distributed.run, one rank per GPU).  A "step" is one SGEMM
D = A*B (alpha = 1, beta = 0) through the C ABI of libsgemm_runner.so; with N ranks the problem is
M = K = 8192, N_total = 8192 * N, column-block sharded: A replicated, B and D column-partitioned, no collective
on the compute path (weak scaling: fixed work per GPU).  Inputs are seeded uniform[-1, 1) FP32 filled on the
device by global element index, so every N sees the same matrices.

Timed region: K steps between CUDA events on the launching stream, bracketed by barrier + synchronise, max over
ranks.  `value` counts algorithmic flops 2*M*N*K only (the 3x tensor work of the split is not counted) and
includes the split pre-pass that is part of every call.  `e2e` repeats the measurement through
sgemm_run_host with pinned HOST buffers (upload A and B, download D inside the timed region).

--impl reference times the reference's CPU GEMM (restated in oracle/, its native runner needs HIP and cannot be
built here) on all host cores, on a column block of the same 8192^3 problem.
"""
from __future__ import annotations

import argparse
import importlib
import json
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

# DRAM bytes one launch of the dominant kernel moved in an ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum), keyed by kernel name, for the 8192^3 workload.
# Source: profiles/bench_default_8192cubed_launches_and_dram.md (three launches, identical to three digits).
NCU_TRAFFIC_BYTES = {"tc2_256x256x32_s3": 4.83e9}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.t = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.t = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
        self.t.start()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--kernel", default=None, help="registered kernel name (default: the tensor-core default)")
    ap.add_argument("--size", type=int, default=8192, help="M = N_per_gpu = K (profiling runs use a smaller case)")
    ap.add_argument("--workload", choices=["c3", "c5"], default="c3",
                    help="c3: M = K = N per GPU = --size, N grows with the GPU count (weak scaling, the default); "
                         "c5: the fixed M = N = 32768, K = 8192 problem column-sharded over the GPUs (strong scaling)")
    ap.add_argument("--allgather", action="store_true",
                    help="also time the optional NCCL all-gather of D's column shards (reported apart from the GEMM)")
    ap.add_argument("--acc-chain", type=int, default=-1,
                    help="k per tensor-core accumulation chain: -1 = as the kernel was generated (128), 0 = all of K in "
                         "one chain (faster, drifts toward zero for same-signed inputs)")
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
    from runner.shard import max_over_ranks, shard_columns
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
    tile_n = r.info("tile_n")

    # c3, weak scaling: N_total = N_PER_GPU * world columns; c5, strong scaling: one fixed problem.
    # Either way this rank owns the columns [n0, n1).
    if args.workload == "c5":
        M, K = 32768, 8192
        n_total = 32768
    else:
        n_total = N_PER_GPU * world
    n0, n1 = shard_columns(n_total, world, rank, tile_n)
    n_local = n1 - n0
    a = torch.empty(M * K, dtype=torch.float32, device=dev)
    b = torch.empty(K * n_local, dtype=torch.float32, device=dev)
    d = torch.zeros(M * n_local, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    r.fill_uniform(a, M * K, stream_id=0, stream=stream)                              # A replicated
    r.fill_uniform(b, K * n_local, stream_id=1, first_index=n0 * K, stream=stream)    # B[:, n0:n1]
    ws_bytes = r.workspace_bytes(M, n_local, K)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    r.set_workspace(ws, ws_bytes)
    torch.cuda.synchronize()

    def step():
        r.launch(a, b, None, d, M, n_local, K, alpha=1.0, beta=0.0, stream=stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    r.set_option("profile", 1)
    launches0 = r.info("launches")
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    launches = r.info("launches") - launches0
    main_count = r.info("profile_count")
    main_ns = r.info("profile_main_ns")
    r.set_option("profile", 0)
    status = r.last_status()
    ms_total = max_over_ranks(dist, ms_total, dev) if world > 1 else ms_total
    ms_step = ms_total / args.steps
    flops_step_all = 2.0 * M * n_total * K
    value = flops_step_all / (ms_step * 1e-3) * 1e-12

    # ---- optional: all-gather of the column shards of D over NVLink (NCCL); never part of `value`
    allgather = None
    if args.allgather and world > 1:
        from runner.shard import gather_columns
        gather_columns(dist, d, M, n_total, world, tile_n)      # warm-up (NCCL channel set-up)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        full_d = gather_columns(dist, d, M, n_total, world, tile_n)
        g1.record()
        barrier()
        ag_ms = max_over_ranks(dist, g0.elapsed_time(g1), dev)
        recv_bytes = (full_d.numel() - d.numel()) * 4
        allgather = {"ms": ag_ms, "bytes_received_per_gpu": recv_bytes, "gb_per_s_per_gpu": recv_bytes / ag_ms * 1e-6,
                     "full_d_elements": full_d.numel()}
        del full_d

    # ---- end to end through the host-buffer entry point (pinned host memory, copies inside the timed region)
    e2e = None
    if not args.no_e2e and args.workload == "c3":   # (the c5 problem would need 6 GiB of pinned host memory per rank)
        ha = torch.empty(M * K, dtype=torch.float32).pin_memory()
        hb = torch.empty(K * n_local, dtype=torch.float32).pin_memory()
        hd = torch.empty(M * n_local, dtype=torch.float32).pin_memory()
        ha.copy_(a)
        hb.copy_(b)
        e2e_steps = max(1, min(args.steps, 5))
        r.run_host(ha, hb, None, hd, M, n_local, K, alpha=1.0, beta=0.0)   # warm-up: allocates the staging buffers
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            r.run_host(ha, hb, None, hd, M, n_local, K, alpha=1.0, beta=0.0)   # synchronises before returning
        dt = time.perf_counter() - t0
        dt = max_over_ranks(dist, dt, dev) if world > 1 else dt
        # the result the host now holds must be the one the device path computed
        same = bool(torch.equal(hd, d.cpu()))
        e2e = {"value": flops_step_all / (dt / e2e_steps) * 1e-12, "unit": UNIT,
               "h2d_bytes_per_step": (M * K + K * n_local) * 4, "d2h_bytes_per_step": M * n_local * 4,
               "steps": e2e_steps, "host_result_equals_device_result": same}

    if rank == 0:
        peaks, peak_src = measured_peaks()
        # roofline of the dominant kernel (generated_gemm): algorithmic flops of one launch / its mean duration.
        # Peak: the tensor pipe runs TF32 at half the BF16 rate and the split issues 3 MMAs per product, so the
        # ceiling for FP32-accurate flops is BF16 / 6 (sustained figure: the kernel is timed inside a long step).
        peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) / 6.0
        achieved = (2.0 * M * n_local * K) / (main_ns / max(main_count, 1) * 1e-9) * 1e-12 if main_ns else None
        traffic = NCU_TRAFFIC_BYTES.get(kernel) if (M, n_local, K) == (8192, 8192, 8192) else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if args.workload == "c5" else "weak",
            "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"column-major NN SGEMM M={M} N={n_total} K={K} (N={n_local} on rank 0), alpha=1, beta=0, "
                                   "seeded uniform[-1,1); 3xTF32 tcgen05 path", "kernel": kernel,
                       "acc_chain": r.info("last_acc_chain"),
                       "parallelism": f"column-block shards x{world}, A replicated, no collective",
                       "l2": f"inputs (A + B = {(M * K + K * n_local) * 4 >> 20} MiB per GPU) exceed the 126 MB L2, no flush needed"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None, "traffic": traffic,
                         "kernel": "generated_gemm", "launches_timed": main_count,
                         "peak_source": f"{peak_src} bf16_tflops_sustained / 6 (TF32 = 1/2 BF16 rate, 3 MMAs per product)"},
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "device_status": status[0], "allgather": allgather,
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle
            tf, cols, dt, threads = cpu_reference_tflops(oracle)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{cols} of 8192 columns of the same problem, {dt:.1f} s of CPU work"}
        print(json.dumps(line), flush=True)
    r.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
