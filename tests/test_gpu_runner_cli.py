"""The GeneratorRunner program: the reference's CLI `<code object> <toml> M N K warmup runs validate` and its
stdout shape (runner/generator_runner.cpp:193-323), parsed the way the reference's tuner parses it."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def run_cli(built, kernel, m, n, k, validate, env=None, warmup=2, runs=5):
    from runner import api
    api.build_library()
    cubin, toml = built.ensure(kernel)
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([str(api.RUNNER_PATH), cubin, toml, str(m), str(n), str(k), str(warmup), str(runs), str(validate)],
                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=e, timeout=600)


def test_cli_on_the_1024_cubed_configuration_as_worded(built):
    """`GeneratorRunner <cubin> <toml> 1024 1024 1024 10 100 1` with beta = 0 on the default cubin: 10 warm-up and 100
    timed runs, validated against the runner's CPU GEMM with the reference's own rule (|gpu - cpu| < 1e-3,
    runner/generator_runner.cpp:289-304) — no mismatch among the 1024 * 1024 elements."""
    ret = run_cli(built, built.DEFAULT_TENSOR, 1024, 1024, 1024, 1, env={"SGEMM_BETA": "0"}, warmup=10, runs=100)
    assert ret.returncode == 0, ret.stdout + ret.stderr
    lines = ret.stdout.strip().split("\n")
    assert lines[-1] == "# of mismatches: 0/1048576"
    assert float(lines[-3].split(":")[-1]) > 0 and "tcgen05 3xTF32" in ret.stderr


@pytest.mark.parametrize("kernel", ["tc_128x256x32_s2", "simt_128x128x16", "ffma_tma_256x128x16_s4"])
def test_cli_stdout_contract_and_validation(built, kernel):
    ret = run_cli(built, kernel, 512, 768, 640, 1)
    assert ret.returncode == 0, ret.stdout + ret.stderr
    lines = ret.stdout.split("\n")
    assert lines[0].startswith("cpuGemm func: ") and lines[0].endswith(" ms")
    assert lines[1].startswith("SIMT gemm: ") and lines[2].startswith("Gflops: ") and lines[3].startswith("GiB/s: ")
    assert lines[4].startswith("ASM gemm: ") and lines[5].startswith("Gflops: ") and lines[6].startswith("GiB/s: ")
    assert lines[7] == f"# of mismatches: 0/{512 * 768}"
    import json, tempfile
    with tempfile.TemporaryDirectory() as tmp:
        ret = run_cli(built, kernel, 512, 768, 640, 0, env={"SGEMM_JSON": f"{tmp}/r.json", "SGEMM_BETA": "0", "SGEMM_SEED": "7"})
        rec = json.load(open(f"{tmp}/r.json"))
    assert (rec["m"], rec["n"], rec["k"], rec["beta"], rec["seed"], rec["validated"]) == (512, 768, 640, 0, 7, False)
    want = {"tc": "tcgen05_3xtf32", "si": "simt_ffma", "ff": "simt_ffma_tma"}[kernel[:2]]   # (a small problem runs on the tensor cubin's companion)
    assert rec["tflops"] > 0 and (rec["variant"].startswith(want) if kernel.startswith("tc") else rec["variant"] == want)
    assert ret.returncode == 0
    gflops = float(ret.stdout.split("\n")[-3].split(":")[-1])   # tuner/sgemm_tuner.py:115
    assert gflops > 0
    assert ("tcgen05" in ret.stderr) == kernel.startswith("tc_")


def test_cli_argument_and_file_errors(built):
    from runner import api
    api.build_library()
    cubin, toml = built.ensure("simt_128x128x16")
    short = subprocess.run([str(api.RUNNER_PATH), cubin, toml, "64", "64"], capture_output=True, text=True)
    assert short.returncode == 255      # the reference returns -1 for argc <= 8
    bad = subprocess.run([str(api.RUNNER_PATH), cubin + ".missing", toml, "64", "64", "64", "1", "1", "0"],
                         capture_output=True, text=True)
    assert bad.returncode not in (0, 255) and "sgemm_open" in bad.stderr


@pytest.mark.parametrize("kernel", ["fp16_tc_128x128x64_s4", "bf16_tc2_256x256x64_s6"])
def test_cli_drives_cubins_for_sixteen_bit_operands(built, kernel):
    """FP32 draws converted on the device, CPU check on the converted values, an empty SIMT block (there is no FFMA
    kernel for 16-bit operands) so that the tuner's parse of the third line from the end still works."""
    ret = run_cli(built, kernel, 512, 768, 640, 1)
    assert ret.returncode == 0, ret.stdout + ret.stderr
    lines = ret.stdout.split("\n")
    assert lines[1] == "SIMT gemm: 0 ms" and lines[4].startswith("ASM gemm: ")
    assert lines[7] == f"# of mismatches: 0/{512 * 768}"
    assert float(lines[-3].split(":")[-1]) > 0            # tuner/sgemm_tuner.py:115
    assert ("BF16" if kernel.startswith("bf16") else "FP16") in ret.stderr
    cubin, toml = built.ensure("bf16_tc2_256x256x64_s6_tt")   # transposed layouts are not what this program drives
    from runner import api
    bad = subprocess.run([str(api.RUNNER_PATH), cubin, toml, "64", "64", "64", "1", "1", "0"], capture_output=True, text=True)
    assert bad.returncode == 2 and "NN layout" in bad.stderr


@pytest.mark.parametrize("ngpus", [1, 2, 8])
def test_cli_shards_over_gpus_and_gathers(built, ngpus, tmp_path):
    """SGEMM_NGPUS / SGEMM_ALLGATHER: the same positional CLI and stdout, the problem column-sharded over the GPUs of
    the box in one process, D all-gathered in place over NVLink and validated on the last GPU's copy.  (One GPU: a
    communicator of one rank — the code path is the same.)"""
    import json
    from runner import api
    if api.device_count() < ngpus:
        pytest.skip(f"needs {ngpus} GPUs")
    out = tmp_path / "r.json"
    env = {"SGEMM_NGPUS": str(ngpus), "SGEMM_ALLGATHER": "1", "SGEMM_BETA": "0", "SGEMM_JSON": str(out)}
    ret = run_cli(built, built.DEFAULT_TENSOR, 1024, 2048 + 96, 1024, 1, env=env)
    assert ret.returncode == 0, ret.stdout + ret.stderr
    lines = ret.stdout.strip().split("\n")
    assert lines[-1] == f"# of mismatches: 0/{1024 * (2048 + 96)}" and lines[-4].startswith("ASM gemm: ")
    rec = json.load(open(out))
    assert rec["ngpus"] == ngpus and len(rec["per_gpu"]) == ngpus and rec["mismatches"] == 0
    assert rec["per_gpu"][0]["n0"] == 0 and rec["per_gpu"][-1]["n1"] == 2048 + 96
    assert all(a["n1"] == b["n0"] for a, b in zip(rec["per_gpu"], rec["per_gpu"][1:]))
    assert "all-gather of D" in ret.stderr and rec["allgather_ms"] > 0
    if ngpus > 1:
        assert f"{ngpus} GPUs, columns sharded" in ret.stderr
