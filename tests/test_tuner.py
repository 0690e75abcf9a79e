"""Tuner host logic with a fake runner program: search, skip of infeasible points, stdout parsing as the
reference does it (tuner/sgemm_tuner.py:112-126), JSONL resume."""
import json
import os
import stat

import pytest

from tuner import sgemm_tuner as t


def fake_runner(tmp_path, body):
    p = tmp_path / "fake_runner.sh"
    p.write_text("#!/bin/sh\n" + body)
    p.chmod(p.stat().st_mode | stat.S_IEXEC)
    return str(p)


def test_candidates_cover_both_variants_and_skip_infeasible():
    keys = [k for k, _, _ in t.candidates()]
    assert len(keys) == len(set(keys)) and any(k.startswith("tensor") for k in keys) and any(k.startswith("simt") for k in keys)
    feasible = 0
    for _, make_config, _ in t.candidates():
        try:
            make_config()
            feasible += 1
        except RuntimeError:
            pass
    assert 0 < feasible < len(keys)   # e.g. 256x256x64 with 7 stages does not fit shared memory


def test_parse_gflops_reads_the_measured_block():
    out = "SIMT gemm: 1 ms\nGflops: 10\nGiB/s: 1\nASM gemm: 0.5 ms\nGflops: 123.5\nGiB/s: 2\n"
    assert t.parse_gflops(out) == 123.5


def test_tune_picks_best_and_resumes(tmp_path, monkeypatch, capsys):
    # the fake runner reports a throughput that depends on the TOML it is given (stages), like a real sweep would
    runner = fake_runner(tmp_path, 'S=$(grep "^stages" "$2" | tr -dc 0-9)\n'
                                   'echo "SIMT gemm: 1 ms"; echo "Gflops: 1"; echo "GiB/s: 1"\n'
                                   'echo "ASM gemm: 1 ms"; echo "Gflops: $((100 + S))"; echo "GiB/s: 1"\n')
    monkeypatch.setattr(t, "SUPPORTED_CLUSTERS", [(2, 1)])
    monkeypatch.setattr(t, "SUPPORTED_TILE_N", [256])
    monkeypatch.setattr(t, "SUPPORTED_DEPTH_K", [32])
    monkeypatch.setattr(t, "SUPPORTED_STAGES", [2, 3, 4])     # 4 stages of 64 KiB do not fit: skipped by RuntimeError
    monkeypatch.setattr(t, "SUPPORTED_WGM", [4])
    monkeypatch.setattr(t, "SUPPORTED_SPLIT", ["prepass"])
    out = tmp_path / "out"
    best = t.tune(512, 512, 512, runner, str(out), include_simt=False)
    assert best["gflops"] == 103 and best["stages"] == 3 and best["tile"] == [256, 256]
    log = [json.loads(l) for l in (out / "tuner_results.jsonl").read_text().splitlines()]
    assert [r["stages"] for r in log] == [2, 3]
    text = capsys.readouterr().out
    assert "Best: 103.0 Gflops" in text and "MT: (256, 256)" in text
    # resume: nothing is measured again (a runner that fails would be noticed)
    failing = fake_runner(tmp_path, "exit 3\n")
    again = t.tune(512, 512, 512, failing, str(out), include_simt=False)
    assert again["gflops"] == 103
    assert len((out / "tuner_results.jsonl").read_text().splitlines()) == 2


def test_runner_failure_is_recorded_not_fatal(tmp_path, monkeypatch, capsys):
    monkeypatch.setattr(t, "SUPPORTED_CLUSTERS", [(1, 1)])
    monkeypatch.setattr(t, "SUPPORTED_TILE_N", [128])
    monkeypatch.setattr(t, "SUPPORTED_DEPTH_K", [32])
    monkeypatch.setattr(t, "SUPPORTED_STAGES", [3])
    monkeypatch.setattr(t, "SUPPORTED_WGM", [1])
    monkeypatch.setattr(t, "SUPPORTED_SPLIT", ["inkernel"])
    best = t.tune(256, 256, 256, fake_runner(tmp_path, "echo boom >&2; exit 2\n"), str(tmp_path / "o"), include_simt=False)
    assert best is None
    assert "No valid configurations found." in capsys.readouterr().out
    # ragged problems are filtered like the reference does (tuner/sgemm_tuner.py:97) unless asked otherwise
    assert t.tune(250, 256, 256, "/bin/false", str(tmp_path / "o2"), include_simt=False) is None
    assert not (tmp_path / "o2" / "tuner_results.jsonl").exists()


def test_sixteen_bit_search_space():
    from generator.generator import DataType
    keys, built = [], 0
    for key, make_config, _ in t.candidates(ab_type=DataType.BF16):
        keys.append(key)
        try:
            cfg = make_config()
        except RuntimeError:
            continue                     # infeasible points are the tuner's skips
        built += 1
        assert cfg.a_type == DataType.BF16 and cfg.mfma[3] == 16 and cfg.terms == 1
    assert built > 20 and all(k.startswith("tensor bf16 ") for k in keys) and len(set(keys)) == len(keys)
