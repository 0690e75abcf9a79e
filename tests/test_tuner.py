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
    best = t.tune(512, 512, 512, runner, str(out), include_simt=False, exhaustive=True)
    assert best["gflops"] == 103 and best["stages"] == 3 and best["tile"] == [256, 256]
    log = [json.loads(l) for l in (out / "tuner_results.jsonl").read_text().splitlines()]
    assert [r["stages"] for r in log] == [2, 3]
    text = capsys.readouterr().out
    assert "Best: 103.0 Gflops" in text and "MT: (256, 256)" in text
    # resume: nothing is measured again (a runner that fails would be noticed)
    failing = fake_runner(tmp_path, "exit 3\n")
    again = t.tune(512, 512, 512, failing, str(out), include_simt=False, exhaustive=True)
    assert again["gflops"] == 103
    assert len((out / "tuner_results.jsonl").read_text().splitlines()) == 2
    # the staged search (the default) reuses the log as well: every point it asks for was measured with 50 runs
    staged = t.tune(512, 512, 512, failing, str(out), include_simt=False)
    assert staged["gflops"] == 103 and len((out / "tuner_results.jsonl").read_text().splitlines()) == 2
    assert "staged search" in capsys.readouterr().out


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


# ------------------------------------------------------------------ the staged search replayed on recorded sweeps
def recorded_points(path):
    """(records, points) of a result file of an exhaustive sweep on a B200: the points are rebuilt from the records
    (structure -> configuration, recorded rasterisation widths / prefetch depths -> variations, default one first)."""
    from generator.generator import DataType, GemmSolutionConfig, GemmOptimizations
    F = DataType.FP32
    recs = [json.loads(l) for l in open(path)]
    recs = [r for r in recs if not r.get("returncode")]
    def canonical(key):     # the tuner's key order: structure (prefetch depth included), then the rasterisation width
        words = key.split(" ", 1)[1].split()
        return " ".join([w for w in words if not w.startswith("wgm")] + [w for w in words if w.startswith("wgm")])
    by_key = {canonical(r["key"]): r for r in recs}
    groups = {}
    for r in recs:
        words = r["key"].split(" ", 1)[1].split()
        knobs = [w for w in words if w.startswith("wgm")]
        structure = " ".join(w for w in words if w not in knobs)
        groups.setdefault(structure, []).append((" " + " ".join(knobs), r))
    points = []
    for structure, members in groups.items():
        r = members[0][1]
        if r["variant"] == "simt_ffma":
            wg = tuple(r["cluster"])
            wt = (r["tile"][0] // wg[0], r["tile"][1] // wg[1])
            config = GemmSolutionConfig(F, F, F, F, (1, 1, 1, 1), wg, wt, r["depth_k"], False, False)
        else:
            config = GemmSolutionConfig(F, F, F, F, (128, r["tile"][1], 1, 8), tuple(r["cluster"]), (1, 1), r["depth_k"], False, False,
                                        vmem_stage=r["stages"] - 1, split=r.get("split") or "prepass")
        default = lambda item: 0 if item[1]["wgm"] == 8 else 1
        variations = [(suffix, (lambda rec=rec: GemmOptimizations(1, wgm=rec["wgm"], plr=rec["plr"]))) for suffix, rec in sorted(members, key=default)]
        points.append((structure, config, variations))
    return recs, by_key, points


@pytest.mark.parametrize("name,m,n,k,shortlist", [("tuner_sweep_8192cubed_tensor", 8192, 8192, 8192, 12),
                                                 ("tuner_sweep_1024cubed_tensor", 1024, 1024, 1024, 14),
                                                 ("tuner_sweep_4096cubed_simt", 4096, 4096, 4096, 10)])
def test_staged_search_finds_the_recorded_best_with_a_quarter_of_the_measurements(golden_dir, name, m, n, k, shortlist, capsys):
    """Replay on sweeps recorded on a B200 (every point of a sub-space measured): the staged search — analytic ranking,
    successive halving, then the rasterisation width on the two best — must end within 1 % of the best
    recorded throughput while asking for at most a quarter of the measurements the exhaustive product made."""
    recs, by_key, points = recorded_points(golden_dir / f"{name}.jsonl")
    asked = []

    def measure(key, config, opt, runs):
        asked.append(key)
        return by_key[key]

    best, calls = t.staged_search(points, measure, m, n, k, shortlist=shortlist)
    top = max(r["gflops"] for r in recs)
    assert calls == len(asked) and calls <= 0.25 * len(recs), (calls, len(recs))
    assert best["gflops"] >= 0.99 * top, (best["key"], best["gflops"], top)


def test_analytic_ranking_orders_the_known_cases():
    """What the sweeps showed, as inequalities the ranking must respect at 8192^3: CTA pairs on 256-column tiles
    before single CTAs, 128-column tiles last; more k in flight before less; and a last wave that is nearly empty
    costs what it wastes."""
    from generator.generator import tensor_config
    e = lambda cfg, shape=(8192, 8192, 8192): t.predict_efficiency(cfg, *shape)
    assert e(tensor_config(256, 32, 3, cluster=2)) > e(tensor_config(256, 32, 2)) > e(tensor_config(128, 32, 3))
    assert e(tensor_config(256, 32, 3, cluster=2)) > e(tensor_config(256, 32, 3, cluster=2, split="inkernel"))
    assert e(tensor_config(256, 16, 6, cluster=2)) > e(tensor_config(256, 16, 2, cluster=2))
    full, ragged = (2048, 9472, 4096), (2048, 9728, 4096)       # 8 x 37 = 296 tiles = 4 waves of 74 pairs; 8 x 38 = 304: 5 waves
    assert e(tensor_config(256, 32, 3, cluster=2), full) > 1.15 * e(tensor_config(256, 32, 3, cluster=2), ragged)


def test_summarise_writes_the_table_recommend_reads(golden_dir, tmp_path):
    table = t.summarise([golden_dir / "tuner_sweep_8192cubed_tensor.jsonl", golden_dir / "tuner_sweep_4096cubed_simt.jsonl"],
                        str(tmp_path / "tuned.json"))
    entries = {(e["m"], e["variant"]): e for e in table["entries"]}
    assert entries[(8192, "tcgen05_3xtf32")]["tile"] == [256, 256] and entries[(8192, "tcgen05_3xtf32")]["cluster"] == [2, 1]
    assert entries[(4096, "simt_ffma")]["tile"] == [128, 128]
    assert json.loads((tmp_path / "tuned.json").read_text()) == table


def test_tma_fed_ffma_structures_are_searched_and_recorded(tmp_path):
    """The FFMA space has a feed dimension; records and the table say which feed a measurement was of, and an existing
    table keeps its entries unless a result file holds a faster one for the same slot."""
    keys = [k for k, _, _ in t.structural_candidates(True, False)]
    tma = [k for k in keys if k.startswith("simt tma ")]
    assert len(tma) == len(t.SUPPORTED_SIMT_TMA) and len(set(keys)) == len(keys)
    for key, make_config, variations in t.structural_candidates(True, False):
        if key.startswith("simt tma "):
            cfg = make_config()
            assert cfg.feed == "tma" and cfg.num_workitems % 128 == 0 and len(variations) == len(t.SUPPORTED_WGM)
            assert t.predict_time_us(cfg, 8192, 8192, 8192) > 0
    fed = {"key": "8192x8192x8192 simt tma g16x16 t16x8 k32 s3 wgm4", "returncode": 0, "tile": [256, 128], "depth_k": 32,
           "stages": 3, "cluster": [16, 16], "variant": "simt_ffma", "wgm": 4, "plr": 1, "split": "prepass", "feed": "tma",
           "runs": 50, "gflops": 60825.0}
    slow = dict(fed, key="8192x8192x8192 simt g16x16 t8x8 k16 wgm8 plr1", tile=[128, 128], depth_k=16, stages=2, feed="ldg", gflops=54000.0)
    assert t.describe(fed) == "simt_ffma tma-fed" and t.describe(slow) == "simt_ffma ldg-fed"
    log = tmp_path / "a.jsonl"
    log.write_text(json.dumps(slow) + "\n")
    table = t.summarise([log], str(tmp_path / "tuned.json"))
    assert [e["feed"] for e in table["entries"]] == ["ldg"]
    log2 = tmp_path / "b.jsonl"
    log2.write_text(json.dumps(fed) + "\n" + json.dumps(dict(fed, key="1024x1024x1024 simt tma g16x16 t16x8 k32 s3 wgm4", gflops=20000.0)) + "\n")
    table = t.summarise([log2], str(tmp_path / "tuned.json"))          # merged into the table written above
    got = {(e["m"], e["feed"]): e["gflops"] for e in table["entries"]}
    assert got == {(8192, "tma"): 60825.0, (1024, "tma"): 20000.0}
    table = t.summarise([log], str(tmp_path / "tuned.json"))           # a slower measurement does not displace the entry
    assert {(e["m"], e["feed"]) for e in table["entries"]} == {(8192, "tma"), (1024, "tma")}
