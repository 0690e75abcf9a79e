"""Host-side behaviour of libsgemm_runner.so that needs no GPU: the library loads, exports every symbol the
header declares, reads the generator's TOML, and refuses to compute without a CUDA device."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def header_symbols():
    text = (ROOT / "include" / "sgemm_runner.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sgemm_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built):
    from runner import api
    L = api.lib()
    names = header_symbols()
    assert len(names) >= 20 and set(names) == set(api.ABI)
    for n in names:
        assert getattr(L, n) is not None


def test_strerror_is_total(built):
    from runner import api
    L = api.lib()
    assert L.sgemm_strerror(0) == b"ok"
    for code in range(-10, 0):
        assert L.sgemm_strerror(code) not in (b"", b"unknown error")
    assert L.sgemm_strerror(-99) == b"unknown error"


def test_toml_reader_reads_generator_output(built):
    from runner import api
    for name in built.REGISTRY:
        _, toml = built.ensure(name)
        cfg = api.parse_config(toml)
        factory, _ = built.REGISTRY[name]
        py = factory()
        assert api.config_tile(cfg) == py.tile_size
        assert cfg.depth_k == py.depth_k and cfg.num_threads == py.num_workitems
        assert cfg.lds_usage_bytes == py.lds_usage_bytes and cfg.vmem_stage == py.vmem_stage
        assert cfg.variant == (1 if py.variant == "tcgen05_3xtf32" else 0)
        assert cfg.entry == b"generated_gemm"


def test_toml_reader_accepts_the_reference_files_shape(built, tmp_path):
    from runner import api
    # what the reference's compile() writes for its default config (multi-line arrays, trailing commas)
    p = tmp_path / "ref.toml"
    p.write_text('a_type = 0\nb_type = 0\ncd_type = 0\nscalar_type = 0\nwave_group = [\n    2,\n    2,\n]\n'
                 'trans_a = false\ntrans_b = false\nmfma = [\n    32,\n    32,\n    1,\n    2,\n]\n'
                 'wave_tiling = [ 4, 2 ]  # inline too\ndepth_k = 16\nvmem_stage = 1\nwavefront_size = 64\n'
                 'lds_usage_bytes = 53_248\nname = ""\nunknown_key = "ignored"\n')
    cfg = api.parse_config(str(p))
    assert api.config_tile(cfg) == (256, 128) and cfg.num_threads == 256 and cfg.lds_usage_bytes == 53248
    assert cfg.variant == 0 and cfg.stages == 2


@pytest.mark.parametrize("text", ['a_type = 0\n', 'a_type = "x"\n', 'mfma = [1, 2\n', 'depth_k = 1.5\n', 'key value\n'])
def test_toml_reader_reports_bad_files(built, tmp_path, text):
    from runner import api
    p = tmp_path / "bad.toml"
    p.write_text(text)
    with pytest.raises(api.SgemmError) as e:
        api.parse_config(str(p))
    assert e.value.code == -2
    with pytest.raises(api.SgemmError):
        api.parse_config(str(tmp_path / "missing.toml"))


def test_open_fails_loudly_without_cubin_or_device(built, tmp_path):
    from runner import api
    _, toml = built.ensure(built.DEFAULT_SIMT)
    with pytest.raises(api.SgemmError) as e:
        api.SgemmRunner(str(tmp_path / "nope.cubin"), toml, 0)
    assert e.value.code == -5
    if api.device_count() == 0:  # no GPU here: the compute path must refuse, never fall back
        cubin, _ = built.ensure(built.DEFAULT_SIMT)
        with pytest.raises(api.SgemmError) as e:
            api.SgemmRunner(cubin, toml, 0)
        assert e.value.code in (-3, -1, -4)


def test_shard_columns_cover_n_in_whole_tiles():
    from runner.shard import all_shards, shard_columns
    for n, world, tile in [(32768, 8, 256), (8192, 3, 256), (1000, 4, 128), (100, 8, 64), (0, 2, 16)]:
        sh = all_shards(n, world, tile)
        assert sh[0][0] == 0 and sh[-1][1] == n
        for (a0, a1), (b0, b1) in zip(sh, sh[1:]):
            assert a1 == b0 and a0 <= a1
        for n0, n1 in sh:
            assert n0 == n1 or (n0 % tile == 0 and (n1 % tile == 0 or n1 == n))  # non-empty shards: whole tiles
        widths = [b - a for a, b in sh]
        assert max(widths) - min(w for w in widths) <= tile or n < world * tile
    with pytest.raises(ValueError):
        shard_columns(10, 2, 2)


def test_kernel_recommendation_names_registered_kernels(built):
    cases = {(8192, 8192, 8192): "tc2_256x256x32_s3", (32, 32, 32): "simt_128x128x16", (4096, 128, 16384): "tc2_256x256x32_s3",
             (256, 8192, 16384): "tc2i_256x256x32_s3", (1024, 1024, 1024): "tc2_256x256x32_s3", (1024, 1024, 16384): "tc_128x128x32_s3",
             (32768, 4096, 8192): "tc2_256x256x32_s3"}
    for shape, want in cases.items():
        got = built.recommend(*shape)
        assert got in built.REGISTRY and got == want, (shape, got)
    for shape in [(1024, 1024, 1024), (300, 5000, 700), (1, 1, 1), (65536, 64, 64)]:
        assert built.recommend(*shape) in built.REGISTRY
    # strict FP32: the FFMA variant; the TMA-fed kernel where the tuner measured it fastest or the problem has many tiles
    strict = {(8192, 8192, 8192): "ffma_tma_256x128x32_s3", (32768, 32768, 8192): "ffma_tma_256x128x32_s3",
              (4096, 4096, 4096): "simt_128x128x16_t16x8", (100, 100, 100): "simt_128x128x16"}
    for shape, want in strict.items():
        assert built.recommend(*shape, strict_fp32=True) == want, shape
    with pytest.raises(ValueError):
        built.recommend(8192, 8192, 8192, operands="bf16", strict_fp32=True)


def test_shard_rule_of_the_library_equals_the_python_restatement(built):
    """sgemm_shard_columns (C ABI, used by the runner program) and runner.shard.shard_columns (used by the benchmark)
    must cut the same shards: whole tiles, as even as possible, ragged tail in the last non-empty shard."""
    from runner import api
    from runner.shard import shard_columns
    for n in (0, 1, 255, 256, 4100, 8192, 32768, 70001):
        for world in (1, 2, 3, 4, 8):
            for tile_n in (1, 32, 128, 256):
                spans = [api.shard_columns(n, world, r, tile_n) for r in range(world)]
                assert spans == [shard_columns(n, world, r, tile_n) for r in range(world)]
                assert spans[0][0] == 0 and spans[-1][1] == n
                assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert api.lib().sgemm_shard_columns(8, 2, 2, 1, None, None) == -1      # rank out of range, NULL outputs


def test_missing_nccl_is_reported_not_fatal(built):
    """The communicator entry points bind NCCL at run time.  With a library that cannot be loaded (simulated through
    SGEMM_NCCL_LIBRARY) they return SGEMM_ERR_COMM with the loader's message; nothing aborts and the single-GPU entry
    points are unaffected.  Runs in a child process because the binding is made once per process."""
    import subprocess, sys, textwrap
    code = textwrap.dedent(f"""
        import importlib, sys
        sys.path.insert(0, {str(ROOT)!r})
        importlib.import_module("amdgpu-arch-gemm_b200")
        from runner import api
        try:
            api.comm_unique_id()
        except api.SgemmError as e:
            print(e.code, "cannot load NCCL" in str(e))
        print(api.lib().sgemm_strerror(-10).decode())
        print(api.shard_columns(1000, 4, 3, 128))
    """)
    env = dict(__import__("os").environ, SGEMM_NCCL_LIBRARY="/nonexistent/libnccl.so.2")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().split("\n")
    assert lines[0] == "-10 True" and "NCCL" in lines[1] and lines[2] == "(768, 1000)"


def test_runner_program_refuses_more_gpus_than_visible(built, tmp_path):
    """`SGEMM_NGPUS` beyond the visible devices is a request the program cannot serve: exit status 3 and a message,
    before anything is opened (host-side failure path; needs no GPU)."""
    import os, subprocess
    from runner import api
    cubin, toml = built.ensure("simt_64x64x16")
    env = dict(os.environ, SGEMM_NGPUS="64")
    ret = subprocess.run([str(api.RUNNER_PATH), cubin, toml, "64", "64", "64", "1", "1", "0"], capture_output=True, text=True, env=env)
    assert ret.returncode == 3 and "more GPUs than" in ret.stderr and ret.stdout == ""
    env = dict(os.environ, SGEMM_NGPUS="0")
    ret = subprocess.run([str(api.RUNNER_PATH), cubin, toml, "64", "64", "64", "1", "1", "0"], capture_output=True, text=True, env=env)
    assert ret.returncode == 3


def test_bench_reports_ncu_traffic_only_for_the_source_it_was_captured_on(built, tmp_path, monkeypatch):
    """bench.py's `roofline.traffic` comes from the tracked record beside the profile summaries, which carries a hash
    of the emitted kernel source: the figure is reported for exactly that source and shape, and a kernel that changed
    since (or another shape) gets null instead of a stale number."""
    import hashlib, importlib, json, sys
    sys.path.insert(0, str(ROOT))
    bench = importlib.import_module("bench")
    cubin = tmp_path / "generated_gemm.cubin"
    cu = tmp_path / "generated_gemm.cu"
    cu.write_text("// kernel source v1\n")
    record = tmp_path / "dram_traffic.json"
    record.write_text(json.dumps({"k": {"shape": [8, 8, 8], "dram_bytes_per_launch": 123.0, "capture": "cmd",
                                        "source_sha256": hashlib.sha256(cu.read_bytes()).hexdigest()}}))
    monkeypatch.setattr(bench, "TRAFFIC_FILE", record)
    assert bench.ncu_traffic("k", str(cubin), (8, 8, 8)) == (123.0, "cmd")
    assert bench.ncu_traffic("k", str(cubin), (8, 8, 16))[0] is None
    assert bench.ncu_traffic("other", str(cubin), (8, 8, 8))[0] is None
    cu.write_text("// kernel source v2\n")
    assert bench.ncu_traffic("k", str(cubin), (8, 8, 8)) == (None, "kernel source changed since the capture")
    # the tracked record: the figure for the default kernel as generated today, or null when the kernel has changed since
    real = json.loads((ROOT / "profiles" / "dram_traffic.json").read_text())
    cubin_path, _ = built.ensure(built.DEFAULT_TENSOR)
    value, _ = importlib.reload(bench).ncu_traffic(built.DEFAULT_TENSOR, cubin_path, real[built.DEFAULT_TENSOR]["shape"])
    assert value in (None, real[built.DEFAULT_TENSOR]["dram_bytes_per_launch"])


def test_header_is_plain_c(tmp_path):
    """The drop-in boundary is a C ABI: include/sgemm_runner.h must compile as C99 (no C++ or torch types), so that
    any language's FFI can bind it."""
    import subprocess
    src = tmp_path / "use_header.c"
    src.write_text('#include "sgemm_runner.h"\nint main(void) { sgemm_config c; (void)c; return SGEMM_ERR_COMM == -10 ? 0 : 1; }\n')
    ret = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", f"-I{ROOT / 'include'}", str(src)],
                         capture_output=True, text=True)
    assert ret.returncode == 0, ret.stderr
