"""Generator API: the reference's usage patterns (test/test_sgemm.py:4-44, tuner/sgemm_tuner.py:52-110) must
work unchanged against this generator, with sm_100a meanings for the knobs."""
import os
import re
import tomllib

import pytest

from generator import generator as g
from generator.generator import (DataType, FunctionArgument, GemmOptimizations, GemmSolutionConfig, compile, gemm)

ARGS = lambda: [
    FunctionArgument("global_buffer", "a", None, 8), FunctionArgument("global_buffer", "b", None, 8),
    FunctionArgument("global_buffer", "c", None, 8), FunctionArgument("global_buffer", "d", None, 8),
    FunctionArgument("by_value", "m", None, 4), FunctionArgument("by_value", "n", None, 4),
    FunctionArgument("by_value", "k", None, 4), FunctionArgument("by_value", "lda", None, 4),
    FunctionArgument("by_value", "ldb", None, 4), FunctionArgument("by_value", "ldc", None, 4),
    FunctionArgument("by_value", "ldd", None, 4), FunctionArgument("by_value", "alpha", None, 4),
    FunctionArgument("by_value", "beta", None, 4), FunctionArgument("by_value", "numWorkgroupX", None, 4),
    FunctionArgument("by_value", "numWorkgroupY", None, 4),
]
F = DataType.FP32


def test_basic_sgemm_gen_reference_style():
    # the reference's generation smoke test, verbatim in shape: a GCN-style config must still generate
    cfg = g.GemmSolutionConfig(F, F, F, F, (16, 16, 1, 4), (2, 2), (2, 2), 16, False, False)
    src = g.gemm(None, "gemm", "sm_100a", cfg, g.GemmOptimizations(1), ARGS())
    assert len(src) and 'extern "C" __global__' in src and "generated_gemm" in src
    assert cfg.tile_size == (64, 64) and cfg.variant == g.VARIANT_SIMT


def test_tile_product_rule_and_properties():
    cfg = g.tensor_config(256, 32, 2)
    assert cfg.tile_size == (128, 256) and cfg.num_workitems == 128 + 32 * 8 and cfg.stages == 2
    assert g.tensor_config(256, 32, 2, epilogue_warps=4).num_workitems == 256   # warp groups of four: 4 + 4 warps
    ring = 2 * (2 * 128 * 32 * 4 + 2 * 256 * 32 * 4) + 1024 + 256
    assert cfg.acc_chain == 128 and cfg.lds_usage_bytes == ring      # chunked accumulation by default (chains of 128 k)
    whole_k = g.tensor_config(256, 32, 2, acc_chain=0)
    assert whole_k.lds_usage_bytes == ring and whole_k.to_dict()["acc_chain"] == 0
    with pytest.raises(RuntimeError):
        g.tensor_config(256, 32, 2, acc_chain=100)                   # not a multiple of depth_k
    with pytest.raises(RuntimeError):
        g.tensor_config(256, 32, 2, epilogue_warps=4, acc_chain=128)   # 256 running-sum registers per thread
    assert g.tensor_config(256, 32, 2, epilogue_warps=4).acc_chain == 0   # ... so the default there is one chain
    assert cfg.tmem_columns == 512
    s = g.simt_config(128, 128, 16, 8, 8)
    assert s.tile_size == (128, 128) and s.num_workitems == 256
    assert s.lds_usage_bytes == 2 * 16 * (128 + 4 + 128 + 4) * 4
    assert s.num_bytes_per_buffer_load == (16, 16)  # the tuner's vector-load filter (tuner/sgemm_tuner.py:102)


@pytest.mark.parametrize("kwargs", [
    dict(mfma=(128, 256, 1, 8), wg=(1, 1), wt=(1, 1), dk=32, vs=2),     # 3 stages of 96 KiB: over the smem budget
    dict(mfma=(128, 512, 1, 8), wg=(1, 1), wt=(1, 1), dk=32, vs=1),     # N beyond the UMMA / TMEM limit
    dict(mfma=(128, 128, 1, 8), wg=(1, 1), wt=(1, 1), dk=48, vs=1),     # k per stage neither 16 nor whole 128-byte spans
    dict(mfma=(128, 128, 1, 8), wg=(3, 1), wt=(1, 1), dk=32, vs=1),     # wave_group not a power of two
    dict(mfma=(1, 1, 1, 1), wg=(16, 16), wt=(8, 8), dk=64, vs=1),       # SIMT static smem over 48 KiB
    dict(mfma=(64, 64, 1, 8), wg=(1, 1), wt=(1, 1), dk=32, vs=1),       # no such atom
])
def test_infeasible_configs_raise_runtime_error(kwargs):
    with pytest.raises(RuntimeError):  # the tuner's skip mechanism (tuner/sgemm_tuner.py:92)
        GemmSolutionConfig(F, F, F, F, kwargs["mfma"], kwargs["wg"], kwargs["wt"], kwargs["dk"], False, False,
                           vmem_stage=kwargs["vs"])


def test_transposes_select_operand_layouts():
    # trans_a / trans_b exist in the reference's config and TOML (generator/generator.py:868-869, 1008-1009) but only NN
    # is implemented there; here they pick the operand layout at generation time
    cfg = g.tensor_config(256, 32, 3, cluster=2, trans_a=True, trans_b=True)
    src = gemm(None, "k", "sm_100a", cfg, GemmOptimizations(1), ARGS())
    assert "#define GEMM_TRANS_A 1" in src and "#define GEMM_TRANS_B 1" in src
    assert "#define TC_A_KMAJOR 1" in src and "#define TC_B_MNMAJOR 1" in src
    assert cfg.to_dict()["trans_a"] is True and cfg.to_dict()["trans_b"] is True
    nn = gemm(None, "k", "sm_100a", g.tensor_config(256, 32, 3, cluster=2), GemmOptimizations(1), ARGS())
    assert "#define GEMM_TRANS_A 0" in nn and "#define TC_A_KMAJOR 0" in nn and "#define TC_B_MNMAJOR 0" in nn
    with pytest.raises(RuntimeError):   # a transposed A is K-major already; the packed-copy knob does not apply
        g.tensor_config(128, 32, 3, trans_a=True, a_major="k")


def test_k_stagger_and_foreign_archs_are_rejected():
    with pytest.raises(RuntimeError):
        gemm(None, "k", "sm_100a", g.simt_config(), GemmOptimizations(1, map_k_idx=4), ARGS())
    with pytest.raises(RuntimeError):
        gemm(None, "k", "gfx90a", g.simt_config(), GemmOptimizations(1), ARGS())
    with pytest.raises(RuntimeError):
        gemm(None, "k", "sm_100a", g.simt_config(), GemmOptimizations(1), ARGS()[:-1])


def test_optimization_defaults_follow_the_reference():
    o0, o1 = GemmOptimizations(0), GemmOptimizations(1)
    assert (o0.wgm, o0.plr, o0.gw, o0.map_k_idx) == (1, 0, 0, 0)
    assert (o1.wgm, o1.plr, o1.gw, o1.map_k_idx) == (1, 1, 1, 0)
    assert GemmOptimizations(1, wgm=4, plr=0).plr == 0


def test_kernel_argument_offsets_match_the_76_byte_segment():
    args = ARGS()
    gemm(None, "k", "sm_100a", g.simt_config(), GemmOptimizations(1), args)
    assert [a.offset for a in args] == [0, 8, 16, 24, 32, 36, 40, 44, 48, 52, 56, 60, 64, 68, 72]


def test_emitted_source_knobs_and_no_cluster_multicast():
    src = gemm(None, "k", "sm_100a", g.tensor_config(128, 32, 3), GemmOptimizations(1, wgm=4), ARGS())
    assert "#define OPT_WGM 4" in src and "#define TC_BN 128" in src and "#define TC_STAGES 3" in src
    assert "tcgen05.mma" in src and "cp.async.bulk.tensor" in src and "generated_gemm_simt" in src
    assert "multicast" not in src
    simt = gemm(None, "k", "sm_100a", g.simt_config(64, 64, 16, 4, 4), GemmOptimizations(0), ARGS())
    assert "#define SIMT_PLR 0" in simt and "tcgen05" not in simt


def test_compile_writes_cu_cubin_toml(tmp_path):
    cfg = g.simt_config(64, 64, 16, 4, 4)
    src = gemm(None, "generated_gemm", "sm_100a", cfg, GemmOptimizations(1), ARGS())
    assert compile("generated_gemm", src, "sm_100a", str(tmp_path), cfg) == 0
    for ext in ("cu", "cubin", "toml"):
        assert (tmp_path / f"generated_gemm.{ext}").stat().st_size > 0
    with open(tmp_path / "generated_gemm.toml", "rb") as f:
        d = tomllib.load(f)
    legacy = ["a_type", "b_type", "cd_type", "scalar_type", "wave_group", "trans_a", "trans_b", "mfma", "wave_tiling",
              "depth_k", "vmem_stage", "wavefront_size", "lds_usage_bytes", "name"]
    assert list(d)[:14] == legacy  # generator/generator.py:1001-1017, same order
    assert d["mfma"] == [1, 1, 1, 1] and d["wave_group"] == [16, 16] and d["variant"] == "simt_ffma"
    assert d["num_threads"] == 256 and d["entry"] == "generated_gemm"
    # a kernel that does not compile returns non-zero and leaves no TOML behind
    assert compile("broken", "this is not CUDA", "sm_100a", str(tmp_path), cfg) != 0
    assert not (tmp_path / "broken.toml").exists()


def test_reference_tuner_filters_work():
    # tuner/sgemm_tuner.py:97-110 in miniature
    cfg = g.tensor_config(128, 32, 3)
    m, n, k = 1024, 1024, 1024
    assert not ((m % cfg.tile_size[0]) or (n % cfg.tile_size[1]) or (k % cfg.depth_k))
    assert cfg.num_bytes_per_buffer_load[0] % 16 == 0


@pytest.mark.parametrize("nx,ny,wgm", [(8, 8, 4), (8, 8, 1), (7, 5, 4), (64, 32, 8), (3, 9, 8), (1, 1, 2)])
def test_tile_raster_model(nx, ny, wgm):
    seen = [g.tile_raster(z, nx, ny, wgm) for z in range(nx * ny)]
    assert sorted(seen) == sorted((x, y) for x in range(nx) for y in range(ny))  # a permutation of the grid
    if nx % wgm == 0 and wgm > 1:  # the reference's formula, test/test_vm.py:735-740
        for z, (x, y) in enumerate(seen):
            assert (x, y) == ((z % wgm) + (z // wgm // ny) * wgm, (z // wgm) % ny)


def test_sixteen_bit_operand_types():
    """FP16 / BF16 A and B on the tensor variant (the reference has the type plumbing, FP32 only:
    generator/generator.py:816-824): operands read where they lie (K-major or MN-major tiles), one MMA per 16 k, no lo
    tiles, no companion kernel."""
    cfg = g.tensor_config(256, 64, 4, cluster=2, ab_type=g.DataType.BF16)
    assert cfg.variant == g.VARIANT_TENSOR and cfg.terms == 1 and cfg.a_major == "mn" and cfg.companion_config() is None
    assert "#define TC_A_KMAJOR 0" in g.gemm(None, "gemm", "sm_100a", cfg, g.GemmOptimizations(1), ARGS())   # MN-major A as it lies
    packed = g.tensor_config(256, 64, 4, cluster=2, ab_type=g.DataType.BF16, a_major="k")                    # ... or a packed copy
    assert "#define TC_A_KMAJOR 1" in g.gemm(None, "gemm", "sm_100a", packed, g.GemmOptimizations(1), ARGS())
    assert cfg.lds_usage_bytes == 4 * (128 + 128) * 64 * 2 + 1024 + 256          # A and B tiles only, 2 bytes per element
    d = cfg.to_dict()
    assert (d["a_type"], d["b_type"], d["cd_type"], d["scalar_type"]) == (2, 2, 0, 0) and d["mfma"] == [128, 256, 1, 16]
    src = g.gemm(None, "gemm", "sm_100a", cfg, g.GemmOptimizations(1), ARGS())
    assert "#define TC_ELEM_BYTES 2" in src and "#define TC_AB_FORMAT 1u" in src and "#define TC_TERMS 1" in src
    assert "generated_gemm_wholek" in src and "generated_gemm_skinny" not in src
    tn = g.tensor_config(128, 32, 4, trans_a=True, ab_type=g.DataType.FP16)
    assert tn.a_major == "mn" and tn.to_dict()["a_type"] == 1     # a transposed A is K-major as it lies: no packed copy
    tt = g.tensor_config(128, 64, 3, trans_a=True, trans_b=True, ab_type=g.DataType.BF16)   # B^T: an MN-major tile as it lies
    assert "#define TC_B_MNMAJOR 1" in g.gemm(None, "gemm", "sm_100a", tt, g.GemmOptimizations(1), ARGS())
    with pytest.raises(RuntimeError):
        g.tensor_config(64, 64, 3, cluster=2, trans_b=True, ab_type=g.DataType.BF16)          # 32 columns per CTA: less than a 64-column chunk
    for bad in (dict(split="inkernel"), dict(bk=16), dict(bk=48)):
        kw = dict(bn=128, bk=64, stages=3, ab_type=g.DataType.FP16)
        kw.update(bad)
        with pytest.raises(RuntimeError):
            g.tensor_config(**kw)
    F, H = g.DataType.FP32, g.DataType.FP16
    with pytest.raises(RuntimeError):
        g.GemmSolutionConfig(H, H, F, F, (1, 1, 1, 1), (16, 16), (8, 8), 16, False, False)    # no 16-bit FFMA kernel
    with pytest.raises(RuntimeError):
        g.GemmSolutionConfig(H, F, F, F, (128, 128, 1, 16), (1, 1), (1, 1), 64, False, False)  # mixed operand types
    with pytest.raises(RuntimeError):
        g.GemmSolutionConfig(H, H, H, F, (128, 128, 1, 16), (1, 1), (1, 1), 64, False, False)  # C and D stay FP32


def test_failed_compile_leaves_the_old_kernel_and_ensure_keeps_calling_it_stale(tmp_path, monkeypatch):
    """compile() must not leave a new source beside an old cubin: after a compiler failure the three files of the
    previous build are still there, unchanged, and kernels.ensure() still reports the kernel as stale (it raises again
    instead of handing out the old cubin as fresh); once the compiler works again the kernel is rebuilt."""
    import kernels

    monkeypatch.setattr(kernels, "GENERATED_DIR", tmp_path)
    monkeypatch.setattr(kernels, "_fresh", set())
    name = "simt_64x64x16"
    monkeypatch.setitem(kernels.REGISTRY, name, (kernels.REGISTRY[name][0], dict(wgm=4)))
    cubin, toml = kernels.ensure(name)
    files = {s: (tmp_path / name / f"generated_gemm.{s}") for s in ("cu", "cubin", "toml")}
    before = {s: f.read_bytes() for s, f in files.items()}
    assert not any(p.name.startswith(".build-") for p in (tmp_path / name).iterdir())   # the scratch directory is gone

    # a changed knob makes the emitted source differ; the compiler is "broken"
    monkeypatch.setitem(kernels.REGISTRY, name, (kernels.REGISTRY[name][0], dict(wgm=2)))
    monkeypatch.setattr(kernels, "_fresh", set())
    monkeypatch.setattr(g, "DEFAULT_NVCC_PATH", "/bin/false")
    for _ in range(2):                                   # stale the first time, and still stale the second time
        with pytest.raises(RuntimeError):
            kernels.ensure(name)
        assert {s: f.read_bytes() for s, f in files.items()} == before
        assert not any(p.name.startswith(".build-") for p in (tmp_path / name).iterdir())
    monkeypatch.undo()
    monkeypatch.setattr(kernels, "GENERATED_DIR", tmp_path)
    monkeypatch.setattr(kernels, "_fresh", set())
    monkeypatch.setitem(kernels.REGISTRY, name, (kernels.REGISTRY[name][0], dict(wgm=2)))
    kernels.ensure(name)
    assert files["cu"].read_bytes() != before["cu"] and b"OPT_WGM 2" in files["cu"].read_bytes()


def test_concurrent_ensure_builds_once(tmp_path):
    """Several processes asking for the same missing kernel (ranks under torchrun) serialise on the kernel's lock:
    all of them end up with the same complete files, and none fails on a half-written cubin."""
    import subprocess, sys, textwrap
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    code = textwrap.dedent(f"""
        import importlib, sys, hashlib
        sys.path.insert(0, {str(root)!r})
        importlib.import_module("amdgpu-arch-gemm_b200")
        import kernels
        from pathlib import Path
        kernels.GENERATED_DIR = Path({str(tmp_path)!r})
        cubin, toml = kernels.ensure("simt_64x64x16")
        print(hashlib.sha256(Path(cubin).read_bytes()).hexdigest(), Path(cubin).stat().st_mtime_ns)
    """)
    procs = [subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, text=True) for _ in range(3)]
    outs = [p.communicate()[0].split() for p in procs]
    assert all(p.returncode == 0 for p in procs)
    assert len({o[0] for o in outs}) == 1 and len({o[1] for o in outs}) == 1    # one build, seen by all


def test_tma_fed_ffma_configuration():
    """feed="tma": the FFMA variant as a producer / consumer kernel over a TMA ring; the register-fed fallback kernel
    travels in the same cubin for operands TMA cannot describe."""
    cfg = g.simt_config(256, 128, 16, 16, 8, feed="tma", stages=4)
    assert cfg.variant == g.VARIANT_SIMT and cfg.tile_size == (256, 128) and cfg.stages == 4
    assert cfg.num_workitems == 128 + 256                                   # the producer's warp group + 256 consumers
    assert cfg.lds_usage_bytes == 4 * (256 + 128 + 128) * 16 * 4 + 128 + 512  # A, B and the raw B that is transposed into it
    assert g.simt_config(256, 128, 16, 16, 8, trans_b=True, feed="tma", stages=4).lds_usage_bytes == 4 * (256 + 128) * 16 * 4 + 128 + 512
    d = cfg.to_dict()
    assert d["variant"] == g.VARIANT_SIMT and d["feed"] == "tma" and d["dynamic_smem_bytes"] == cfg.lds_usage_bytes
    assert d["fallback_entry"] == g.SIMT_FALLBACK_ENTRY and d["fallback_tile"] == [128, 128, 16] and d["fallback_threads"] == 256
    src = g.gemm(None, "gemm", "sm_100a", cfg, g.GemmOptimizations(1, wgm=8), ARGS())
    for needle in ("#define FT_ENTRY generated_gemm\n", "#define SIMT_ENTRY generated_gemm_simt\n", "#define FT_BM 256\n",
                   "#define FT_TM 16\n", "#define FT_STAGES 4\n", "cp.async.bulk.tensor.2d", "setmaxnreg.inc"):
        assert needle in src, needle
    assert "multicast" not in src
    plain = g.simt_config(128, 128, 16, 8, 8)
    assert "feed" not in plain.to_dict() and plain.to_dict()["dynamic_smem_bytes"] == 0
    assert "cp.async.bulk" not in g.gemm(None, "gemm", "sm_100a", plain, g.GemmOptimizations(1), ARGS())
    with pytest.raises(RuntimeError, match="untransposed A"):
        g.simt_config(256, 128, 16, 16, 8, trans_a=True, feed="tma", stages=4)
    with pytest.raises(RuntimeError, match="groups of four warps"):
        g.simt_config(64, 64, 16, 8, 8, feed="tma", stages=4)               # 64 consumers
    with pytest.raises(RuntimeError, match="LDS usage"):
        g.simt_config(256, 256, 64, 16, 8, feed="tma", stages=8)
    with pytest.raises(RuntimeError, match="FFMA variant"):
        g.tensor_config(256, 32, 3, cluster=2, feed="tma")
