"""GPU parity on the path the library takes BY ITSELF at the sizes the benchmark quotes: the default cubin, no option
overrides, operands filled on the device by global element index exactly as bench.py fills them.

  * 8192^3 on the default kernel (the CTA-pair kernel with chunked accumulation that bench.py times), for uniform
    [-1, 1) inputs and for same-signed inputs (where a whole-K tensor-core chain would miss the bound);
  * the skinny / irregular shapes, with the kernel, split-K and accumulation chain the library picks for them;
  * column shards of the 32768 x 32768 x 8192 problem as rank r of 8 computes them.

Checked against the CPU oracle (oracle/shard_check.py: sampled columns with the reference's cpuGemm arithmetic,
runner/generator_runner.cpp:16-33, tolerance 1e-5 * sum|a||b| per element, plus linearity checksums over every
element of the result)."""
import numpy as np
import pytest

from oracle import oracle, shard_check

pytestmark = pytest.mark.gpu

TENSOR, SIMT, COMPANION = 1, 2, 3


@pytest.fixture()
def default_runner(built):
    """The default tensor cubin with the library's own defaults: nothing is set on the handle."""
    from runner import api
    cubin, toml = built.ensure(built.DEFAULT_TENSOR)
    r = api.SgemmRunner(cubin, toml, 0)
    yield r
    assert r.last_status()[0] == 0
    r.close()


class DeviceBuffers:
    def __init__(self, r, *counts):
        self.r = r
        self.ptrs = [r.dev_alloc(max(c, 1) * 4) for c in counts]

    def __enter__(self):
        return self.ptrs

    def __exit__(self, *exc):
        self.r.sync()
        for p in self.ptrs:
            self.r.dev_free(p)


_a_cache = {}


def host_a(m, k):
    if (m, k) not in _a_cache:
        _a_cache.clear()
        _a_cache[(m, k)] = shard_check.global_a(m, k)
    return _a_cache[(m, k)]


def run_shard_on_device(r, m, k, n0, n1):
    """What one rank of bench.py does: fill A and B[:, n0:n1] on the device by global index, one launch, D back."""
    from runner.shard import fill_shard_inputs
    width = n1 - n0
    with DeviceBuffers(r, m * k, k * width, m * width) as (pa, pb, pd):
        fill_shard_inputs(r, pa, pb, m, k, n0, n1)
        r.memset(pd, 0xFF, m * width * 4)              # NaN pattern: every element must be written
        r.launch(pa, pb, None, pd, m, width, k, alpha=1.0, beta=0.0)
        d = np.empty(m * width, dtype=np.float32)
        r.sync()
        r.download(d, pd)
    return d


def check_shard(d, m, k, n0, n1, tile_n, columns=64):
    a = host_a(m, k)
    cols = shard_check.sample_columns(n0, n1, tile_n, columns, seed=n0)
    assert cols[0] == n0 and cols[-1] == n1 - 1 and len(cols) >= min(columns, n1 - n0)
    sampled = d.reshape(n1 - n0, m)[cols - n0]
    ratio = shard_check.worst_ratio_of_columns(sampled, cols, m, k, a=a)
    assert ratio <= 1.0, f"sampled columns: worst |err| / (1e-5 sum|a||b|) = {ratio}"
    rows, columns_ratio = shard_check.checksum_ratios(d, n0, n1, m, k, a=a)
    assert rows <= 1.0 and columns_ratio <= 1.0, (rows, columns_ratio)
    return ratio


# --------------------------------------------------------------------- 8192^3 on the kernel the benchmark times
def test_8192_cubed_on_the_default_kernel_as_the_benchmark_runs_it(default_runner):
    r = default_runner
    m = n = k = 8192
    d = run_shard_on_device(r, m, k, 0, n)
    assert r.info("last_variant") == TENSOR and r.info("last_acc_chain") == 128 and r.info("last_split_k") == 1
    assert r.info("last_tile_n") == 256 and r.info("tile_m") == 256          # the CTA-pair kernel, 256 x 256 tiles
    check_shard(d, m, k, 0, n, r.info("tile_n"), columns=96)
    d2 = run_shard_on_device(r, m, k, 0, n)
    assert d.tobytes() == d2.tobytes()                                       # bit-reproducible


def test_8192_cubed_same_signed_inputs_on_the_default_kernel(default_runner):
    """|A| and |B|: nothing cancels, so the truncating adds of one long tensor-core chain would show (16 times the
    bound at K = 8192); the default kernel's chains of 128 k must stay inside it.  Through the host-buffer entry
    point, i.e. the pipelined column chunks, which must pick the kernel the whole problem gets."""
    r = default_runner
    m = n = k = 8192
    a = np.abs(host_a(m, k))
    b = np.abs(oracle.fill_uniform(k * n, 1))
    d = np.zeros(m * n, dtype=np.float32)
    r.run_host(a, b, None, d, m, n, k, alpha=1.0, beta=0.0)
    assert r.info("last_variant") == TENSOR and r.info("last_acc_chain") == 128
    cols = shard_check.sample_columns(0, n, r.info("tile_n"), 96, seed=5)
    b_sub = np.ascontiguousarray(b.reshape(n, k)[cols]).reshape(-1)
    ref = oracle.gemm(a, b_sub, None, 1.0, 0.0, m, len(cols), k)
    bound = oracle.abs_bound(a, b_sub, m, len(cols), k)
    ratio = oracle.worst_ratio(np.ascontiguousarray(d.reshape(n, m)[cols]).reshape(-1), ref, bound)
    assert ratio <= 1.0, ratio
    _a_cache.clear()


# ----------------------------------------------------- the skinny / irregular shapes, library defaults, full oracle
@pytest.mark.parametrize("mnk,variant,split_k,acc_chain,tile_n", [
    ((1024, 1024, 1024), COMPANION, 2, 128, 128),   # small problem: no pre-pass launch
    ((8192, 8192, 256), TENSOR, 1, 0, 256),         # K of two chains: the main kernel's whole-K twin
    ((4096, 128, 16384), COMPANION, 4, 128, 128),   # 32 tiles for 148 SMs: deterministic split-K on the companion kernel
    ((1000, 1000, 1000), COMPANION, 2, 128, 128),   # not a multiple of any tile: TMA zero fill and predicated stores
    ((127, 257, 513), SIMT, 4, 0, 0),               # lda = 127: TMA cannot describe it, FFMA fallback
])
@pytest.mark.parametrize("beta", [0.0, 1.0])
def test_benchmark_shapes_with_library_defaults(default_runner, mnk, variant, split_k, acc_chain, tile_n, beta):
    r = default_runner
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=0)
    with DeviceBuffers(r, m * k, k * n, m * n, m * n) as (pa, pb, pc, pd):
        r.upload(pa, a); r.upload(pb, b); r.upload(pc, c)
        outs = []
        for _ in range(2):
            r.memset(pd, 0xFF, m * n * 4)
            r.launch(pa, pb, pc if beta else None, pd, m, n, k, alpha=1.0, beta=beta)
            d = np.empty(m * n, dtype=np.float32)
            r.sync()
            r.download(d, pd)
            outs.append(d)
    assert r.info("last_variant") == variant
    if r.info("sm_count") == 148:          # the split-K factor is sized for the SMs of the device
        assert r.info("last_split_k") == split_k, r.info("last_split_k")
    assert r.info("last_acc_chain") == acc_chain and r.info("last_tile_n") == tile_n
    assert outs[0].tobytes() == outs[1].tobytes()
    ref = oracle.gemm(a, b, c, 1.0, beta, m, n, k)
    bound = oracle.abs_bound(a, b, m, n, k) + abs(beta) * np.abs(c).astype(np.float64)
    ratio = oracle.worst_ratio(outs[0], ref, bound)
    assert ratio <= 1.0, ratio
    if beta and k <= 1024:
        # the reference runner's own rule (|gpu - cpu| < 1e-3, runner/generator_runner.cpp:295) with its beta = 1; it is
        # an absolute bound, meaningful only while the FP32 sums themselves stay well below 1e-3 of rounding error
        assert oracle.count_mismatches(outs[0], ref) == 0


# ------------------------------------------------------------- 32768 x 32768 x 8192, column shards of rank r of 8
@pytest.mark.parametrize("rank", [0, 3, 7])
def test_shards_of_the_32768_problem_as_rank_r_of_8_computes_them(default_runner, rank):
    from runner.shard import shard_columns
    r = default_runner
    m, n_total, k, world = 32768, 32768, 8192, 8
    tile_n = r.info("tile_n")
    n0, n1 = shard_columns(n_total, world, rank, tile_n)
    assert (n0, n1) == (rank * 4096, (rank + 1) * 4096)
    d = run_shard_on_device(r, m, k, n0, n1)
    assert r.info("last_variant") == TENSOR and r.info("last_acc_chain") == 128 and r.info("last_split_k") == 1
    check_shard(d, m, k, n0, n1, tile_n, columns=64)
    if rank == 7:
        _a_cache.clear()
