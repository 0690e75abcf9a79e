"""GPU parity of the TMA-fed, warp-specialised FFMA kernel (csrc/sgemm_ffma_tma.cuh), called through the C ABI.

It computes what the register-fed FFMA kernel computes — per element one fused multiply-add per k, k ascending, strict
FP32 — so it is held to the oracle's bound (|D - D_ref| <= 1e-5 * sum_l |a_il||b_lj|, oracle.REL_TOL) and, for equal
split-K factors, to bit-equality with the register-fed kernel, whatever the two kernels' tiles."""
import numpy as np
import pytest

from oracle import oracle
from test_gpu_parity import check, run, runner_of, stored  # noqa: F401  (runner_of is a fixture)

pytestmark = pytest.mark.gpu

SIMT = 2
KERNELS = ["ffma_tma_256x128x32_s3", "ffma_tma_256x128x16_s4", "ffma_tma_128x256x16_s4", "ffma_tma_128x128x16_s4", "ffma_tma_128x128x16_t16x8_s6"]
SHAPES = [(1, 1, 1), (8, 8, 8), (32, 32, 32), (33, 65, 129), (127, 257, 513), (256, 128, 16), (257, 129, 17),
          (512, 384, 96), (1000, 1000, 1000), (1024, 1024, 1024), (130, 4, 2048), (4, 300, 77)]


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("mnk", SHAPES)
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (0.5, -1.5)])
def test_matches_oracle_and_the_register_fed_kernel(runner_of, kernel, mnk, alpha, beta):
    m, n, k = mnk
    lda, ldb = (m + 3) // 4 * 4, (k + 3) // 4 * 4   # TMA needs 16-byte row pitches; pad ragged shapes
    a, b, c = oracle.make_inputs(m, n, k, seed=0, lda=lda, ldb=ldb)
    r = runner_of(kernel)
    d = run(r, a, b, c, m, n, k, alpha, beta, force=SIMT, split_k=1, lda=lda, ldb=ldb)
    assert r.info("last_variant") == SIMT and r.info("last_feed_tma") == 1
    check(d, a, b, c, m, n, k, alpha, beta, lda=lda, ldb=ldb)
    ref = runner_of("simt_128x128x16")
    d_ldg = run(ref, a, b, c, m, n, k, alpha, beta, force=SIMT, split_k=1, lda=lda, ldb=ldb)
    assert ref.info("last_feed_tma") == 0
    assert np.array_equal(d.view(np.uint32), d_ldg.view(np.uint32))


@pytest.mark.parametrize("kernel", ["ffma_tma_256x128x16_s4", "ffma_tma_128x128x16_s4"])
@pytest.mark.parametrize("mnk,split", [((256, 128, 4096), 4), ((130, 70, 1000), 3), ((512, 256, 8192), 0), ((96, 96, 515), 7)])
def test_split_k_is_deterministic_and_right(runner_of, kernel, mnk, split):
    m, n, k = mnk
    lda, ldb = (m + 3) // 4 * 4, (k + 3) // 4 * 4
    a, b, c = oracle.make_inputs(m, n, k, seed=3, lda=lda, ldb=ldb)
    r = runner_of(kernel)
    d1 = run(r, a, b, c, m, n, k, 1.0, 1.0, force=SIMT, split_k=split, lda=lda, ldb=ldb)
    used = r.info("last_split_k")
    assert r.info("last_feed_tma") == 1 and (used == split if split else used > 1)
    check(d1, a, b, c, m, n, k, 1.0, 1.0, lda=lda, ldb=ldb)
    d2 = run(r, a, b, c, m, n, k, 1.0, 1.0, force=SIMT, split_k=split, lda=lda, ldb=ldb)
    assert np.array_equal(d1.view(np.uint32), d2.view(np.uint32))


def test_transposed_b(runner_of):
    m, n, k = 300, 260, 200
    a, b, c = oracle.make_inputs(m, n, k, seed=5)
    bt, ldb = stored(b, k, n, True, ld=264)
    r = runner_of("ffma_tma_256x128x16_s4_nt")
    d = run(r, a, bt, c, m, n, k, 2.0, 0.25, force=SIMT, ldb=ldb)
    assert r.info("last_feed_tma") == 1
    ref = oracle.gemm(a, b, c, 2.0, 0.25, m, n, k)
    bound = 2.0 * oracle.abs_bound(a, b, m, n, k) + 0.25 * np.abs(c).astype(np.float64)
    assert oracle.worst_ratio(d, ref, bound) <= 1.0


def test_padded_leading_dimensions_leave_the_padding_alone(runner_of):
    m, n, k = 200, 150, 120
    lda, ldb, ldc, ldd = 208, 128, 204, 212
    a, b, c = oracle.make_inputs(m, n, k, seed=7, lda=lda, ldb=ldb, ldc=ldc)
    r = runner_of("ffma_tma_256x128x16_s4")
    canary = np.full(ldd * n, 123.25, dtype=np.float32)
    d = run(r, a, b, c, m, n, k, 1.0, 1.0, force=SIMT, lda=lda, ldb=ldb, ldc=ldc, ldd=ldd, d_init=canary)
    assert r.info("last_feed_tma") == 1
    check(d, a, b, c, m, n, k, 1.0, 1.0, lda=lda, ldb=ldb, ldc=ldc, ldd=ldd)
    assert np.all(d.reshape(n, ldd)[:, m:] == 123.25)


def test_operands_tma_cannot_describe_go_to_the_register_fed_kernel(runner_of):
    m, n, k = 127, 257, 513          # odd leading dimensions
    a, b, c = oracle.make_inputs(m, n, k, seed=0)
    r = runner_of("ffma_tma_256x128x16_s4")
    r.set_option("repitch", 0)
    d = run(r, a, b, c, m, n, k, 1.0, 0.0, force=SIMT)
    assert r.info("last_variant") == SIMT and r.info("last_feed_tma") == 0
    check(d, a, b, c, m, n, k, 1.0, 0.0)

