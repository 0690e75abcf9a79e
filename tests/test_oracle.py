"""The CPU oracle against the reference's own outputs (golden vectors made by running the unmodified reference
generator + GCN VM, tests/golden/make_golden.py) and against itself (restatement == reference loop order)."""
import numpy as np
import pytest

from oracle import oracle

GOLDEN_CASES = [
    "vm_16x16x64_arange", "vm_32x32x64_arange", "vm_64x48x64_mapk4_arange", "vm_64x48x64_3buf_arange",
    "vm_64x64x32_wgm2_arange", "vm_32x32x32_seed0_mfma32_beta0", "vm_32x32x32_seed0_mfma32_beta1",
    "vm_32x32x32_seed0_mfma16_beta0", "vm_32x32x32_seed0_mfma16_beta1",
]


def load(golden_dir, name):
    z = np.load(golden_dir / f"{name}.npz")
    m, n, k = (int(x) for x in z["mnk"])
    return z["a"], z["b"], z["c"], z["d"], m, n, k, float(z["alpha"]), float(z["beta"])


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_reference_vm(golden_dir, name):
    a, b, c, d_vm, m, n, k, alpha, beta = load(golden_dir, name)
    d = oracle.gemm(a, b, c, alpha, beta, m, n, k)
    if "arange" in name:  # the reference's own acceptance rule for its fixtures (test/test_vm.py:536-537, 626-627)
        assert np.allclose(d, d_vm, rtol=1e-5)
    # and the build's parity rule
    assert oracle.worst_ratio(d, d_vm, oracle.abs_bound(a, b, m, n, k)) <= 1.0


@pytest.mark.parametrize("name", GOLDEN_CASES[:2])
def test_golden_matches_numpy_as_the_reference_checks_it(golden_dir, name):
    a, b, c, d_vm, m, n, k, _, _ = load(golden_dir, name)
    ref = (b.reshape(n, k) @ a.reshape(k, m)) + c.reshape(n, m)  # test/test_vm.py:531-535
    assert np.allclose(d_vm.reshape(n, m), ref, rtol=1e-5)


@pytest.mark.parametrize("mnk", [(1, 1, 1), (7, 5, 3), (33, 17, 65), (128, 96, 200)])
def test_restatement_is_bit_identical_to_reference_loop_order(mnk):
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=3)
    fast = oracle.gemm(a, b, c, 0.75, -1.25, m, n, k)
    ref = oracle.gemm(a, b, c, 0.75, -1.25, m, n, k, ref_order=True)
    assert fast.tobytes() == ref.tobytes()


def test_c_restatement_matches_pure_python_loop():
    m, n, k = 6, 5, 9
    a, b, c = oracle.make_inputs(m, n, k, seed=11)
    assert oracle.gemm(a, b, c, 1.5, 0.5, m, n, k).tobytes() == oracle.gemm_python(a, b, c, 1.5, 0.5, m, n, k).tobytes()


def test_leading_dimensions():
    m, n, k = 10, 7, 13
    a, b, c = oracle.make_inputs(m, n, k, seed=5)
    ap, bp, cp = oracle.make_inputs(m, n, k, seed=5, lda=16, ldb=20, ldc=12)
    dense = oracle.gemm(a, b, c, 1.0, 1.0, m, n, k)
    padded = oracle.gemm(ap, bp, cp, 1.0, 1.0, m, n, k, lda=16, ldb=20, ldc=12, ldd=11)
    assert oracle.strip_ld(padded, m, n, 11).tobytes() == dense.tobytes()


def test_seeded_fill_numpy_equals_c_and_is_uniform():
    x = oracle.fill_uniform(100003, stream=2, first_index=17)
    y = oracle.fill_uniform_numpy(100003, stream=2, first_index=17)
    assert x.tobytes() == y.tobytes()
    assert x.min() >= -1.0 and x.max() < 1.0 and abs(float(x.mean())) < 0.01
    assert oracle.fill_uniform(8, 0).tobytes() != oracle.fill_uniform(8, 1).tobytes()
    # a slice of a stream equals the stream sliced (device fills shard by first_index)
    assert oracle.fill_uniform(50, 4, first_index=100).tobytes() == oracle.fill_uniform(150, 4)[100:].tobytes()


def test_empty_and_degenerate_shapes():
    a, b, c = oracle.make_inputs(4, 3, 1, seed=0)
    assert oracle.gemm(a, b, c, 1.0, 0.0, 4, 3, 1).shape == (12,)
    z = oracle.gemm(np.zeros(1, np.float32), np.zeros(1, np.float32), c, 1.0, 2.0, 4, 3, 0, lda=4, ldb=1)
    assert np.array_equal(z, 2.0 * c)   # K = 0: D = beta*C


def test_reference_comparison_rule_and_metrics():
    x = np.array([0.0, 1.0, 2.0, np.nan], dtype=np.float32)
    y = np.array([0.0005, 1.002, 2.0, 0.0], dtype=np.float32)
    assert oracle.count_mismatches(x, y, 1e-3) == 2  # |diff| >= 1e-3 and NaN (runner/Utils/Math.hpp:5-8)
    assert oracle.gflops(1024, 1024, 1024, 1.0) == pytest.approx(2 * 1024 ** 3 * 1e-6)
    assert oracle.mem_bw(1024, 1024, 1024, 1.0) == pytest.approx(4 * 1024 * 1024 * 4 / 1024 / 1024)


def test_worst_ratio_flags_errors():
    m = n = k = 8
    a, b, c = oracle.make_inputs(m, n, k)
    d = oracle.gemm(a, b, c, 1.0, 0.0, m, n, k)
    s = oracle.abs_bound(a, b, m, n, k)
    assert oracle.worst_ratio(d, d, s) == 0.0
    bad = d.copy()
    bad[5] += 1e-3
    assert oracle.worst_ratio(bad, d, s) > 1.0
    bad[5] = np.nan
    assert oracle.worst_ratio(bad, d, s) == np.inf


def test_shard_checks_accept_a_correct_shard_and_catch_an_offset_error():
    """The checker of the multi-GPU workload (oracle/shard_check.py) on the CPU: a shard of D computed in FP64 from
    the globally indexed inputs passes the sampled-column check and both checksums; the same shard computed from a B
    that was filled with the wrong first index (one column off) fails all three."""
    from oracle import shard_check
    m, n, k, tile_n = 96, 320, 200, 64
    a = shard_check.global_a(m, k)
    for n0, n1 in ((0, 128), (128, 320)):
        cols = shard_check.sample_columns(n0, n1, tile_n, 24, seed=1)
        assert cols[0] == n0 and cols[-1] == n1 - 1 and len(set(cols)) == len(cols) <= 24
        assert {n0 + tile_n - 1, n0 + tile_n}.issubset(set(cols) | {n1}) or n1 - n0 <= tile_n
        for shift, ok in ((0, True), (1, False)):
            b = oracle.fill_uniform(k * (n1 - n0), 1, first_index=(n0 + shift) * k)
            d = (b.reshape(n1 - n0, k).astype(np.float64) @ a.reshape(k, m).astype(np.float64)).astype(np.float32)
            ratio = shard_check.worst_ratio_of_columns(d[cols - n0], cols, m, k)
            rows, columns = shard_check.checksum_ratios(d.reshape(-1), n0, n1, m, k, block=64)
            assert (ratio <= 1.0) == ok and (rows <= 1.0) == ok and (columns <= 1.0) == ok, (n0, shift, ratio, rows, columns)
