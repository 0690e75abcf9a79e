"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle and the golden vectors of
the reference's own generator + VM.  Tolerance (FP32 GEMM): per element |D - D_ref| <= 1e-5 * sum_l |a_il||b_lj|
(oracle.REL_TOL); split-free FP32 kernels and the 3xTF32 kernel are held to the same bound."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

TENSOR_KERNELS = ["tc_128x256x32_s2", "tc_128x128x32_s3", "tc_128x64x32_s4", "tc_128x64x64_s2", "tc_128x128x32_s3_ak",
                  "tc_128x256x16_s4", "tc_128x128x16_s7", "tc_128x128x16_s6_ak",
                  "tc2_256x256x32_s3", "tc2_256x256x16_s6", "tc2_256x128x32_s4",
                  "tc2i_256x256x32_s3", "tc2i_256x256x16_s6", "tci_128x256x32_s2", "tci_128x128x32_s3",
                  "tc2_256x256x32_s3_e4", "tc2h_256x256x32_s3"]
# (kernels built for transposed operands have their own tests below)
SIMT_KERNELS = ["simt_128x128x16", "simt_128x128x16_t16x8", "simt_64x64x16", "simt_128x64x8_plr0", "legacy_32x32x2_1wave", "legacy_16x16x4_2x2x2x2"]
AUTO, TENSOR, SIMT, SKINNY = 0, 1, 2, 3
_runners = {}


@pytest.fixture(scope="module")
def runner_of(built):
    from runner import api

    def get(name):
        if name not in _runners:
            cubin, toml = built.ensure(name)
            _runners[name] = api.SgemmRunner(cubin, toml, 0)
        r = _runners[name]
        r.set_option("force_variant", AUTO)
        r.set_option("split_k", 0)
        r.set_option("skinny_below_intensity", 0)   # parity tests pick kernels explicitly
        r.set_option("skinny_below_flops", 0)
        r.set_option("repitch", 1)
        r.set_workspace(None, 0)
        return r

    yield get
    for r in _runners.values():
        assert r.last_status()[0] == 0  # no kernel ever gave up on a wait
        r.close()
    _runners.clear()


def run(r, a, b, c, m, n, k, alpha=1.0, beta=0.0, force=AUTO, split_k=0, lda=0, ldb=0, ldc=0, ldd=0, d_init=None):
    r.set_option("force_variant", force)
    r.set_option("split_k", split_k)
    d = np.zeros(max((ldd or m) * n, 1), dtype=np.float32) if d_init is None else d_init.copy()
    r.run_host(a, b, c if beta != 0.0 else None, d, m, n, k, alpha=alpha, beta=beta, lda=lda, ldb=ldb, ldc=ldc, ldd=ldd)
    return d[: (ldd or m) * n]


def check(d, a, b, c, m, n, k, alpha, beta, lda=0, ldb=0, ldc=0, ldd=0):
    ref = oracle.gemm(a, b, c, alpha, beta, m, n, k, lda=lda or None, ldb=ldb or None, ldc=ldc or None)
    bound = abs(alpha) * oracle.abs_bound(a, b, m, n, k, lda=lda or None, ldb=ldb or None)
    if beta != 0.0:
        bound = bound + abs(beta) * np.abs(oracle.strip_ld(c, m, n, ldc or m)).astype(np.float64)
    got = oracle.strip_ld(d, m, n, ldd or m)
    ratio = oracle.worst_ratio(got, ref, bound)
    assert ratio <= 1.0, f"worst |err| / (1e-5 * sum|a||b|) = {ratio}"
    return ratio


def stored(flat, rows, cols, transposed, ld=0):
    """Column-major rows x cols matrix (flat) as the kernel expects it: as is, or stored transposed (cols x rows
    column-major), optionally with a padded leading dimension."""
    mat = flat.reshape(cols, rows)                    # numpy row = one column of the matrix
    if transposed:
        mat = np.ascontiguousarray(mat.T)             # rows x cols array = cols-contiguous storage
    inner = mat.shape[1]
    ld = ld or inner
    out = np.zeros(mat.shape[0] * ld, dtype=np.float32)
    out.reshape(mat.shape[0], ld)[:, :inner] = mat
    return out, ld


# ------------------------------------------------------------------------------------------- golden vectors
GOLDEN = ["vm_16x16x64_arange", "vm_32x32x64_arange", "vm_64x48x64_mapk4_arange", "vm_64x48x64_3buf_arange",
          "vm_64x64x32_wgm2_arange", "vm_32x32x32_seed0_mfma32_beta0", "vm_32x32x32_seed0_mfma32_beta1",
          "vm_32x32x32_seed0_mfma16_beta0", "vm_32x32x32_seed0_mfma16_beta1"]


@pytest.mark.parametrize("kernel", TENSOR_KERNELS + SIMT_KERNELS)
@pytest.mark.parametrize("name", GOLDEN)
def test_golden_vectors_of_the_reference_vm(runner_of, golden_dir, kernel, name):
    z = np.load(golden_dir / f"{name}.npz")
    m, n, k = (int(x) for x in z["mnk"])
    a, b, c, d_vm = z["a"], z["b"], z["c"], z["d"]
    alpha, beta = float(z["alpha"]), float(z["beta"])
    r = runner_of(kernel)
    d = run(r, a, b, c, m, n, k, alpha, beta, force=TENSOR if kernel in TENSOR_KERNELS else SIMT)
    assert r.info("last_variant") == (TENSOR if kernel in TENSOR_KERNELS else SIMT)
    bound = oracle.abs_bound(a, b, m, n, k) + abs(beta) * np.abs(c).astype(np.float64)
    assert oracle.worst_ratio(d, d_vm, bound) <= 1.0
    if "arange" in name:
        assert np.allclose(d, d_vm, rtol=1e-5)  # the reference's acceptance rule, test/test_vm.py:536-537


# ------------------------------------------------------------------------------- seeded shapes vs the oracle
SHAPES = [(1, 1, 1), (8, 8, 8), (32, 32, 32), (33, 65, 129), (127, 257, 513), (128, 256, 32), (129, 255, 33),
          (256, 512, 96), (1000, 1000, 1000), (1024, 1024, 1024), (130, 4, 2048), (4, 300, 77)]


@pytest.mark.parametrize("kernel", ["tc_128x256x32_s2", "tc_128x128x32_s3", "tc_128x64x64_s2", "tc_128x128x32_s3_ak",
                                    "tc_128x256x16_s4", "tc_128x128x16_s6_ak", "tc2_256x256x32_s3", "tc2_256x128x32_s4",
                                    "tc2i_256x256x32_s3", "tc2i_256x256x16_s6", "tci_128x256x32_s2", "tc2h_256x256x32_s3"])
@pytest.mark.parametrize("mnk", SHAPES)
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (0.5, -1.5)])
def test_tensor_kernels_match_oracle(runner_of, kernel, mnk, alpha, beta):
    m, n, k = mnk
    lda, ldb = (m + 3) // 4 * 4, (k + 3) // 4 * 4   # TMA needs 16-byte row pitches; pad ragged shapes
    a, b, c = oracle.make_inputs(m, n, k, seed=0, lda=lda, ldb=ldb)
    r = runner_of(kernel)
    d = run(r, a, b, c, m, n, k, alpha, beta, force=TENSOR, lda=lda, ldb=ldb)
    assert r.info("last_variant") == TENSOR
    check(d, a, b, c, m, n, k, alpha, beta, lda=lda, ldb=ldb)


@pytest.mark.parametrize("kernel", SIMT_KERNELS)
@pytest.mark.parametrize("mnk", SHAPES)
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (0.5, -1.5)])
def test_simt_kernels_match_oracle(runner_of, kernel, mnk, alpha, beta):
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=0)
    r = runner_of(kernel)
    d = run(r, a, b, c, m, n, k, alpha, beta, force=SIMT)
    assert r.info("last_variant") == SIMT
    check(d, a, b, c, m, n, k, alpha, beta)


@pytest.mark.parametrize("kernel,ta,tb", [("tc2_256x256x32_s3", False, False), ("tc_128x256x32_s2", False, False),
                                          ("tc2_256x256x32_s3_tt", True, True)])
@pytest.mark.parametrize("mnk", SHAPES + [(4096, 128, 2048)])
def test_companion_kernel_matches_oracle(runner_of, kernel, ta, tb, mnk):
    # every tensor-variant cubin carries a second tcgen05 kernel (128 x 128 x 32 tiles, lo terms made in the kernel)
    # for low-intensity shapes; forced here on all shapes
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=41)
    pad = lambda x: (x + 3) // 4 * 4
    sa, lda = stored(a, m, k, ta, pad(k if ta else m))
    sb, ldb = stored(b, k, n, tb, pad(n if tb else k))
    r = runner_of(kernel)
    launches = r.info("launches")
    d = run(r, sa, sb, c, m, n, k, 0.5, 2.0, force=SKINNY, lda=lda, ldb=ldb)
    assert r.info("last_variant") == SKINNY
    assert r.info("launches") - launches == (1 if r.info("last_split_k") == 1 else 2)   # no pre-pass
    check(d, a, b, c, m, n, k, 0.5, 2.0)


def test_low_intensity_shapes_take_the_companion_kernel(runner_of):
    r = runner_of("tc2_256x256x32_s3")
    r.set_option("skinny_below_intensity", 200)          # the library's defaults: flop per byte of A and B,
    r.set_option("skinny_below_flops", 1 << 33)          # and problems this small
    for (m, n, k), want in [((4096, 128, 4096), SKINNY), ((64, 4096, 8192), SKINNY), ((2048, 2048, 2048), TENSOR),
                            ((4096, 4096, 256), TENSOR), ((1024, 1024, 1024), SKINNY), ((1536, 1536, 1536), SKINNY)]:
        a, b, c = oracle.make_inputs(m, n, k, seed=2)
        d = run(r, a, b, c, m, n, k, 1.0, 0.0)
        assert r.info("last_variant") == want, (m, n, k)
        check(d, a, b, c, m, n, k, 1.0, 0.0)
    from runner import api
    with pytest.raises(api.SgemmError) as e:             # an FFMA-only cubin has no companion to force
        run(runner_of("simt_128x128x16"), a, b, c, m, n, k, force=SKINNY)
    assert e.value.code == -6


def test_variant_selection(runner_of):
    r = runner_of("tc_128x256x32_s2")
    for (m, n, k), want in [((32, 32, 32), SIMT), ((127, 257, 513), SIMT), ((1000, 1000, 1000), TENSOR),
                            ((1024, 1024, 1024), TENSOR)]:
        a, b, c = oracle.make_inputs(m, n, k, seed=1)
        d = run(r, a, b, c, m, n, k, 1.0, 0.0)
        assert r.info("last_variant") == want, (m, n, k)
        check(d, a, b, c, m, n, k, 1.0, 0.0)
    # a forced tensor path on a shape TMA cannot describe goes through aligned copies of the operands; with that
    # switched off it is an error, not a silent fallback
    from runner import api
    a, b, c = oracle.make_inputs(127, 257, 513, seed=1)
    d = run(r, a, b, c, 127, 257, 513, 0.5, 2.0, force=TENSOR)
    assert r.info("last_variant") == TENSOR
    check(d, a, b, c, 127, 257, 513, 0.5, 2.0)
    r.set_option("repitch", 0)
    with pytest.raises(api.SgemmError) as e:
        run(r, a, b, c, 127, 257, 513, force=TENSOR)
    assert e.value.code == -6
    r.set_option("repitch", 1)
    with pytest.raises(api.SgemmError) as e:  # lda smaller than M
        r.run_host(a, b, None, np.zeros(127 * 257, np.float32), 127, 257, 513, lda=100)
    assert e.value.code == -1


def test_unaligned_base_pointers_take_the_simt_kernel(runner_of):
    # TMA needs 16-byte aligned operand bases: a buffer that starts 4 bytes into an allocation is served by the
    # FFMA kernel of the same cubin, and forcing the tensor path on it is refused.
    from runner import api
    m, n, k = 512, 512, 512
    a, b, c = oracle.make_inputs(m, n, k, seed=3)
    r = runner_of("tc2_256x256x32_s3")
    pa, pb, pd = r.dev_alloc(a.nbytes + 16), r.dev_alloc(b.nbytes + 16), r.dev_alloc(m * n * 4)
    try:
        r.upload(pa + 4, a)
        r.upload(pb, b)
        r.launch(pa + 4, pb, None, pd, m, n, k)
        assert r.info("last_variant") == SIMT
        got = np.empty(m * n, np.float32)
        r.sync()
        r.download(got, pd)
        check(got, a, b, None, m, n, k, 1.0, 0.0)
        r.set_option("force_variant", TENSOR)        # forced: the tensor kernel on an aligned copy of A
        r.launch(pa + 4, pb, None, pd, m, n, k)
        assert r.info("last_variant") == TENSOR
        r.sync()
        r.download(got, pd)
        check(got, a, b, None, m, n, k, 1.0, 0.0)
        r.set_option("repitch", 0)                   # ... unless copies are switched off: then it is refused
        with pytest.raises(api.SgemmError) as e:
            r.launch(pa + 4, pb, None, pd, m, n, k)
        assert e.value.code == -6
        r.set_option("repitch", 1)
        r.set_option("force_variant", AUTO)
        r.launch(pa, pb, None, pd, m, n, k)          # aligned: tensor path (A's content is shifted, only the variant matters)
        assert r.info("last_variant") == TENSOR
    finally:
        r.sync()
        for p in (pa, pb, pd):
            r.dev_free(p)


# ----------------------------------------------------------------- the skinny benchmark shapes, full oracle
@pytest.mark.parametrize("mnk", [(8192, 8192, 256), (4096, 128, 16384)])
def test_skinny_shapes_full_oracle(runner_of, mnk):
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=0)
    r = runner_of("tc_128x256x32_s2")
    d = run(r, a, b, c, m, n, k, 1.0, 0.0)
    assert r.info("last_variant") == TENSOR
    if mnk == (4096, 128, 16384):
        assert r.info("last_split_k") > 1   # 32 output tiles for 148 SMs: K must be cut
    check(d, a, b, c, m, n, k, 1.0, 0.0)
    d2 = run(r, a, b, c, m, n, k, 1.0, 0.0)
    assert d.tobytes() == d2.tobytes()      # bit-reproducible, split-K included
    ds = run(runner_of("simt_128x128x16"), a, b, c, m, n, k, 1.0, 0.0, force=SIMT)
    check(ds, a, b, c, m, n, k, 1.0, 0.0)


# ------------------------------------------------ 8192^3: column-sampled oracle + a checksum over every tile
@pytest.mark.parametrize("kernel,force", [("tc_128x256x32_s2", TENSOR), ("simt_128x128x16", SIMT)])
def test_8192_cubed_sampled_and_checksummed(runner_of, kernel, force):
    m = n = k = 8192
    a, b, c = oracle.make_inputs(m, n, k, seed=0)
    r = runner_of(kernel)
    d = run(r, a, b, c, m, n, k, 1.0, 0.0, force=force)
    D = d.reshape(n, m)                                    # row j = column j of D
    # (1) exact oracle on 96 sampled columns (every tile column of the 256-wide tiling is hit)
    cols = np.unique(np.concatenate([np.arange(0, n, 128) + 7, np.array([0, 1, 255, 256, n - 1])]))
    b_sub = np.ascontiguousarray(b.reshape(n, k)[cols]).reshape(-1)
    ref = oracle.gemm(a, b_sub, None, 1.0, 0.0, m, len(cols), k)
    bound = oracle.abs_bound(a, b_sub, m, len(cols), k)
    assert oracle.worst_ratio(np.ascontiguousarray(D[cols]).reshape(-1), ref, bound) <= 1.0
    # (2) linearity checksum over ALL of D: D @ 1 = A @ (B @ 1), in FP64, bounded by |A| @ (|B| @ 1) * 1e-5
    A = a.reshape(k, m).astype(np.float64)
    Bm = b.reshape(n, k).astype(np.float64)
    rowsum = D.astype(np.float64).sum(axis=0)
    want = Bm.sum(axis=0) @ A
    slack = oracle.REL_TOL * (np.abs(Bm).sum(axis=0) @ np.abs(A))
    assert np.all(np.abs(rowsum - want) <= slack)
    colsum = D.astype(np.float64).sum(axis=1)
    want_c = Bm @ A.sum(axis=1)
    slack_c = oracle.REL_TOL * (np.abs(Bm) @ np.abs(A).sum(axis=1))
    assert np.all(np.abs(colsum - want_c) <= slack_c)


# ------------------------------------------------------------------------------ determinism and split-K
@pytest.mark.parametrize("kernel,force", [("tc_128x128x32_s3", TENSOR), ("simt_64x64x16", SIMT)])
def test_split_k_is_deterministic_and_in_tolerance(runner_of, kernel, force):
    m, n, k = 200, 136, 4096
    lda, ldb = 200, 4096
    a, b, c = oracle.make_inputs(m, n, k, seed=7)
    r = runner_of(kernel)
    outs = {}
    for split in (1, 3, 4, 16):
        d1 = run(r, a, b, c, m, n, k, 2.0, 1.0, force=force, split_k=split)
        assert r.info("last_split_k") <= split
        d2 = run(r, a, b, c, m, n, k, 2.0, 1.0, force=force, split_k=split)
        assert d1.tobytes() == d2.tobytes()
        check(d1, a, b, c, m, n, k, 2.0, 1.0)
        outs[split] = d1
    assert r.info("last_split_k") > 1


def test_split_k_beyond_the_k_blocks_is_clamped(runner_of):
    m, n, k = 64, 64, 40
    a, b, c = oracle.make_inputs(m, n, k, seed=2)
    for kernel, force in (("tc_128x128x32_s3", TENSOR), ("simt_64x64x16", SIMT)):
        r = runner_of(kernel)
        d = run(r, a, b, c, m, n, k, 1.0, 0.0, force=force, split_k=64)
        assert 1 <= r.info("last_split_k") <= 3
        check(d, a, b, c, m, n, k, 1.0, 0.0)


# -------------------------------------------------------------------------- leading dimensions, canaries
@pytest.mark.parametrize("kernel,force", [("tc_128x256x32_s2", TENSOR), ("tc_128x128x32_s3_ak", TENSOR),
                                          ("simt_128x128x16", SIMT)])
def test_leading_dimensions_and_untouched_padding(runner_of, kernel, force):
    m, n, k = 300, 270, 200
    lda, ldb, ldc, ldd = 304, 208, 301, 303
    a, b, c = oracle.make_inputs(m, n, k, seed=9, lda=lda, ldb=ldb, ldc=ldc)
    canary = np.full(ldd * n, np.float32(-777.25))
    r = runner_of(kernel)
    d = run(r, a, b, c, m, n, k, 1.0, 1.0, force=force, lda=lda, ldb=ldb, ldc=ldc, ldd=ldd, d_init=canary)
    check(d, a, b, c, m, n, k, 1.0, 1.0, lda=lda, ldb=ldb, ldc=ldc, ldd=ldd)
    pad = d.reshape(n, ldd)[:, m:]
    assert np.all(pad == np.float32(-777.25))   # rows >= M of every column keep the caller's bytes


@pytest.mark.parametrize("mnk", [(70001, 3, 5), (3, 70001, 5), (5, 7, 100003), (1, 65537, 1), (262147, 1, 2)])
def test_extreme_aspect_ratios(runner_of, mnk):
    # one dimension far beyond 65535 (the old grid-dimension limit) and the others tiny
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=17)
    for kernel in ("tc2_256x256x32_s3", "simt_128x128x16"):
        d = run(runner_of(kernel), a, b, c, m, n, k, 1.0, 1.0)
        check(d, a, b, c, m, n, k, 1.0, 1.0)


def test_degenerate_sizes(runner_of):
    for kernel in ("tc_128x128x32_s3", "simt_64x64x16"):
        r = runner_of(kernel)
        c = oracle.fill_uniform(12, 5)
        d = np.full(12, np.float32(9.0))
        r.run_host(None, None, c, d, 4, 3, 0, alpha=1.0, beta=2.0, lda=4, ldb=1)   # K = 0: D = beta*C
        assert np.array_equal(d, np.float32(2.0) * c)
        r.run_host(None, None, None, d, 4, 3, 0, alpha=1.0, beta=0.0, lda=4, ldb=1)
        assert np.all(d == 0.0)
        r.run_host(None, None, None, d, 0, 3, 5, lda=1, ldb=5, ldc=1, ldd=1)        # M = 0: nothing to do
        r.run_host(None, None, None, d, 4, 0, 5, lda=4, ldb=5)                      # N = 0


def test_beta_zero_never_reads_c(runner_of):
    m, n, k = 160, 96, 64
    a, b, _ = oracle.make_inputs(m, n, k, seed=4)
    for kernel, force in (("tc_128x128x32_s3", TENSOR), ("simt_64x64x16", SIMT)):
        d = run(runner_of(kernel), a, b, None, m, n, k, 1.0, 0.0, force=force)   # C = NULL
        check(d, a, b, None, m, n, k, 1.0, 0.0)


# ------------------------------------------------------------------------- seeded random sweep of the API
def test_random_shapes_layouts_and_options(runner_of):
    # 80 seeded cases: random sizes (ragged on purpose), leading-dimension padding, alpha/beta, kernel and variant;
    # every one against the oracle, a few also for run-to-run bit equality
    rng = np.random.default_rng(20240607)
    pool = ["tc2_256x256x32_s3", "tc_128x256x32_s2", "tc_128x128x16_s7", "tc2i_256x256x32_s3", "tc2h_256x256x32_s3", "tc2_256x256x32_s3_tt",
            "tc2_256x256x32_s3_tn", "simt_128x128x16", "simt_64x64x16_tt", "legacy_32x32x2_1wave"]
    for case in range(80):
        kernel = pool[int(rng.integers(len(pool)))]
        ta, tb = kernel.endswith(("_tt", "_tn")), kernel.endswith(("_tt", "_nt"))
        m, n, k = (int(rng.integers(1, 700)) for _ in range(3))
        if case % 7 == 0:
            k = int(rng.integers(2000, 6000))               # long K: split-K territory
        alpha = float(rng.choice([1.0, -0.5, 2.25]))
        beta = float(rng.choice([0.0, 0.0, 1.0, -1.75]))
        tensor_cubin = kernel.startswith("tc")
        pad4 = lambda x: (x + 3) // 4 * 4
        extra = int(rng.choice([0, 0, 4, 12]))
        a, b, c = oracle.make_inputs(m, n, k, seed=1000 + case)
        sa, lda = stored(a, m, k, ta, (pad4(k if ta else m) + extra) if tensor_cubin else 0)
        sb, ldb = stored(b, k, n, tb, (pad4(n if tb else k) + extra) if tensor_cubin else 0)
        ldd = m + int(rng.choice([0, 0, 3]))
        force = int(rng.choice([AUTO, TENSOR, SIMT, SKINNY])) if tensor_cubin else SIMT
        split = int(rng.choice([0, 0, 1, 3]))
        r = runner_of(kernel)
        d = run(r, sa, sb, c, m, n, k, alpha, beta, force=force, split_k=split, lda=lda, ldb=ldb, ldd=ldd)
        check(d, a, b, c, m, n, k, alpha, beta, ldd=ldd)
        if case % 5 == 0:
            d2 = run(r, sa, sb, c, m, n, k, alpha, beta, force=force, split_k=split, lda=lda, ldb=ldb, ldd=ldd)
            assert d.tobytes() == d2.tobytes(), (case, kernel, m, n, k)


# ------------------------------------------------------------------------------------------ transposes
@pytest.mark.parametrize("kernel,ta,tb", [
    ("tc2_256x256x32_s3_tn", True, False), ("tc2_256x256x32_s3_nt", False, True), ("tc2_256x256x32_s3_tt", True, True),
    ("tc_128x128x32_s3_tt", True, True), ("tc2i_256x256x32_s3_tt", True, True),
    ("simt_128x128x16_tn", True, False), ("simt_128x128x16_nt", False, True), ("simt_64x64x16_tt", True, True)])
@pytest.mark.parametrize("mnk", [(32, 32, 32), (129, 255, 33), (300, 520, 1000), (1024, 768, 512), (4, 300, 77)])
@pytest.mark.parametrize("padded", [False, True])
def test_transposed_operands(runner_of, kernel, ta, tb, mnk, padded):
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=31)
    a_rows, b_rows = (k if ta else m), (n if tb else k)           # contiguous extent of A and B as stored
    pad = lambda x: (x + 3) // 4 * 4 + (8 if padded else 0)
    tensor = kernel.startswith("tc")
    sa, lda = stored(a, m, k, ta, pad(a_rows) if (tensor or padded) else 0)
    sb, ldb = stored(b, k, n, tb, pad(b_rows) if (tensor or padded) else 0)
    r = runner_of(kernel)
    d = run(r, sa, sb, c, m, n, k, 1.25, 0.5, force=TENSOR if tensor else SIMT, lda=lda, ldb=ldb)
    assert r.info("last_variant") == (TENSOR if tensor else SIMT)
    check(d, a, b, c, m, n, k, 1.25, 0.5)      # against the NN oracle on the logical matrices
    if tensor:                                  # the FFMA kernel inside the same cubin follows the same flags
        d2 = run(r, sa, sb, c, m, n, k, 1.25, 0.5, force=SIMT, lda=lda, ldb=ldb)
        check(d2, a, b, c, m, n, k, 1.25, 0.5)


def test_transposed_leading_dimension_checks(runner_of):
    from runner import api
    m, n, k = 64, 96, 128
    a, b, c = oracle.make_inputs(m, n, k, seed=1)
    r = runner_of("tc2_256x256x32_s3_tt")
    with pytest.raises(api.SgemmError) as e:       # A is stored K x M: lda must cover K, not M
        r.run_host(a, b, None, np.zeros(m * n, np.float32), m, n, k, lda=m, ldb=n)
    assert e.value.code == -1
    with pytest.raises(api.SgemmError) as e:       # B is stored N x K: ldb must cover N
        r.run_host(a, b, None, np.zeros(m * n, np.float32), m, n, k, lda=k, ldb=64)
    assert e.value.code == -1


# ------------------------------------------------------------------------------------ pipelined host path
@pytest.mark.parametrize("kernel,force", [("tc2_256x256x32_s3", AUTO), ("tc_128x128x32_s3_ak", TENSOR), ("tc2h_256x256x32_s3", TENSOR),
                                          ("simt_128x128x16", SIMT)])
@pytest.mark.parametrize("beta,ldd", [(0.0, 0), (0.75, 2052)])
def test_pipelined_host_call_equals_the_single_launch(runner_of, kernel, force, beta, ldd):
    # sgemm_run_host overlaps uploads, GEMM and downloads over column chunks for large problems; chunking must not
    # change a single bit of D (same kernel, same split-K partition per element), padding rows included
    m, n, k = 2048, 4096 + 96, 2048          # a ragged last chunk
    a, b, c = oracle.make_inputs(m, n, k, seed=23)
    canary = np.full((ldd or m) * n, np.float32(3.5))
    r = runner_of(kernel)
    outs = []
    for pipelined in (1, 0):
        r.set_option("pipeline_host", pipelined)
        launches = r.info("launches")
        outs.append(run(r, a, b, c, m, n, k, 1.0, beta, force=force, ldd=ldd, d_init=canary))
        count = r.info("launches") - launches
        assert (count > 3) == bool(pipelined)      # eight chunks against one launch chain
    r.set_option("pipeline_host", 1)
    assert outs[0].tobytes() == outs[1].tobytes()
    check(outs[0], a, b, c, m, n, k, 1.0, beta, ldd=ldd)


# ------------------------------------------------------------------------------------ workspace handling
def test_lent_workspace(runner_of):
    from runner import api
    m, n, k = 256, 256, 2048
    a, b, c = oracle.make_inputs(m, n, k, seed=6)
    r = runner_of("tc_128x128x32_s3")
    base = run(r, a, b, c, m, n, k, 1.0, 0.0, force=TENSOR, split_k=4)
    r.set_option("force_variant", TENSOR)
    r.set_option("split_k", 4)
    need = r.workspace_bytes(m, n, k)
    assert need >= (m * k + k * n + 4 * m * n) * 4
    ws = r.dev_alloc(need)
    try:
        r.set_workspace(ws, need)
        lent = run(r, a, b, c, m, n, k, 1.0, 0.0, force=TENSOR, split_k=4)
        assert lent.tobytes() == base.tobytes()
        r.set_workspace(ws, need - 256)
        with pytest.raises(api.SgemmError) as e:
            run(r, a, b, c, m, n, k, 1.0, 0.0, force=TENSOR, split_k=4)
        assert e.value.code == -7
    finally:
        r.set_workspace(None, 0)
        r.sync()
        r.dev_free(ws)


# ------------------------------------------------------------------------------------ failure detection
def test_bounded_wait_runs_out_reports_and_leaves_the_context_usable(built):
    # A wait whose barrier nothing completes must give up after its limit, record the status words and return:
    # the host sees SGEMM_ERR_DEVICE_STATUS with the tag, the status is cleared by the read, and the same handle
    # computes correctly afterwards.  (The waiting kernel is a one-block self-test around the GEMM kernel's own
    # wait routine; no pipeline is left hanging behind it.)
    from runner import api
    cubin, toml = built.ensure("tc2_256x256x32_s3")
    with api.SgemmRunner(cubin, toml, 0) as r:
        assert r.last_status()[0] == 0
        r.wait_selftest(timeout_ms=20, tag=0x51DE)
        with pytest.raises(api.SgemmError) as e:
            r.last_status()
        assert e.value.code == -8 and "0x51de" in str(e.value)
        assert r.last_status()[0] == 0                       # cleared by the failing read
        m, n, k = 300, 260, 520
        a, b, c = oracle.make_inputs(m, n, k, seed=5, lda=300, ldb=520)
        d = run(r, a, b, c, m, n, k, 1.0, 1.0, force=TENSOR, split_k=2)
        check(d, a, b, c, m, n, k, 1.0, 1.0)
        assert r.last_status()[0] == 0
    cubin, toml = built.ensure("ffma_tma_256x128x16_s4")     # the TMA-fed FFMA kernel has its own copy of the wait routine
    with api.SgemmRunner(cubin, toml, 0) as r:
        r.wait_selftest(timeout_ms=20, tag=0x51DF)
        with pytest.raises(api.SgemmError) as e:
            r.last_status()
        assert e.value.code == -8 and "0x51df" in str(e.value)
        assert r.last_status()[0] == 0
        m, n, k = 300, 260, 520
        a, b, c = oracle.make_inputs(m, n, k, seed=5, lda=300, ldb=520)
        d = run(r, a, b, c, m, n, k, 1.0, 1.0, force=SIMT, split_k=2)
        assert r.info("last_feed_tma") == 1
        check(d, a, b, c, m, n, k, 1.0, 1.0, lda=300, ldb=520)
        assert r.last_status()[0] == 0
    cubin, toml = built.ensure("simt_128x128x16")
    with api.SgemmRunner(cubin, toml, 0) as r:               # a register-fed FFMA cubin has no bounded waits
        with pytest.raises(api.SgemmError) as e:
            r.wait_selftest()
        assert e.value.code == -6


# ------------------------------------------------------------------------------ helpers on the device
def test_device_fill_equals_host_generator(runner_of):
    r = runner_of("simt_64x64x16")
    count = 1_000_003
    p = r.dev_alloc(count * 4)
    try:
        r.fill_uniform(p, count, stream_id=3, first_index=12345)
        got = np.empty(count, dtype=np.float32)
        r.download(got, p)
        assert got.tobytes() == oracle.fill_uniform(count, 3, first_index=12345).tobytes()
    finally:
        r.dev_free(p)


@pytest.mark.parametrize("kernel", ["tc_128x256x32_s2", "simt_64x64x16", "legacy_32x32x2_1wave"])
def test_tile_rasterisation_on_device_matches_the_model(runner_of, built, kernel):
    from generator import generator as g
    wgm = built.REGISTRY[kernel][1].get("wgm", 1)
    r = runner_of(kernel)
    for nx, ny in [(8, 8), (7, 5), (64, 32), (1, 9)]:
        assert r.tile_map(nx, ny) == [g.tile_raster(z, nx, ny, wgm) for z in range(nx * ny)]


# ------------------------------------------------------------------------------------------ C and D aliased
@pytest.mark.parametrize("kernel,force", [("tc2_256x256x32_s3", TENSOR), ("tc2_256x256x32_s3_c0", TENSOR),
                                          ("tc2_256x256x32_s3", SKINNY), ("simt_128x128x16", SIMT)])
@pytest.mark.parametrize("mnk,split_k", [((300, 520, 1100), 1), ((300, 520, 200), 1), ((260, 132, 1100), 3)])
def test_in_place_update_c_is_d(runner_of, kernel, force, mnk, split_k):
    """D = alpha*A*B + beta*D with C and D the same device buffer (BLAS semantics; the reference's runner keeps them
    apart): every element of C is read by the thread that later overwrites it, before it does so."""
    m, n, k = mnk
    lda, ldb = (m + 3) // 4 * 4, (k + 3) // 4 * 4
    a, b, c = oracle.make_inputs(m, n, k, seed=11, lda=lda, ldb=ldb)
    r = runner_of(kernel)
    r.set_option("force_variant", force)
    r.set_option("split_k", split_k)
    da, db, dd = r.dev_alloc(a.nbytes), r.dev_alloc(b.nbytes), r.dev_alloc(c.nbytes)
    try:
        r.upload(da, a); r.upload(db, b); r.upload(dd, c)
        r.launch(da, db, dd, dd, m, n, k, alpha=0.75, beta=-1.25, lda=lda, ldb=ldb)
        r.sync()
        d = np.empty_like(c)
        r.download(d, dd)
    finally:
        for p in (da, db, dd):
            r.dev_free(p)
    assert r.last_status()[0] == 0
    check(d, a, b, c, m, n, k, 0.75, -1.25, lda=lda, ldb=ldb)


# --------------------------------------------------------------- operands TMA cannot describe, at tensor speed
@pytest.mark.parametrize("kernel", ["tc2_256x256x32_s3", "tc2i_256x256x32_s3", "tc_128x128x32_s3_ak", "tc2_256x256x32_s3_tt",
                                    "tc2_256x256x32_s3_tn"])
@pytest.mark.parametrize("mnk", [(1031, 1027, 1029), (515, 2050, 1023)])
def test_ragged_leading_dimensions_run_on_the_tensor_path(runner_of, kernel, mnk):
    """Natural (odd) leading dimensions: in auto mode a problem of this size is served by the tensor kernel through
    aligned copies of the operands (one more pass over them), not by the four times slower FFMA kernel."""
    m, n, k = mnk
    ta, tb = kernel.endswith(("_tt", "_tn")), kernel.endswith(("_tt", "_nt"))
    a, b, c = oracle.make_inputs(m, n, k, seed=13)
    sa, lda = stored(a, m, k, ta)
    sb, ldb = stored(b, k, n, tb)
    r = runner_of(kernel)
    d = run(r, sa, sb, c, m, n, k, 0.75, -1.25, force=AUTO, lda=lda, ldb=ldb)
    assert r.info("last_variant") == TENSOR and r.last_status()[0] == 0
    check(d, a, b, c, m, n, k, 0.75, -1.25)
    d2 = run(r, sa, sb, c, m, n, k, 0.75, -1.25, force=AUTO, lda=lda, ldb=ldb)
    assert np.array_equal(d, d2)


# ------------------------------------------------------------------ a few columns: the companion's 32-column tiles
@pytest.mark.parametrize("kernel", ["tc2_256x256x32_s3", "tc2_256x256x32_s3_tt"])
@pytest.mark.parametrize("mnk,tile_n", [((8192, 8, 1024), 32), ((3000, 32, 4096), 32), ((16384, 1, 8192), 32), ((2048, 33, 2048), 128),
                                        ((4096, 128, 1024), 128)])
def test_thin_problems_take_the_narrow_companion(runner_of, kernel, mnk, tile_n):
    m, n, k = mnk
    ta = tb = kernel.endswith("_tt")
    r = runner_of(kernel)
    r.set_option("skinny_below_intensity", 200)      # the library's default rule
    lda, ldb = ((k if ta else m) + 3) // 4 * 4, ((n if tb else k) + 3) // 4 * 4
    a, b, c = oracle.make_inputs(m, n, k, seed=17)
    sa, lda = stored(a, m, k, ta, ld=lda)
    sb, ldb = stored(b, k, n, tb, ld=ldb)
    d = run(r, sa, sb, c, m, n, k, 0.5, -1.5, force=AUTO, lda=lda, ldb=ldb)
    assert r.info("last_variant") == SKINNY and r.info("last_tile_n") == tile_n
    check(d, a, b, c, m, n, k, 0.5, -1.5)


def test_pipelined_host_call_with_ragged_leading_dimensions(runner_of):
    """Large host call with natural odd leading dimensions: column chunks on three streams, every chunk through aligned
    copies of its operands, the copy of A made once and reused by the later (and narrower, last) chunks."""
    m, n, k = 2049, 4100, 2049
    a, b, c = oracle.make_inputs(m, n, k, seed=19)
    r = runner_of("tc2_256x256x32_s3")
    d = run(r, a, b, c, m, n, k, 1.0, 0.5, force=AUTO)
    assert r.info("last_variant") == TENSOR and r.last_status()[0] == 0
    check(d, a, b, c, m, n, k, 1.0, 0.5)
    r.set_option("pipeline_host", 0)
    d1 = run(r, a, b, c, m, n, k, 1.0, 0.5, force=AUTO)
    r.set_option("pipeline_host", 1)
    assert np.array_equal(d, d1)          # the chunked call computes what the single launch computes
