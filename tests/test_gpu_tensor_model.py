"""The device against the host model of its arithmetic (oracle/tensor_model.py): not "within tolerance" but equal as
FP32 values, element for element — the check the reference makes possible with its instruction-level VM
(test/test_vm.py:447-627), here for the tcgen05 3xTF32 kernels, the FFMA kernels and the split-K path."""
import numpy as np
import pytest

import tensor_cases
from oracle import tensor_model
from test_gpu_parity import AUTO, SIMT, SKINNY, TENSOR, run, runner_of, stored  # noqa: F401  (runner_of is a fixture)

pytestmark = pytest.mark.gpu


def colmajor(mat):
    return np.ascontiguousarray(mat.T, dtype=np.float32).reshape(-1)


def as_matrix(flat, rows, cols):
    return flat[: rows * cols].reshape(cols, rows).T


def test_recorded_cases_model_and_device_agree(runner_of, golden_dir):
    recorded = np.load(golden_dir / "tcgen05_recorded.npz")
    runners = {1: runner_of("tc_128x128x32_s3_1x"), 3: runner_of("tc2_256x256x32_s3_c0")}   # whole K in one chain
    for name, (a_mat, b_mat, terms) in tensor_cases.cases().items():
        m, k = a_mat.shape
        n = b_mat.shape[1]
        d = as_matrix(run(runners[terms], colmajor(a_mat), colmajor(b_mat), None, m, n, k, force=TENSOR, split_k=1), m, n)
        assert np.array_equal(d, recorded[name]), f"{name}: the device no longer returns what was recorded"
        assert np.array_equal(d, tensor_model.accumulate(a_mat, b_mat, terms)), f"{name}: model and device differ"


def test_hand_examples_on_the_device(runner_of):
    """The rules the model states, one tiny GEMM each: row 0 of a 4 x 8 A times column 0 of an 8 x 4 B."""
    r = runner_of("tc_128x128x32_s3_1x")
    for a_row, b_col, expected, rule in tensor_cases.hand_examples():
        a_mat, b_mat = np.zeros((4, 8), np.float32), np.zeros((8, 4), np.float32)
        a_mat[0, :len(a_row)] = a_row
        b_mat[:len(b_col), 0] = b_col
        d = as_matrix(run(r, colmajor(a_mat), colmajor(b_mat), None, 4, 4, 8, force=TENSOR, split_k=1), 4, 4)
        assert float(d[0, 0]) == expected, rule


TENSOR_CASES = [("tc2_256x256x32_s3", TENSOR), ("tc2_256x256x32_s3_c0", TENSOR), ("tc_128x256x32_s2", TENSOR), ("tc_128x128x16_s7", TENSOR),
                ("tc2i_256x256x32_s3", TENSOR), ("tc2h_256x256x32_s3", TENSOR), ("tc_128x128x32_s3_ak", TENSOR), ("tc2_256x256x32_s3_e4", TENSOR),
                ("tc2_256x256x32_s3", SKINNY), ("tc2_256x256x32_s3_tt", TENSOR), ("tc2_256x256x32_s3_tn", TENSOR)]


@pytest.mark.parametrize("kernel,force", TENSOR_CASES)
@pytest.mark.parametrize("mnk", [(96, 80, 72), (130, 4, 300), (257, 129, 65), (200, 136, 520)])
@pytest.mark.parametrize("alpha,beta,split_k,chain", [(1.0, 0.0, 1, -1), (0.75, -1.25, 1, -1), (-2.5, 0.3, 3, -1),
                                                       (0.75, -1.25, 1, 64), (1.0, 0.5, 2, 0)])
def test_tensor_kernels_equal_the_model_bit_for_bit(runner_of, kernel, force, mnk, alpha, beta, split_k, chain):
    m, n, k = mnk
    ta = kernel.endswith("_tt") or kernel.endswith("_tn")
    tb = kernel.endswith("_tt") or kernel.endswith("_nt")
    a_mat = tensor_cases.uniform((m, k), 7 * m + k)
    b_mat = tensor_cases.uniform((k, n), 7 * n + k + 1)
    c_mat = tensor_cases.uniform((m, n), m + n + k)
    # operands as stored: 16-byte pitches for the tensor maps
    a, lda = stored(colmajor(a_mat), m, k, ta, ld=((k if ta else m) + 3) // 4 * 4)
    b, ldb = stored(colmajor(b_mat), k, n, tb, ld=((n if tb else k) + 3) // 4 * 4)
    r = runner_of(kernel)
    if chain > 0 and r.info("skinny_acc_chain" if force == SKINNY else "acc_chain") == 0:
        with pytest.raises(Exception, match="without chunked accumulation"):
            r.set_option("acc_chain", chain)
            try:
                run(r, a, b, colmajor(c_mat), m, n, k, alpha, beta, force=force, split_k=split_k, lda=lda, ldb=ldb)
            finally:
                r.set_option("acc_chain", -1)
        return
    r.set_option("acc_chain", chain)    # -1: as generated, 0: one chain, else k per chain
    try:
        d = run(r, a, b, colmajor(c_mat), m, n, k, alpha, beta, force=force, split_k=split_k, lda=lda, ldb=ldb)
    finally:
        r.set_option("acc_chain", -1)
    assert r.info("last_variant") == force
    used_split = r.info("last_split_k")
    bk = 32 if force == SKINNY else int(kernel.split("_")[1].split("x")[2])
    # the runner reports the chain it launched with: the requested one, or 0 when the whole-K twin of the main kernel
    # served a problem of at most two chains
    per_unit = tensor_model.split_ranges(k, bk, used_split)[0][1]      # k range of one launch unit
    assert chain < 0 or r.info("last_acc_chain") == (0 if force == TENSOR and per_unit <= 2 * chain else chain)
    want = tensor_model.gemm(a_mat, b_mat, c_mat, alpha, beta, terms=3, split_k=used_split, bk=bk,
                             chain=r.info("last_acc_chain"))
    assert np.array_equal(as_matrix(d, m, n), want)


@pytest.mark.parametrize("kernel,bk", [("simt_128x128x16", 16), ("simt_64x64x16", 16), ("simt_128x64x8_plr0", 8),
                                       ("legacy_32x32x2_1wave", None), ("simt_64x64x16_tt", 16),
                                       ("ffma_tma_128x128x16_s4", 16), ("ffma_tma_256x128x32_s3", 32)])   # (TMA-fed where lda, ldb allow)
@pytest.mark.parametrize("mnk", [(96, 80, 72), (33, 65, 129), (130, 4, 300)])
@pytest.mark.parametrize("alpha,beta,split_k", [(1.0, 0.0, 1), (0.75, -1.25, 1), (-2.5, 0.3, 3)])
def test_simt_kernels_equal_the_fma_chain_bit_for_bit(runner_of, built, kernel, bk, mnk, alpha, beta, split_k):
    m, n, k = mnk
    t = kernel.endswith("_tt")
    if bk is None:
        from runner import api
        bk = api.parse_config(built.ensure(kernel)[1]).depth_k
    a_mat = tensor_cases.uniform((m, k), 3 * m + k)
    b_mat = tensor_cases.uniform((k, n), 3 * n + k + 1)
    c_mat = tensor_cases.uniform((m, n), m + n + k + 2)
    a, lda = stored(colmajor(a_mat), m, k, t)
    b, ldb = stored(colmajor(b_mat), k, n, t)
    r = runner_of(kernel)
    d = run(r, a, b, colmajor(c_mat), m, n, k, alpha, beta, force=SIMT, split_k=split_k, lda=lda, ldb=ldb)
    if kernel.startswith("ffma_tma") and not r.info("last_feed_tma"):
        bk = 16   # operands TMA cannot describe ran on the cubin's register-fed kernel, whose k per stage cuts the splits
    want = tensor_model.simt_gemm(a_mat, b_mat, c_mat, alpha, beta, split_k=r.info("last_split_k"), bk=bk)
    assert np.array_equal(as_matrix(d, m, n), want)


def test_same_signed_inputs_need_the_chunked_accumulation(runner_of):
    """With inputs of one sign nothing cancels, and the truncating adds of one long tensor-core chain all err the same
    way: at K = 8192 the whole-K kernel misses the parity bound by an order of magnitude, the chunked kernel (chains
    of 128, added in FP32 with round-to-nearest) stays well inside it."""
    from oracle import oracle
    m, n, k = 256, 256, 8192
    a, b, _ = oracle.make_inputs(m, n, k, seed=3)
    a, b = np.abs(a), np.abs(b)
    ref = oracle.gemm(a, b, None, 1.0, 0.0, m, n, k)
    bound = oracle.abs_bound(a, b, m, n, k)
    whole = oracle.worst_ratio(run(runner_of("tc2_256x256x32_s3_c0"), a, b, None, m, n, k, force=TENSOR, split_k=1), ref, bound)
    chunked = oracle.worst_ratio(run(runner_of("tc2_256x256x32_s3"), a, b, None, m, n, k, force=TENSOR, split_k=1), ref, bound)
    assert chunked <= 1.0, chunked
    assert whole > 5.0, whole
    # against the exact product (FP64) the chunked kernel is closer than the FP32 oracle's own sequential sum
    exact = a.reshape(k, m).T.astype(np.float64) @ b.reshape(n, k).T.astype(np.float64)
    got = run(runner_of("tc2_256x256x32_s3"), a, b, None, m, n, k, force=TENSOR, split_k=1).reshape(n, m).T
    assert float((np.abs(got - exact) / (1e-5 * exact)).max()) <= 0.4
    print(f"same-signed inputs, K = {k}: worst ratio {whole:.2f} (one chain) -> {chunked:.3f} (chains of 128)")


@pytest.mark.parametrize("kernel", ["bf16_tc2_256x256x64_s6", "fp16_tc_128x128x64_s4", "bf16_tc_128x256x32_s4_tn",
                                    "fp16_tc2_256x128x64_s4_tn"])
@pytest.mark.parametrize("mnk", [(96, 80, 72), (257, 129, 520), (64, 40, 2300)])
@pytest.mark.parametrize("alpha,beta,split_k,chain", [(1.0, 0.0, 1, -1), (0.75, -1.25, 1, 128), (-2.5, 0.3, 3, -1)])
def test_half_operand_kernels_equal_the_model_bit_for_bit(runner_of, kernel, mnk, alpha, beta, split_k, chain):
    """kind::f16 uses the same adder with 16 products per instruction: the model with mma_k = 16 on the operand values
    (FP16 / BF16 numbers, which the TF32 cut leaves untouched) predicts the device exactly."""
    from test_gpu_half_operands import narrow, stored16
    m, n, k = mnk
    kind, trans_a = kernel.split("_")[0], kernel.endswith("_tn")
    a_bits, a_val = narrow(tensor_cases.uniform((m, k), 5 * m + k), kind)
    b_bits, b_val = narrow(tensor_cases.uniform((k, n), 5 * n + k + 1), kind)
    c_mat = tensor_cases.uniform((m, n), m + n + k)
    lda, ldb = ((k if trans_a else m) + 7) // 8 * 8, (k + 7) // 8 * 8
    r = runner_of(kernel)
    r.set_option("force_variant", AUTO)
    r.set_option("split_k", split_k)
    r.set_option("acc_chain", chain)
    d = np.zeros(m * n, dtype=np.float32)
    try:
        flat16 = lambda bits: np.ascontiguousarray(bits.T).reshape(-1)  # noqa: E731  (column-major words of an m x k array)
        r.run_host(stored16(flat16(a_bits), m, k, trans_a, lda), stored16(flat16(b_bits), k, n, False, ldb),
                   colmajor(c_mat), d, m, n, k, alpha=alpha, beta=beta, lda=lda, ldb=ldb)
    finally:
        r.set_option("acc_chain", -1)
    bk = int(kernel.split("_")[2].split("x")[2])
    want = tensor_model.gemm(a_val, b_val, c_mat, alpha, beta, terms=1, split_k=r.info("last_split_k"), bk=bk,
                             chain=r.info("last_acc_chain"), mma_k=16)
    assert np.array_equal(as_matrix(d, m, n), want)
