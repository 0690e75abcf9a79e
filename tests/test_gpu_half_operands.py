"""FP16 / BF16 operands on the tensor-core path (FP32 accumulate, FP32 C and D): the reference plumbs a_type/b_type
through its configuration and TOML (generator/generator.py:816-824, 1001-1004) but implements FP32 only; here the
16-bit types are served by kind::f16 MMAs.  The oracle runs on the same operand values widened to FP32 — the
products of 16-bit values are exact in FP32, so the same parity bound applies."""
import numpy as np
import pytest

from oracle import oracle
from test_gpu_parity import AUTO, SIMT, TENSOR, runner_of  # noqa: F401  (runner_of is a fixture)

pytestmark = pytest.mark.gpu


def to_bf16_bits(x):
    """FP32 -> BF16 words, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(h):
    return (h.astype(np.uint32) << 16).view(np.float32)


def narrow(x, kind):
    """(16-bit words as uint16, the same values as FP32)."""
    if kind == "bf16":
        bits = to_bf16_bits(x)
        return bits, from_bf16_bits(bits)
    half = np.ascontiguousarray(x, dtype=np.float32).astype(np.float16)
    return half.view(np.uint16), half.astype(np.float32)


def stored16(flat_bits, rows, cols, transposed, ld):
    """Column-major rows x cols matrix of 16-bit words as the kernel expects it (see test_gpu_parity.stored)."""
    mat = flat_bits.reshape(cols, rows)
    if transposed:
        mat = np.ascontiguousarray(mat.T)
    out = np.zeros(mat.shape[0] * ld, dtype=np.uint16)
    out.reshape(mat.shape[0], ld)[:, :mat.shape[1]] = mat
    return out


KERNELS = ["bf16_tc2_256x256x64_s6", "bf16_tc2_256x256x128_s3", "fp16_tc2_256x256x128_s3", "bf16_tc2_256x256x64_s6_ak", "fp16_tc_128x128x64_s4", "bf16_tc_128x256x32_s4_tn", "fp16_tc2_256x128x64_s4_tn",
           "bf16_tc2_256x256x64_s6_tt", "fp16_tc_128x128x64_s4_nt"]


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("mnk", [(8, 8, 8), (96, 80, 72), (129, 255, 33), (256, 512, 96), (1000, 1000, 1000), (130, 4, 2048),
                                 (512, 384, 4096)])
@pytest.mark.parametrize("alpha,beta,split_k", [(1.0, 0.0, 0), (0.5, -1.5, 0), (-2.0, 0.25, 3)])
def test_half_operands_match_oracle(runner_of, kernel, mnk, alpha, beta, split_k):
    m, n, k = mnk
    kind = kernel.split("_")[0]
    trans_a, trans_b = kernel.endswith(("_tn", "_tt")), kernel.endswith(("_nt", "_tt"))
    a32, b32, c = oracle.make_inputs(m, n, k, seed=5)
    a_bits, a_val = narrow(a32, kind)
    b_bits, b_val = narrow(b32, kind)
    lda = ((k if trans_a else m) + 7) // 8 * 8          # 16-byte pitches for the tensor maps (packed copies need none)
    ldb = ((n if trans_b else k) + 7) // 8 * 8
    r = runner_of(kernel)
    r.set_option("force_variant", AUTO)
    r.set_option("split_k", split_k)
    d = np.zeros(m * n, dtype=np.float32)
    r.run_host(stored16(a_bits, m, k, trans_a, lda), stored16(b_bits, k, n, trans_b, ldb), c if beta != 0.0 else None, d,
               m, n, k, alpha=alpha, beta=beta, lda=lda, ldb=ldb)
    assert r.info("last_variant") == TENSOR and r.last_status()[0] == 0
    ref = oracle.gemm(a_val, b_val, c, alpha, beta, m, n, k)
    bound = abs(alpha) * oracle.abs_bound(a_val, b_val, m, n, k)
    if beta != 0.0:
        bound = bound + abs(beta) * np.abs(c).astype(np.float64)
    assert oracle.worst_ratio(d, ref, bound) <= 1.0
    # run to run the result is the same, bit for bit
    d2 = np.zeros(m * n, dtype=np.float32)
    r.run_host(stored16(a_bits, m, k, trans_a, lda), stored16(b_bits, k, n, trans_b, ldb), c if beta != 0.0 else None, d2,
               m, n, k, alpha=alpha, beta=beta, lda=lda, ldb=ldb)
    assert np.array_equal(d, d2)


def test_half_operands_large_problem_and_chunked_accumulation(runner_of):
    """4096 x 4096 x 4096 in BF16 (pipelined host path, chains of 1024 k), checked on a column sample; same-signed
    operands stay inside the bound thanks to the chunked accumulation."""
    m = n = k = 4096
    r = runner_of("bf16_tc2_256x256x64_s6")
    a32, b32, _ = oracle.make_inputs(m, n, k, seed=9)
    a_bits, a_val = narrow(np.abs(a32), "bf16")
    b_bits, b_val = narrow(np.abs(b32), "bf16")
    d = np.zeros(m * n, dtype=np.float32)
    r.set_option("split_k", 0)
    r.run_host(a_bits, b_bits, None, d, m, n, k)
    assert r.info("last_variant") == TENSOR and r.info("last_acc_chain") == 1024
    cols = np.arange(0, n, 97)
    b_cols = np.ascontiguousarray(b_val.reshape(n, k)[cols]).reshape(-1)
    ref = oracle.gemm(a_val, b_cols, None, 1.0, 0.0, m, len(cols), k)
    bound = oracle.abs_bound(a_val, b_cols, m, len(cols), k)
    got = np.ascontiguousarray(d.reshape(n, m)[cols]).reshape(-1)
    assert oracle.worst_ratio(got, ref, bound) <= 1.0


def test_half_kernels_refuse_what_they_cannot_serve(runner_of):
    r = runner_of("fp16_tc_128x128x64_s4")
    a = np.zeros(64 * 64, dtype=np.uint16)
    d = np.zeros(64 * 64, dtype=np.float32)
    r.set_option("force_variant", SIMT)
    with pytest.raises(Exception, match="tensor-core kernel only"):
        r.run_host(a, a, None, d, 64, 64, 64)
    r.set_option("force_variant", AUTO)
    with pytest.raises(Exception, match="multiples of 8"):
        r.run_host(np.zeros(68 * 64, dtype=np.uint16), np.zeros(68 * 64, dtype=np.uint16), None, d, 64, 64, 64, lda=64, ldb=68)
