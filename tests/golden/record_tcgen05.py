"""Record what the sm_100a tensor cores return for the cases of tests/tensor_cases.py (needs a B200).

    python tests/golden/record_tcgen05.py

runs every case through the C ABI with the plain TF32 kernel (terms = 1) or the 3xTF32 kernel (terms = 3), alpha = 1,
beta = 0, no split-K, and writes the outputs to tests/golden/tcgen05_recorded.npz.  The committed file is what the CPU
tests hold the host model of the arithmetic (oracle/tensor_model.py) against, bit for bit; the inputs are not stored,
they are regenerated from the index-hash generator."""
import importlib
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path[:0] = [str(ROOT), str(HERE.parent)]
importlib.import_module("amdgpu-arch-gemm_b200")
import kernels  # noqa: E402
import tensor_cases  # noqa: E402
from runner import api  # noqa: E402

KERNEL_OF_TERMS = {1: "tc_128x128x32_s3_1x", 3: "tc2_256x256x32_s3_c0"}   # both accumulate all of K in TMEM


def device_gemm(r, a_mat, b_mat):
    m, k = a_mat.shape
    n = b_mat.shape[1]
    a = np.ascontiguousarray(a_mat.T, dtype=np.float32).reshape(-1)   # column-major m x k
    b = np.ascontiguousarray(b_mat.T, dtype=np.float32).reshape(-1)   # column-major k x n
    d = np.zeros(m * n, dtype=np.float32)
    r.run_host(a, b, None, d, m, n, k, alpha=1.0, beta=0.0)
    assert r.last_status()[0] == 0
    return d.reshape(n, m).T.copy()


def main():
    api.build_library()
    runners = {}
    for terms, name in KERNEL_OF_TERMS.items():
        cubin, toml = kernels.ensure(name)
        r = api.SgemmRunner(cubin, toml, 0)
        r.set_option("force_variant", 1)
        r.set_option("split_k", 1)
        runners[terms] = r
    out = {}
    for name, (a_mat, b_mat, terms) in tensor_cases.cases().items():
        out[name] = device_gemm(runners[terms], a_mat, b_mat)
    for r in runners.values():
        r.close()
    target = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE / "tcgen05_recorded.npz"
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({len(out)} cases, {sum(v.size for v in out.values())} elements)")


if __name__ == "__main__":
    main()
