"""Generate the golden vectors under tests/golden/ from the UNMODIFIED reference.

Run in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py --reference /path/to/amdgpu-arch-gemm

The script imports the reference's kernel generator (generator/generator.py) and its GCN
virtual machine (vm/gcn_virtual_machine.py), emits the reference SGEMM kernel for single-wave
configurations, interprets it once per workgroup and stores inputs + the D matrix the VM leaves
in its vector memory.  The GPU box has no copy of the reference, so the resulting ``.npz`` files
are committed and this script is the record of how they were made.

Cases
-----
* the four whole-kernel fixtures of the reference's own tests (test/test_vm.py:447-627,
  :743-963): arange/ones inputs, alpha = beta = 1;
* the 32x32x32 configuration with seeded uniform[-1,1) inputs (streams seed, seed+1, seed+2 of
  the index-hash generator in oracle/oracle.py), alpha = 1, beta in {0, 1}, for both single-wave
  32x32 tilings (mfma 32x32x2 with tiling 1x1, mfma 16x16x4 with tiling 2x2);
* multi-workgroup problems (64x48x64 over its 4x3 grid with the K-stagger and the three-buffer knobs, 64x64x32 over
  its 4x4 grid with the workgroup remap) run workgroup by workgroup, so the full D (not only one tile) is pinned.
"""
from __future__ import annotations

import argparse
import contextlib
import io
import struct
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import oracle  # noqa: E402  (seeded inputs only)


def load_reference(path: str):
    sys.path.insert(0, path)
    import generator.generator as G  # type: ignore
    import vm.gcn_virtual_machine as V  # type: ignore

    assert Path(G.__file__).resolve().is_relative_to(Path(path).resolve()), G.__file__
    return G, V


def kernel_arguments(G):
    names = [("global_buffer", n, 8) for n in "abcd"]
    names += [("by_value", n, 4) for n in ("m", "n", "k", "lda", "ldb", "ldc", "ldd", "alpha", "beta",
                                            "numWorkgroupX", "numWorkgroupY")]
    return [G.FunctionArgument(t, n, None, s) for (t, n, s) in names]


def run_reference_kernel(G, V, mfma, wave_tiling, depth_k, vmem_stage, opt_kwargs, m, n, k, a, b, c,
                         alpha, beta):
    """Interpret the reference kernel for every workgroup of the grid; return flat column-major D."""
    cfg = G.GemmSolutionConfig(G.DataType.FP32, G.DataType.FP32, G.DataType.FP32, G.DataType.FP32,
                               mfma, (1, 1), wave_tiling, depth_k, False, False, vmem_stage=vmem_stage)
    mt0, mt1 = cfg.tile_size
    assert m % mt0 == 0 and n % mt1 == 0 and k % depth_k == 0 and k >= 2 * depth_k
    nwg_x, nwg_y = m // mt0, n // mt1
    a_off, b_off = 0, m * k * 4
    c_off = b_off + n * k * 4
    d_off = c_off + m * n * 4
    assert d_off + m * n * 4 <= 65536, "problem does not fit the VM's 64 KiB vector memory"
    d_full = np.zeros(m * n, dtype=np.float32)
    for wy in range(nwg_y):
        for wx in range(nwg_x):
            opt = G.GemmOptimizations(1, **opt_kwargs)
            vm = V.GcnVirtualMachine(104, 256, 64)
            for lane in range(vm.wavefront_size):
                vm.v[0][lane] = lane
            vm.s[0] = vm.s[1] = 0
            vm.s[2], vm.s[3] = wx, wy
            sm = vm.smem.mem
            for i, off in enumerate((a_off, b_off, c_off, d_off)):
                sm[8 * i:8 * i + 8] = int.to_bytes(off, 8, "little")
            for i, v in enumerate((m, n, k, m, k, m, m)):
                sm[32 + 4 * i:36 + 4 * i] = int.to_bytes(v, 4, "little")
            sm[60:64] = struct.pack("f", alpha)
            sm[64:68] = struct.pack("f", beta)
            sm[68:72] = int.to_bytes(nwg_x, 4, "little")
            sm[72:76] = int.to_bytes(nwg_y, 4, "little")
            vm.vmem.mem[a_off:a_off + a.nbytes] = bytearray(a)
            vm.vmem.mem[b_off:b_off + b.nbytes] = bytearray(b)
            vm.vmem.mem[c_off:c_off + c.nbytes] = bytearray(c)
            ctx = G.GpuContext()
            G.gemm(ctx, "gemm", "gfx90a:xnack-", cfg, opt, kernel_arguments(G))
            with contextlib.redirect_stdout(io.StringIO()):
                vm.run(ctx)
            d_wg = np.frombuffer(bytes(vm.vmem.mem[d_off:d_off + m * n * 4]), dtype=np.float32)
            # Which tile this workgroup wrote is decided by the kernel (workgroup remap); take every
            # element it changed from the zero-initialised D region.
            touched = d_wg != 0
            d_full[touched] = d_wg[touched]
    return d_full


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    G, V = load_reference(args.reference)

    def save(name, **kw):
        np.savez_compressed(HERE / f"{name}.npz", **kw)
        print(f"wrote {name}.npz  D[0:4] = {kw['d'][:4]}")

    # --- the reference's own whole-kernel fixtures ------------------------------------------------
    def arange_case(name, mfma, m, n, k, vmem_stage=1, opt_kwargs=None):
        a = np.arange(m * k, dtype=np.float32)
        b = np.arange(n * k, dtype=np.float32)
        c = np.ones(m * n, dtype=np.float32)
        d = run_reference_kernel(G, V, mfma, (1, 1), 16, vmem_stage, opt_kwargs or {"plr": 1}, m, n, k,
                                 a, b, c, 1.0, 1.0)
        save(name, a=a, b=b, c=c, d=d, mnk=np.array([m, n, k]), alpha=np.float32(1), beta=np.float32(1))

    arange_case("vm_16x16x64_arange", (16, 16, 1, 4), 16, 16, 64)
    arange_case("vm_32x32x64_arange", (32, 32, 1, 2), 32, 32, 64)
    arange_case("vm_64x48x64_mapk4_arange", (16, 16, 1, 4), 64, 48, 64, opt_kwargs={"plr": 1, "map_k_idx": 4})
    arange_case("vm_64x48x64_3buf_arange", (16, 16, 1, 4), 64, 48, 64, vmem_stage=2)
    arange_case("vm_64x64x32_wgm2_arange", (16, 16, 1, 4), 64, 64, 32, opt_kwargs={"plr": 1, "wgm": 2})

    # --- configuration 1: 32^3, seeded uniform inputs ---------------------------------------------
    m = n = k = 32
    a, b, c = oracle.make_inputs(m, n, k, seed=args.seed)
    for tag, mfma, wt in (("mfma32", (32, 32, 1, 2), (1, 1)), ("mfma16", (16, 16, 1, 4), (2, 2))):
        for beta in (0.0, 1.0):
            d = run_reference_kernel(G, V, mfma, wt, 16, 1, {"plr": 1}, m, n, k, a, b, c, 1.0, beta)
            save(f"vm_32x32x32_seed{args.seed}_{tag}_beta{int(beta)}", a=a, b=b, c=c, d=d,
                 mnk=np.array([m, n, k]), alpha=np.float32(1), beta=np.float32(beta))


if __name__ == "__main__":
    main()
