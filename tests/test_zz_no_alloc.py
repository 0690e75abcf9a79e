"""sgemm_launch_noalloc: the SGEMM entry point for callers that are not allowed to allocate device memory
when they call (a serving loop whose memory budget is frozen, a real-time path that cannot take a blocking driver
call, a process whose GPU memory is managed by somebody else's allocator).  Its scratch is a fixed array inside the library, so
the things to check are: it computes what sgemm_launch computes, it keeps doing so when the array is reused by
the next call (the array still holds the previous call's data), and it refuses problems that would not fit
instead of allocating.  Collected last on purpose: a failure here cannot hide a failure elsewhere."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture()
def runner(built):
    from runner import api
    cubin, toml = built.ensure(built.DEFAULT_TENSOR)
    r = api.SgemmRunner(cubin, toml, 0)
    yield r
    assert r.last_status()[0] == 0
    r.close()


def device_inputs(r, m, n, k, seed):
    a, b, c = oracle.make_inputs(m, n, k, seed=seed)
    bufs = [r.dev_alloc(x.nbytes) for x in (a, b, c)] + [r.dev_alloc(m * n * 4)]
    for p, x in zip(bufs, (a, b, c)):
        r.upload(p, x)
    return (a, b, c), bufs


def fetch(r, dptr, count):
    out = np.empty(count, dtype=np.float32)
    r.sync()
    r.download(out, dptr)
    return out


@pytest.mark.parametrize("force,split_k,mnk", [
    (1, 4, (256, 320, 2048)),    # tensor path: lo copies of A and B + four split-K partial products in the scratch
    (2, 8, (200, 136, 4096)),    # SIMT path: split-K partial products only
    (0, 0, (512, 512, 512)),     # whatever the library picks on its own
])
def test_matches_the_allocating_entry_point_on_two_calls_in_a_row(runner, force, split_k, mnk):
    from runner import api
    m, n, k = mnk
    r = runner
    r.set_option("force_variant", force)
    r.set_option("split_k", split_k)
    assert 0 < r.workspace_bytes(m, n, k) <= api.noalloc_scratch_bytes()
    (a, b, c), (pa, pb, pc, pd) = device_inputs(r, m, n, k, seed=21)
    (a2, b2, c2), (qa, qb, qc, qd) = device_inputs(r, m, n, k, seed=22)
    try:
        # existing entry point (handle-owned, allocated workspace) as the reference
        r.launch(pa, pb, pc, pd, m, n, k, alpha=1.0, beta=0.5)
        want = fetch(r, pd, m * n)
        r.launch(qa, qb, qc, qd, m, n, k, alpha=1.0, beta=0.5)
        want2 = fetch(r, qd, m * n)
        for p in (pd, qd):
            r.memset(p, 0, m * n * 4)
        owned_before = r.info("workspace_bytes")
        # two allocation-free calls back to back: the second one finds the first one's data in the scratch
        r.launch_noalloc(pa, pb, pc, pd, m, n, k, alpha=1.0, beta=0.5)
        r.launch_noalloc(qa, qb, qc, qd, m, n, k, alpha=1.0, beta=0.5)
        got, got2 = fetch(r, pd, m * n), fetch(r, qd, m * n)
        assert r.info("workspace_bytes") == owned_before           # the handle's own workspace did not grow
        for g, w, (x, y, z) in ((got, want, (a, b, c)), (got2, want2, (a2, b2, c2))):
            bound = oracle.abs_bound(x, y, m, n, k) + 0.5 * np.abs(z).astype(np.float64)
            assert oracle.worst_ratio(g, w, bound) <= 1.0           # the tolerance of the parity tests
            assert g.tobytes() == w.tobytes()                       # and in fact the same bits: same kernels, same order
        # and against the CPU oracle, so that both entry points being wrong together cannot pass
        ref = oracle.gemm(a, b, c, 1.0, 0.5, m, n, k)
        assert oracle.worst_ratio(got, ref, oracle.abs_bound(a, b, m, n, k) + 0.5 * np.abs(c).astype(np.float64)) <= 1.0
    finally:
        r.sync()
        for p in (pa, pb, pc, pd, qa, qb, qc, qd):
            r.dev_free(p)


def test_refuses_problems_beyond_the_fixed_scratch(runner):
    from runner import api
    r = runner
    m = n = k = 8192                        # needs 512 MiB of lo copies: far beyond the 32 MiB array
    assert r.workspace_bytes(m, n, k) > api.noalloc_scratch_bytes()
    dummy = r.dev_alloc(256)                # never dereferenced: the size check comes before any launch
    try:
        launches = r.info("launches")
        with pytest.raises(api.SgemmError) as e:
            r.launch_noalloc(dummy, dummy, None, dummy, m, n, k)
        assert e.value.code == -9 and "scratch" in str(e.value)
        assert r.info("launches") == launches
    finally:
        r.dev_free(dummy)


def test_counts_the_aligned_copies_of_operands_tma_cannot_read(runner):
    """An A that starts 4 bytes into an allocation cannot be read by TMA where it lies: the tensor path first copies it
    to an aligned pitch inside the scratch.  The size check must count that copy — a problem that fits with an aligned A
    and does not fit with this one is refused with the scratch-limit code before anything is launched, and a smaller one
    of the same kind is computed correctly out of the fixed array."""
    from runner import api
    r = runner
    r.set_option("force_variant", 1)
    r.set_option("split_k", 1)
    m, n, k = 2048, 128, 2048              # lo copies of A and B: 17 MiB, with the aligned copy of A: 33 MiB
    base = r.dev_alloc(m * k * 4 + 256)
    other = r.dev_alloc(max(k * n, m * n) * 4)
    try:
        assert r.workspace_bytes(m, n, k) <= api.noalloc_scratch_bytes() < r.workspace_bytes(m, n, k, a=base + 4, b=other)
        launches = r.info("launches")
        with pytest.raises(api.SgemmError) as e:
            r.launch_noalloc(base + 4, other, None, other, m, n, k)
        assert e.value.code == -9 and r.info("launches") == launches
    finally:
        r.dev_free(base)
        r.dev_free(other)
    m, n, k = 512, 128, 1024
    a, b, c = oracle.make_inputs(m, n, k, seed=23)
    pa, pb, pd = r.dev_alloc(a.nbytes + 16), r.dev_alloc(b.nbytes), r.dev_alloc(m * n * 4)
    try:
        r.upload(pa + 4, a)
        r.upload(pb, b)
        for _ in range(2):
            r.memset(pd, 0, m * n * 4)
            r.launch_noalloc(pa + 4, pb, None, pd, m, n, k)
            got = fetch(r, pd, m * n)
            assert r.info("last_variant") == 1
            ref = oracle.gemm(a, b, None, 1.0, 0.0, m, n, k)
            assert oracle.worst_ratio(got, ref, oracle.abs_bound(a, b, m, n, k)) <= 1.0
    finally:
        r.sync()
        for p in (pa, pb, pd):
            r.dev_free(p)


def test_on_another_gpu_it_touches_no_other_gpu_and_no_thread_state(built):
    """A rank that works on GPU 1 must not grow a context on GPU 0 behind its back, and a caller that only uses this C
    ABI has no "current device" for the entry point to switch or restore: the array's address is looked up with the
    handle's own context pushed.  Checked in a fresh process (no other test has touched a GPU there): after two
    allocation-free calls on GPU 1 that equal the allocating entry point's results, GPU 0 has no active primary context
    in this process, GPU 1 has one, and the calling thread still has no current context.  Needs two GPUs."""
    import subprocess, sys, textwrap
    from pathlib import Path
    from runner import api
    if api.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = Path(__file__).resolve().parent.parent
    cubin, toml = built.ensure(built.DEFAULT_TENSOR)
    code = textwrap.dedent(f"""
        import ctypes, importlib, sys
        import numpy as np
        sys.path.insert(0, {str(root)!r})
        importlib.import_module("amdgpu-arch-gemm_b200")
        from runner import api
        from oracle import oracle
        m, n, k = 256, 320, 1024
        a, b, c = oracle.make_inputs(m, n, k, seed=31)
        r = api.SgemmRunner({cubin!r}, {toml!r}, 1)
        r.set_option("force_variant", 1)
        bufs = [r.dev_alloc(x.nbytes) for x in (a, b, c)] + [r.dev_alloc(m * n * 4)]
        for p, x in zip(bufs, (a, b, c)):
            r.upload(p, x)
        outs = []
        for call in (r.launch, r.launch_noalloc, r.launch_noalloc):
            r.memset(bufs[3], 0, m * n * 4)
            call(bufs[0], bufs[1], bufs[2], bufs[3], m, n, k, alpha=1.0, beta=0.5)
            d = np.empty(m * n, np.float32)
            r.sync()
            r.download(d, bufs[3])
            outs.append(d.tobytes())
        cuda = ctypes.CDLL("libcuda.so.1")
        flags, active = ctypes.c_uint(), ctypes.c_int()
        state = []
        for dev in (0, 1):
            assert cuda.cuDevicePrimaryCtxGetState(dev, ctypes.byref(flags), ctypes.byref(active)) == 0
            state.append(active.value)
        current = ctypes.c_void_p()
        assert cuda.cuCtxGetCurrent(ctypes.byref(current)) == 0
        print(outs[0] == outs[1] == outs[2], state, current.value)
        r.close()
    """)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip().splitlines()[-1] == "True [0, 1] None"
