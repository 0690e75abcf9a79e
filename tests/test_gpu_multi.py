"""The multi-GPU surface of the C ABI on real GPUs: communicators over the handles of one process, the sharded
host-buffer call (A uploaded in slices and completed over NVLink) and the in-place all-gather of D.

With one GPU the communicator has one rank: the calls must still work and equal their single-GPU counterparts bit for
bit.  With two or more GPUs (the tests skip otherwise) two handles of one process shard a problem, each rank driven by
its own host thread — the sharded calls are collective — and the assembled result is compared with the single-GPU
call and with the CPU oracle (reference arithmetic: runner/generator_runner.cpp:16-33)."""
import threading

import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu


def open_runners(built, count, kernel=None):
    from runner import api
    cubin, toml = built.ensure(kernel or built.DEFAULT_TENSOR)
    return [api.SgemmRunner(cubin, toml, i) for i in range(count)]


def close_all(runners):
    for r in runners:
        assert r.last_status()[0] == 0
        r.close()


def test_one_rank_communicator_equals_the_single_gpu_calls(built):
    from runner import api
    (r,) = open_runners(built, 1)
    try:
        assert (r.info("comm_rank"), r.info("comm_world")) == (-1, 0)
        m, n, k = 1024, 1536, 2048                      # 26 MiB of operands: the unpipelined host path
        a, b, c = oracle.make_inputs(m, n, k, seed=3)
        want = np.zeros(m * n, np.float32)
        r.run_host(a, b, c, want, m, n, k, alpha=1.0, beta=0.5)
        with pytest.raises(api.SgemmError) as e:        # no communicator yet
            r.run_host_sharded(a, b, c, np.zeros(m * n, np.float32), m, n, k, alpha=1.0, beta=0.5)
        assert e.value.code == -10
        api.comm_init_all([r])
        assert (r.info("comm_rank"), r.info("comm_world")) == (0, 1)
        got = np.zeros(m * n, np.float32)
        r.run_host_sharded(a, b, c, got, m, n, k, alpha=1.0, beta=0.5)
        assert got.tobytes() == want.tobytes()
        dd = r.dev_alloc(m * n * 4)
        try:
            r.upload(dd, want)
            r.allgather_columns(dd, m, n)               # one rank: nothing to exchange, nothing changes
            back = np.empty(m * n, np.float32)
            r.sync()
            r.download(back, dd)
            assert back.tobytes() == want.tobytes()
        finally:
            r.dev_free(dd)
        r.comm_destroy()
        assert r.info("comm_world") == 0
        with pytest.raises(api.SgemmError):
            api.comm_init_all([r, r])                   # two handles of one communicator on one GPU
    finally:
        close_all([r])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mnk,beta,kernel", [
    ((2048, 4096 + 96, 2048), 0.0, None),                    # pipelined host path, ragged last shard
    ((1000, 700, 520), 0.75, None),                          # small: single launch per rank, ragged slices of A
    ((512, 256, 1024), 0.0, None),                           # fewer tiles than ranks at world 8: empty shards
    ((1024, 2048, 1000), 0.5, "tc2_256x256x32_s3_tn")])      # A stored transposed (K x M): its slices are cut along M
def test_sharded_host_call_and_allgather_over_several_gpus(built, world, mnk, beta, kernel):
    from runner import api
    from runner.shard import shard_columns
    if api.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    m, n, k = mnk
    a, b, c = oracle.make_inputs(m, n, k, seed=29)
    logical_a, lda = a, 0
    if kernel and kernel.endswith("_tn"):
        a, lda = np.ascontiguousarray(a.reshape(k, m).T).reshape(-1), k      # K x M column-major storage, lda = K
    runners = open_runners(built, world, kernel)
    try:
        tile_n = runners[0].info("tile_n")
        single = np.zeros(m * n, np.float32)
        runners[0].run_host(a, b, c, single, m, n, k, alpha=1.0, beta=beta, lda=lda)
        # A shard is a smaller problem and would choose kernel and split-K by its own size; a caller that wants the
        # sharded result to equal the unsharded one bit for bit pins both to what the whole problem got
        variant, split_k = runners[0].info("last_variant"), runners[0].info("last_split_k")
        for r in runners:
            r.set_option("force_variant", variant)
            r.set_option("split_k", split_k)
        api.comm_init_all(runners)
        spans = [shard_columns(n, world, r, tile_n) for r in range(world)]
        assert spans == [api.shard_columns(n, world, r, tile_n) for r in range(world)]
        outs = [np.zeros(max(m * (n1 - n0), 1), np.float32) for n0, n1 in spans]
        full = [r.dev_alloc(m * n * 4) for r in runners]
        gathered = [np.empty(m * n, np.float32) for _ in runners]
        errors = []
        ready = threading.Barrier(world)

        def rank_main(i):
            r, (n0, n1) = runners[i], spans[i]
            w = n1 - n0
            try:
                # the host call: this rank's slice of A goes up, the others' slices come over NVLink
                r.run_host_sharded(a, b[n0 * k:], c[n0 * m:] if beta else None, outs[i], m, w, k, alpha=1.0, beta=beta, lda=lda)
                # the device call into a full-size D ...
                if w:
                    da, db, dc = r.dev_alloc(a.nbytes), r.dev_alloc(max(w * k, 1) * 4), r.dev_alloc(max(w * m, 1) * 4)
                    r.upload(da, a)
                    r.upload(db, b[n0 * k:n1 * k])
                    r.upload(dc, c[n0 * m:n1 * m])
                    r.memset(full[i], 0xFF, m * n * 4)
                    r.launch(da, db, dc if beta else None, full[i] + n0 * m * 4, m, w, k, alpha=1.0, beta=beta, lda=lda)
                    r.sync()
                    for p in (da, db, dc):
                        r.dev_free(p)
            except Exception as exc:   # noqa: BLE001 - reported by the main thread
                errors.append((i, exc))
            ready.wait(timeout=240)
            if errors:                 # a rank that failed would leave the others waiting inside the collective: skip it
                return
            try:
                # ... then the in-place all-gather
                r.allgather_columns(full[i], m, n)
                r.sync()
                r.download(gathered[i], full[i])
            except Exception as exc:   # noqa: BLE001
                errors.append((i, exc))

        threads = [threading.Thread(target=rank_main, args=(i,), daemon=True) for i in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=300)
        assert not errors, errors
        assert not any(t.is_alive() for t in threads)
        assembled = np.concatenate([o[: m * (n1 - n0)] for o, (n0, n1) in zip(outs, spans)])
        assert assembled.tobytes() == single.tobytes()         # sharding changes no bit
        for g in gathered:
            assert g.tobytes() == single.tobytes()             # every rank holds all of D after the all-gather
        ref = oracle.gemm(logical_a, b, c, 1.0, beta, m, n, k)
        bound = oracle.abs_bound(logical_a, b, m, n, k) + abs(beta) * np.abs(c).astype(np.float64)
        assert oracle.worst_ratio(single, ref, bound) <= 1.0
        for r, p in zip(runners, full):
            r.dev_free(p)
    finally:
        close_all(runners)
