"""The N > 1 host path on CPU: two `gloo` ranks shard the columns of one GEMM, each computes its shard, the
optional all-gather reassembles D, and the timing reduction takes the max over ranks.  The per-shard product is
done by NumPy here — this test covers the sharding, gathering and reduction logic, not a kernel."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, tile_n, out_dir):
    import importlib
    sys.path.insert(0, str(ROOT))
    importlib.import_module("amdgpu-arch-gemm_b200")
    from runner.shard import gather_columns, max_over_ranks, shard_columns
    from oracle import oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n0, n1 = shard_columns(n, world, rank, tile_n)
        a = oracle.fill_uniform(m * k, 0)                                   # A replicated
        b_local = oracle.fill_uniform(k * (n1 - n0), 1, first_index=n0 * k)  # B[:, n0:n1], filled by global index
        d_local = (b_local.reshape(n1 - n0, k).astype(np.float64) @ a.reshape(k, m).astype(np.float64)).astype(np.float32)
        full = gather_columns(dist, torch.from_numpy(d_local.reshape(-1)), m, n, world, tile_n).numpy()
        slowest = max_over_ranks(dist, float(rank + 1))
        np.save(Path(out_dir) / f"rank{rank}.npy", full)
        (Path(out_dir) / f"rank{rank}.txt").write_text(f"{n0} {n1} {slowest}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m,n,k,tile_n", [(48, 96, 40, 16), (33, 50, 17, 16)])
def test_two_ranks_shard_gather_and_reduce(tmp_path, m, n, k, tile_n):
    world = 2
    mp.start_processes(_worker, args=(world, _free_port(), m, n, k, tile_n, str(tmp_path)), nprocs=world, join=True,
                       start_method="spawn")
    from oracle import oracle
    a = oracle.fill_uniform(m * k, 0)
    b = oracle.fill_uniform(k * n, 1)
    want = (b.reshape(n, k).astype(np.float64) @ a.reshape(k, m).astype(np.float64)).astype(np.float32).reshape(-1)
    spans = []
    for r in range(world):
        got = np.load(tmp_path / f"rank{r}.npy")
        assert got.shape == want.shape and np.array_equal(got, want)   # every rank holds the full, correctly ordered D
        n0, n1, slowest = (tmp_path / f"rank{r}.txt").read_text().split()
        spans.append((int(n0), int(n1)))
        assert float(slowest) == float(world)                          # max over ranks of (rank + 1)
    assert spans[0][0] == 0 and spans[0][1] == spans[1][0] and spans[1][1] == n
