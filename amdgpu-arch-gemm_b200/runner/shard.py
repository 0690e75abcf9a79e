"""Column-block sharding of one SGEMM over the GPUs of a box (one process per GPU).

D's columns are independent, and in column-major storage ``B[:, n0:n1]``, ``C[:, n0:n1]`` and ``D[:, n0:n1]``
are contiguous ranges ``[n0*ld, n1*ld)``: a shard is a pointer offset and each rank runs the unmodified
single-GPU kernel on ``N' = n1 - n0`` columns with A replicated.  No collective sits on the compute path;
``gather_columns`` is the optional all-gather of D, and ``max_over_ranks`` the timing reduction.
"""
from __future__ import annotations

from typing import List, Tuple


def shard_columns(n: int, world: int, rank: int, tile_n: int = 1) -> Tuple[int, int]:
    """Columns [n0, n1) of rank ``rank``: whole tiles of ``tile_n`` columns, as even as possible, earlier
    ranks take the extra tile; the last non-empty shard absorbs a ragged tail."""
    if world < 1 or not (0 <= rank < world) or n < 0 or tile_n < 1:
        raise ValueError("bad shard request")
    tiles = (n + tile_n - 1) // tile_n
    base, extra = divmod(tiles, world)
    t0 = rank * base + min(rank, extra)
    t1 = t0 + base + (1 if rank < extra else 0)
    return min(t0 * tile_n, n), min(t1 * tile_n, n)


def all_shards(n: int, world: int, tile_n: int = 1) -> List[Tuple[int, int]]:
    return [shard_columns(n, world, r, tile_n) for r in range(world)]


def fill_shard_inputs(runner, a, b, m: int, k: int, n0: int, n1: int, seed: int = 0, stream=0) -> None:
    """Fill this rank's operands of the sharded workload on the device: the replicated A (M x K, generator stream
    ``seed``) and the columns [n0, n1) of B (K x N, stream ``seed + 1``), both by GLOBAL element index — column j of
    B starts at index j*K — so that 1, 2, 4 and 8 GPUs compute on the same matrices.  ``a`` and ``b`` are device
    buffers (tensors or addresses) of M*K and K*(n1 - n0) floats."""
    runner.fill_uniform(a, m * k, stream_id=seed, stream=stream)
    if n1 > n0:
        runner.fill_uniform(b, k * (n1 - n0), stream_id=seed + 1, first_index=n0 * k, stream=stream)


def gather_columns(dist, local_d, m: int, n: int, world: int, tile_n: int = 1):
    """All-gather the column shards of D (flat column-major tensors) into the full M x N matrix on every rank through
    ``torch.distributed`` (any backend; the native in-place form over NCCL is ``SgemmRunner.allgather_columns``).
    Equal shards are gathered straight into the result; shards of different width are padded to the widest one for
    the collective and cut back afterwards."""
    import torch

    shards = all_shards(n, world, tile_n)
    widths = [n1 - n0 for n0, n1 in shards]
    if len(set(widths)) == 1:
        full = torch.empty(m * n, dtype=local_d.dtype, device=local_d.device)
        dist.all_gather_into_tensor(full, local_d[: m * widths[0]].contiguous())
        return full
    widest = max(widths)
    padded = torch.zeros(m * widest, dtype=local_d.dtype, device=local_d.device)
    padded[: local_d.numel()] = local_d
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([parts[r][: m * w] for r, w in enumerate(widths)])


def make_communicator(dist, runner, rank: int, world: int) -> None:
    """Give ``runner`` (one ``SgemmRunner`` per process, one process per GPU) the library's own communicator over all
    ranks: rank 0 makes the id, ``torch.distributed`` (the host-side plumbing) hands it to the others, every rank
    joins with its GPU."""
    from runner import api

    box = [api.comm_unique_id() if rank == 0 else None]
    if world > 1:
        dist.broadcast_object_list(box, src=0)
    runner.comm_init(box[0], rank, world)


def max_over_ranks(dist, value: float, device="cpu") -> float:
    import torch

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
