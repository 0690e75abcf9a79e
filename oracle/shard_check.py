"""TEST INFRASTRUCTURE — oracle checks of column shards of a seeded SGEMM (the multi-GPU workload).

Only the test-suite and the benchmark's parity leg (after its timed regions) may import this module; it is a
checker built on the CPU oracle, never part of the product path.

The sharded workload: A (M x K, generator stream ``seed``) is replicated, rank r of g owns the columns [n0, n1)
of B (K x N, stream ``seed + 1``) and of D = A * B.  Every matrix is filled by GLOBAL element index, so column j of
B holds the generator's values for indices j*K .. j*K + K - 1 whatever the sharding.  What a rank computed is
checked here from nothing but (M, K, seed) and the global column numbers: an offset error in a shard's fill or
in its pointer arithmetic changes the values the oracle expects and fails the check.

Arithmetic and tolerance are those of the reference's CPU validation GEMM (runner/generator_runner.cpp:16-33)
as restated in ``oracle.gemm``, with the bound |D - D_ref| <= 1e-5 * sum_l |a_il||b_lj| per element.
"""
from __future__ import annotations

import numpy as np

from . import oracle


def sample_columns(n0: int, n1: int, tile_n: int, count: int, seed: int = 0) -> np.ndarray:
    """Global column numbers to check in the shard [n0, n1): its first and last column, the first and last column
    of its first, a middle and its last tile, and seeded random columns up to ``count`` (sorted, unique)."""
    width = n1 - n0
    if width <= 0:
        return np.zeros(0, dtype=np.int64)
    fixed = {n0, n1 - 1}
    tiles = (width + tile_n - 1) // tile_n
    for t in {0, tiles // 2, tiles - 1}:
        fixed.add(min(n0 + t * tile_n, n1 - 1))
        fixed.add(min(n0 + (t + 1) * tile_n - 1, n1 - 1))
    rng = np.random.default_rng(seed * 1000003 + n0)
    extra = rng.choice(width, size=min(width, max(0, count - len(fixed))), replace=False) + n0
    return np.unique(np.concatenate([np.fromiter(fixed, dtype=np.int64), extra.astype(np.int64)]))


def global_a(m: int, k: int, seed: int = 0) -> np.ndarray:
    """The replicated A of the workload (flat, column-major, lda = M)."""
    return oracle.fill_uniform(m * k, seed)


def global_b_columns(k: int, cols, seed: int = 0) -> np.ndarray:
    """Columns ``cols`` (global numbers) of B, dense and in that order (flat, ldb = K)."""
    out = np.empty(len(cols) * k, dtype=np.float32)
    for i, c in enumerate(cols):
        out[i * k:(i + 1) * k] = oracle.fill_uniform(k, seed + 1, first_index=int(c) * k)
    return out


def worst_ratio_of_columns(d_cols: np.ndarray, cols, m: int, k: int, seed: int = 0, a: np.ndarray | None = None) -> float:
    """max |D - D_ref| / (1e-5 * sum|a||b|) over the given columns of D = A * B (alpha 1, beta 0).
    ``d_cols`` holds the columns in the order of ``cols``, M values each; parity holds iff the result is <= 1."""
    cols = np.asarray(cols, dtype=np.int64)
    if cols.size == 0:
        return 0.0
    a = global_a(m, k, seed) if a is None else a
    b = global_b_columns(k, cols, seed)
    ref = oracle.gemm(a, b, None, 1.0, 0.0, m, len(cols), k)
    bound = oracle.abs_bound(a, b, m, len(cols), k)
    return oracle.worst_ratio(np.ascontiguousarray(d_cols, dtype=np.float32).reshape(-1), ref, bound)


def checksum_ratios(d_shard: np.ndarray, n0: int, n1: int, m: int, k: int, seed: int = 0, a: np.ndarray | None = None,
                    block: int = 512):
    """Linearity checksums over EVERY element of a shard of D (flat, M per column), in FP64:
    sum_j D[i, j] = sum_l A[i, l] * (sum_j B[l, j]) per row and sum_i D[i, j] = sum_l (sum_i A[i, l]) * B[l, j] per
    column, each against 1e-5 times the same expression on absolute values.  Returns (worst row ratio, worst
    column ratio); both must be <= 1.  Works through A and B in blocks so that no FP64 copy of a whole matrix is made."""
    width = n1 - n0
    a = global_a(m, k, seed) if a is None else a
    A = a.reshape(k, m)                                    # row l = column l of A
    D = np.ascontiguousarray(d_shard, dtype=np.float32).reshape(width, m)
    b_sum = np.zeros(k, dtype=np.float64)
    b_abs = np.zeros(k, dtype=np.float64)
    a_colsum = np.zeros(k, dtype=np.float64)
    a_colabs = np.zeros(k, dtype=np.float64)
    for l0 in range(0, k, block):
        blk = A[l0:l0 + block].astype(np.float64)
        a_colsum[l0:l0 + block] = blk.sum(axis=1)
        a_colabs[l0:l0 + block] = np.abs(blk).sum(axis=1)
    col_want = np.empty(width, dtype=np.float64)
    col_slack = np.empty(width, dtype=np.float64)
    col_got = np.empty(width, dtype=np.float64)
    row_got = np.zeros(m, dtype=np.float64)
    for j0 in range(0, width, block):
        cols = np.arange(n0 + j0, n0 + min(j0 + block, width))
        Bb = global_b_columns(k, cols, seed).reshape(len(cols), k).astype(np.float64)
        b_sum += Bb.sum(axis=0)
        b_abs += np.abs(Bb).sum(axis=0)
        col_want[j0:j0 + len(cols)] = Bb @ a_colsum
        col_slack[j0:j0 + len(cols)] = np.abs(Bb) @ a_colabs
        Db = D[j0:j0 + len(cols)].astype(np.float64)
        col_got[j0:j0 + len(cols)] = Db.sum(axis=1)
        row_got += Db.sum(axis=0)
    row_want = np.zeros(m, dtype=np.float64)
    row_slack = np.zeros(m, dtype=np.float64)
    for l0 in range(0, k, block):
        blk = A[l0:l0 + block].astype(np.float64)
        row_want += b_sum[l0:l0 + block] @ blk
        row_slack += b_abs[l0:l0 + block] @ np.abs(blk)
    tiny = np.finfo(np.float64).tiny
    row_ratio = float(np.max(np.abs(row_got - row_want) / (oracle.REL_TOL * row_slack + tiny)))
    col_ratio = float(np.max(np.abs(col_got - col_want) / (oracle.REL_TOL * col_slack + tiny)))
    return row_ratio, col_ratio
