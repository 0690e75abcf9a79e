"""The kernels' barrier protocols under random interleavings (tests/pipeline_model.py): every supported combination
of stages, cluster shape, epilogue width and split placement must finish without a wrong tag, an overwrite of live
data or a deadlock — and deliberately broken variants of the protocol must be caught.  The TMA-fed FFMA kernel's
protocol is modelled together with its register hand-over, the one wait on the device that has no limit."""
import re
from pathlib import Path

import pytest

from pipeline_model import FfmaModel, Model, ProtocolError


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("inkernel", [False, True])
@pytest.mark.parametrize("stages,kblocks,tiles", [(2, 1, 5), (2, 7, 4), (3, 8, 6), (4, 3, 9), (7, 2, 3), (3, 1, 1)])
def test_protocol_holds_under_random_schedules(cta_group, inkernel, stages, kblocks, tiles):
    for seed in range(6):
        for epi in (4, 8):
            assert Model(tiles, kblocks, stages, cta_group, epi, inkernel, units=2, seed=seed).run()


def test_more_units_than_tiles_and_single_unit():
    assert Model(tiles=1, kblocks=4, stages=3, cta_group=2, units=3, seed=1).run()   # idle units finish at once
    assert Model(tiles=7, kblocks=5, stages=2, cta_group=2, inkernel=True, units=1, seed=2).run()


def test_missing_commit_to_the_peer_deadlocks():
    # the leader must free the stage in BOTH CTAs of a pair; committing only to its own copy starves the peer's producer
    with pytest.raises(ProtocolError, match="deadlock"):
        Model(tiles=3, kblocks=6, stages=2, cta_group=2, units=1, seed=0, bug="no_empty_commit_to_peer").run()


def test_accumulator_barrier_must_count_both_ctas():
    # tmem_empty with a count of one CTA's epilogue warps lets the issuer reuse an accumulator the peer still reads
    caught = 0
    for seed in range(40):
        try:
            Model(tiles=6, kblocks=1, stages=2, cta_group=2, units=1, seed=seed, bug="tempty_counts_one_cta").run()
        except ProtocolError:
            caught += 1
    assert caught >= 30


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("inkernel", [False, True])
@pytest.mark.parametrize("stages,kblocks,tiles,chunk", [(3, 8, 5, 4), (2, 7, 4, 3), (3, 9, 3, 1), (4, 5, 6, 2), (3, 4, 5, 8)])
def test_chunked_accumulation_hands_buffers_over_per_chunk(cta_group, inkernel, stages, kblocks, tiles, chunk):
    """Accumulator buffers alternate per hand-over (a tile may take an odd number of them), every chunk reaches the
    running sum exactly once and a buffer is never overwritten while it is read."""
    for seed in range(4):
        assert Model(tiles, kblocks, stages, cta_group, 8, inkernel, units=2, seed=seed, chunk=chunk).run()


def test_buffer_choice_per_tile_is_caught_with_chunks():
    with pytest.raises(ProtocolError):
        for seed in range(8):   # the issuer picks the buffer by tile, the epilogue by hand-over: they disagree
            Model(tiles=5, kblocks=6, stages=3, cta_group=1, units=1, seed=seed, chunk=2, bug="buffer_per_tile").run()


# ------------------------------------------------------------------------- the TMA-fed FFMA kernel's protocol
FFMA_HEADER = Path(__file__).resolve().parent.parent / "amdgpu-arch-gemm_b200" / "csrc" / "sgemm_ffma_tma.cuh"


def ffma_register_shares(threads: int):
    """(launch, first group, consumers) registers per thread as the kernel header computes them: its FT_REGS_* macros
    evaluated here (C integer arithmetic on positive numbers is Python's floor division)."""
    text = FFMA_HEADER.read_text()
    env = {"FT_THREADS": threads, "FT_CONSUMERS": threads - 128}
    for name in ("FT_WARPS_PER_PARTITION", "FT_REGS_LAUNCH", "FT_REGS_PRODUCER", "FT_REGS_CONSUMER_RAW", "FT_REGS_CONSUMER"):
        body = re.search(rf"^#define {name} (.*)$", text, re.M).group(1).split("//")[0].strip()
        ternary = re.fullmatch(r"\((.*) > (\d+) \? (\d+) : (.*)\)", body)
        if ternary:
            body = f"({ternary.group(3)} if {ternary.group(1)} > {ternary.group(2)} else {ternary.group(4)})"
        env[name] = eval(body.replace("/", "//"), {}, env)
    return env["FT_REGS_LAUNCH"], env["FT_REGS_PRODUCER"], env["FT_REGS_CONSUMER"]


@pytest.mark.parametrize("transpose", [True, False])
@pytest.mark.parametrize("stages,steps", [(2, 1), (2, 9), (3, 8), (4, 3), (6, 13), (12, 5)])
@pytest.mark.parametrize("consumer_warps", [4, 8, 16])
def test_ffma_tma_protocol_holds_under_random_schedules(transpose, stages, steps, consumer_warps):
    launch, small, consumer = ffma_register_shares(128 + 32 * consumer_warps)
    for seed in range(5):
        assert FfmaModel(steps, stages, consumer_warps, transpose, seed, regs_launch=launch, regs_small=small,
                         regs_consumer=consumer, handover=consumer_warps >= 8).run()


def test_ffma_register_shares_fit_the_launch_allocation():
    assert ffma_register_shares(384) == (168, 40, 232)     # 256 consumers: 16 x 8 accumulators each
    assert ffma_register_shares(640) == (96, 40, 104)      # 512 consumers
    for threads in (384, 512, 640):
        launch, small, consumer = ffma_register_shares(threads)
        groups = threads // 128
        assert small + (groups - 1) * consumer <= groups * launch and consumer > launch and consumer % 8 == 0


def test_a_hand_over_beyond_the_launch_allocation_deadlocks_in_the_model():
    # the budget a first version of the kernel used: shares of the 512 registers a partition owns, not of the 5 x 96 a
    # block of 640 threads is launched with -> the last consumer warps wait for registers that never come
    with pytest.raises(ProtocolError, match="deadlock"):
        FfmaModel(steps=6, stages=3, consumer_warps=16, seed=0, regs_launch=96, regs_small=40, regs_consumer=(512 - 40) // 4 // 8 * 8).run()
    assert FfmaModel(steps=6, stages=3, consumer_warps=16, seed=0, regs_launch=96, regs_small=40, regs_consumer=104).run()


def test_ffma_protocol_bugs_are_caught():
    caught = 0
    for seed in range(30):      # consumers that do not wait for the transposed tile read a stale or missing one
        try:
            FfmaModel(steps=8, stages=3, consumer_warps=8, seed=seed, bug="ready_not_waited").run()
        except ProtocolError:
            caught += 1
    assert caught >= 25
    caught = 0
    for seed in range(30):      # an "empty" barrier that counts one warp too few frees a stage that is still read
        try:
            FfmaModel(steps=12, stages=2, consumer_warps=8, seed=seed, bug="empty_count_short").run()
        except ProtocolError:
            caught += 1
    assert caught >= 25
