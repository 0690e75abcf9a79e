"""The kernel's barrier protocol under random interleavings (tests/pipeline_model.py): every supported combination
of stages, cluster shape, epilogue width and split placement must finish without a wrong tag, an overwrite of live
data or a deadlock — and deliberately broken variants of the protocol must be caught."""
import pytest

from pipeline_model import Model, ProtocolError


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
