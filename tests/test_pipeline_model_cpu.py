"""The barrier protocol of the GEMM kernels on a CPU model (tests/pipeline_model.py): no deadlock, no stage or
accumulator hazard under random interleavings, and a withheld arrival ends in the bounded-wait status of the role
that depends on it -- the failure path checked without a GPU."""
import pytest

from tests.pipeline_model import EPILOGUE, MMA, PRODUCER, SCALE, Pipeline


@pytest.mark.parametrize("tiles,kblocks,stages,raw,groups", [
    (1, 1, 4, 2, 3), (1, 4, 4, 2, 3), (3, 8, 4, 2, 3), (5, 64, 4, 2, 3),      # 128x256 tiles: 4 stages, 2 slabs, 3 atom groups
    (4, 7, 6, 4, 4), (2, 16, 8, 4, 4), (3, 13, 11, 4, 4), (7, 3, 9, 4, 4),    # narrower tiles: deeper rings
    (2, 5, 1, 1, 1), (6, 9, 2, 1, 2),                                         # degenerate rings still may not deadlock
])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_every_role_finishes_without_hazard(tiles, kblocks, stages, raw, groups, seed):
    p = Pipeline(tiles, kblocks, stages, raw, groups, seed=seed)
    timed_out = p.run()
    assert timed_out == {} and p.status == 0
    assert p.finished == {"producer", "scale", "mma", "epilogue"}
    # every barrier ends on a phase boundary: nothing is left half-arrived
    for bars in (p.full, p.empty, p.raw_full, p.raw_empty, p.atom_full, p.atom_empty, p.acc_full, p.acc_empty):
        assert all(b.pending == b.count for b in bars)


@pytest.mark.parametrize("drop,role", [
    (("full1", 2), MMA),            # a TMA load that never completes: the MMA warp's wait runs out
    (("empty0", 1), PRODUCER),      # a tcgen05.commit that never arrives: the producer cannot refill the stage
    (("raw_full0", 1), SCALE),      # a scale slab that never lands
    (("atom_full1", 0), MMA),       # scale atoms never published
    (("acc_full0", 1), EPILOGUE),   # the accumulator is never handed to the epilogue
    (("acc_empty1", 0), MMA),       # the epilogue never releases an accumulator
])
def test_withheld_arrival_ends_in_a_reported_timeout(drop, role):
    p = Pipeline(tiles=6, kblocks=12, stages=4, raw_slots=2, atom_groups=3, drop=drop, seed=3, wait_budget=3000)
    timed_out = p.run()
    name = {PRODUCER: "producer", MMA: "mma", SCALE: "scale", EPILOGUE: "epilogue"}[role]
    # the role that depends on the missing arrival ends in a wait that ran out; the status word holds the code of
    # whichever blocked role had been waiting longest (a role stalled behind the dependent one may get there first)
    assert timed_out.get(name) == role, timed_out
    assert p.status in (PRODUCER, MMA, SCALE, EPILOGUE) and p.abort
    # ... and every other role left its loop instead of hanging
    assert set(timed_out) | p.finished == {"producer", "scale", "mma", "epilogue"}
