"""Rank layout of every group kind on a 16-rank job (reference: galvatron/core/runtime/comm_groups.py:71-236: TP / SP
consecutive blocks, CP strided by tp, DP strided by tp x cp, PP strided by world / pp, embedding group = {first, last}
stage). Pure enumeration, no process group is created."""
import itertools

import pytest

from hetu_galvatron_b200.parallel.mesh import Mesh


def _partition(groups, world):
    flat = sorted(r for g in groups for r in g)
    return flat == list(range(world))


@pytest.mark.parametrize("world,pp", [(8, 1), (8, 2), (16, 2), (16, 4)])
def test_groups_partition_the_world(world, pp):
    m = Mesh(world, 0, pp)
    S = world // pp
    assert m.stage_size == S
    assert m.enumerate_groups("world") == [list(range(world))]
    assert _partition(m.enumerate_groups("stage"), world)
    assert m.enumerate_groups("pp") == [[s * S + i for s in range(pp)] for i in range(S)]
    for tp, cp in itertools.product((1, 2, 4), (1, 2, 4)):
        if S % (tp * cp):
            continue
        for kind in ("tp", "cp", "tpcp", "dp"):
            groups = m.enumerate_groups(kind, tp, cp)
            assert _partition(groups, world), (kind, tp, cp)
            size = {"tp": tp, "cp": cp, "tpcp": tp * cp, "dp": S // (tp * cp)}[kind]
            assert all(len(g) == size for g in groups)
            assert all(len({r // S for r in g}) == 1 for g in groups)          # never across pipeline stages
        assert _partition(m.enumerate_groups("wdp", tp), world)


def test_strides_match_the_reference_layout():
    m = Mesh(16, 0, 2)                                   # two stages of 8
    assert m.enumerate_groups("tp", 2)[:2] == [[0, 1], [2, 3]]                    # consecutive
    assert m.enumerate_groups("cp", 2, 2)[:2] == [[0, 2], [1, 3]]                 # strided by tp
    assert m.enumerate_groups("dp", 2, 2)[:2] == [[0, 4], [1, 5]]                 # strided by tp x cp
    assert m.enumerate_groups("tpcp", 2, 2)[0] == [0, 1, 2, 3]
    assert m.enumerate_groups("wdp", 2)[:2] == [[0, 2, 4, 6], [1, 3, 5, 7]]       # same weight shard: cp and dp ranks
    assert m.enumerate_groups("wdp", 1)[0] == list(range(8))                      # Ulysses / no TP: the whole stage
    assert m.enumerate_groups("pp")[3] == [3, 11]
    assert m.enumerate_groups("embed")[3] == [3, 11]                              # first and last stage
    assert Mesh(8, 0, 1).enumerate_groups("embed") == [[i] for i in range(8)]
    assert Mesh(16, 0, 4).enumerate_groups("embed")[1] == [1, 13]


def test_coordinates_and_neighbours():
    for rank in range(16):
        m = Mesh(16, rank, 2)
        c = m.coords(2, 2)
        assert rank == m.stage * 8 + c["dp"] * 4 + c["cp"] * 2 + c["tp"] and c["dp_size"] == 2
        prev, nxt = m.pp_prev_next()
        assert prev == (rank - 8 if rank >= 8 else None) and nxt == (rank + 8 if rank < 8 else None)
        assert rank in m.enumerate_groups("tp", 2)[rank // 2]
    with pytest.raises(AssertionError):
        Mesh(6, 0, 4)
