"""Exhaustive check of the relayout index maps on 8 ranks: for every pair of layouts (tensor-parallel degree, zigzag
context-parallel degree, sequence-sharded or replicated over the tp ranks) every destination rank must assemble exactly
its piece of the stage's [seq, batch] micro-batch from the pieces the source layout leaves on the ranks. Pure index
arithmetic, no process group (the same maps drive both the all-gather path and the peer-memory gather kernel)."""
import itertools

import pytest
import torch

from hetu_galvatron_b200.parallel.reshard import Layout, batch_range, seq_positions, source_map

STAGE, SEQ, BATCH = 8, 64, 16
LAYOUTS = [Layout(tp, cp, sharded) for tp in (1, 2, 4, 8) for cp in (1, 2, 4, 8) if tp * cp <= STAGE
           for sharded in ((False, True) if tp > 1 else (False,))]


def _pieces(layout, x):
    out = []
    for r in range(STAGE):
        lo, hi = batch_range(layout, r, STAGE, BATCH)
        out.append(x[seq_positions(layout, r, SEQ)][:, lo:hi])
    return out


def test_every_layout_covers_the_micro_batch_exactly():
    x = torch.arange(SEQ * BATCH).view(SEQ, BATCH)
    for lay in LAYOUTS:
        seen = torch.zeros(SEQ, BATCH, dtype=torch.int64)
        for r in range(STAGE):
            lo, hi = batch_range(lay, r, STAGE, BATCH)
            pos = seq_positions(lay, r, SEQ)
            assert pos.numel() == SEQ // lay.seq_parts() and len(set(pos.tolist())) == pos.numel()
            seen[pos.view(-1, 1), torch.arange(lo, hi).view(1, -1)] += 1
        copies = 1 if (lay.seq_sharded or lay.tp == 1) else lay.tp          # replicas over the tp ranks
        assert (seen == copies).all(), lay
    # zigzag: rank c of cp ranks owns chunks c and 2cp-1-c
    pos = seq_positions(Layout(1, 4, False), 1, SEQ)
    assert pos.tolist() == list(range(8, 16)) + list(range(48, 56))


@pytest.mark.parametrize("old,new", [(a, b) for a, b in itertools.product(LAYOUTS, LAYOUTS) if a != b],
                         ids=lambda l: "tp%d_cp%d_%s" % (l.tp, l.cp, "s" if l.seq_sharded else "r"))
def test_destination_assembles_its_piece_from_the_source_pieces(old, new):
    x = torch.arange(SEQ * BATCH).view(SEQ, BATCH)
    src = _pieces(old, x)
    want = _pieces(new, x)
    rows_old, cols_old = SEQ // old.seq_parts(), BATCH // old.dp(STAGE)
    stacked = torch.stack(src)                                    # [rank, rows_old, cols_old]
    assert stacked.shape == (STAGE, rows_old, cols_old)
    for d in range(STAGE):
        src_rank, src_row, src_col = source_map(old, new, d, STAGE, BATCH, SEQ)
        assert src_rank.min() >= 0 and src_rank.max() < STAGE
        assert src_row.max() < rows_old and src_col.max() < cols_old
        got = stacked[src_rank, src_row.view(-1, 1), src_col.view(1, -1)]
        assert torch.equal(got, want[d]), (old, new, d)
