"""The tables of a step, built on the CPU: rows, segments, the tile lists that tiled kernels walk, and what
is refused before anything is launched."""
import numpy as np
import pytest
import torch

from kappai_b200.engine.batch import BatchError, PartTables, Segment, build_step_context
from kappai_b200.parts.attention import BIG_TILE, ROW_TILE, attention_tiles

CPU = torch.device("cpu")


class Tiles:
    """Stands for an attention part: the step tables it asks for."""

    step_tables_key = "tiles"

    def step_tables(self, segs):
        return attention_tiles(segs)


BUILDERS = {"tiles": Tiles()}


def seg(req, n, pos_start, slot, page=16, want=()):
    pages = -(-(pos_start + n) // page)
    table = list(range(100 * slot, 100 * slot + pages))
    slots = [table[p // page] * page + p % page for p in range(pos_start, pos_start + n)]
    return Segment(req=req, tokens=list(range(n)), pos_start=pos_start, want=list(want), slot=slot,
                   block_tables={"g": table}, token_slots={"g": slots})


def test_rows_segments_and_slots():
    ctx = build_step_context([seg("a", 5, 0, 0, want=[4]), seg("b", 1, 37, 1, want=[0]), seg("c", 3, 16, 2)],
                             {"g": 16}, CPU, 1000, 4096)
    assert ctx.n_rows == 9 and ctx.n_seg == 3 and ctx.n_out == 2
    assert ctx.positions.tolist() == [0, 1, 2, 3, 4, 37, 16, 17, 18]
    assert ctx.row_seg.tolist() == [0] * 5 + [1] + [2] * 3
    assert ctx.cu_rows.tolist() == [0, 5, 6, 9]
    assert ctx.logit_rows.tolist() == [4, 5]
    assert ctx.max_seg_len == 5 and ctx.max_context == 38 and not ctx.decode_only
    view = ctx.paged["g"]
    assert view.slot_map.tolist()[5] == (100 + 2) * 16 + 5          # position 37 of b: third page, offset 5


def test_tile_lists_cover_every_row_once_and_big_tiles_come_longest_first():
    segs = [seg("a", 300, 0, 0), seg("b", 1, 900, 1), seg("c", 130, 512, 2), seg("d", 64, 64, 3)]
    full = build_step_context(segs, {"g": 16}, CPU, 1000, 4096, BUILDERS)
    ctx = full.tables["tiles"]
    cu = full.cu_rows.tolist()
    for size, t_seg, t_row0 in ((ROW_TILE, ctx.tile_seg, ctx.tile_row0), (BIG_TILE, ctx.big_tile_seg, ctx.big_tile_row0)):
        covered = np.zeros(full.n_rows, int)
        for s, r0 in zip(t_seg.tolist(), t_row0.tolist()):
            assert cu[s] <= r0 < cu[s + 1] and (r0 - cu[s]) % size == 0
            covered[r0:min(r0 + size, cu[s + 1])] += 1
        assert (covered == 1).all()
    assert ctx.n_tiles == len(ctx.tile_seg) and ctx.n_big_tiles == len(ctx.big_tile_seg)
    # the position of a big tile's last row never grows along the list
    last = []
    for s, r0 in zip(ctx.big_tile_seg.tolist(), ctx.big_tile_row0.tolist()):
        end = min(r0 + BIG_TILE, cu[s + 1])
        last.append(segs[s].pos_start + end - cu[s] - 1)
    assert last == sorted(last, reverse=True)
    assert last[0] == 900


def test_decoded_tokens_that_lead_a_mixed_step_are_set_apart():
    segs = [seg("a", 1, 900, 0), seg("b", 2, 40, 1), seg("c", 300, 0, 2), seg("d", 1, 77, 3)]
    full = build_step_context(segs, {"g": 16}, CPU, 1000, 4096, BUILDERS)
    ctx = full.tables["tiles"]
    assert ctx.n_short_rows == 3 and ctx.n_short_tiles == 2
    assert ctx.tile_seg.tolist()[:2] == [0, 1]                        # the lead's small tiles come first
    assert sorted(set(ctx.big_tile_seg.tolist())) == [2, 3]           # big tiles: the other segments only
    covered = np.zeros(full.n_rows, int)
    cu = full.cu_rows.tolist()
    for s, r0 in zip(ctx.big_tile_seg.tolist(), ctx.big_tile_row0.tolist()):
        covered[r0:min(r0 + BIG_TILE, cu[s + 1])] += 1
    assert covered.tolist() == [0] * 3 + [1] * 301
    # all short, or no short lead: one kernel takes the step, nothing is set apart
    c2 = build_step_context([seg("a", 9, 9, 0), seg("b", 1, 4, 1)], {"g": 16}, CPU, 1000, 4096, BUILDERS).tables["tiles"]
    assert c2.n_short_rows == 0 and c2.n_short_tiles == 0 and c2.n_big_tiles == 2
    # short segments only: the split kernel takes the step and no tile list is built
    assert "tiles" not in build_step_context([seg("a", 1, 9, 0), seg("b", 3, 4, 1)], {"g": 16}, CPU, 1000, 4096,
                                             BUILDERS).tables


def test_a_part_adds_tables_of_its_own_to_the_upload():
    class Scan:
        step_tables_key = "scan"

        def step_tables(self, segs):
            return PartTables(arrays={"seg_end": segs.cu_rows[1:] - 1, "odd": np.arange(3)},
                              scalars={"n_long": sum(n > 2 for n in segs.seg_len)})

    ctx = build_step_context([seg("a", 5, 0, 0), seg("b", 1, 37, 1), seg("c", 3, 16, 2)], {"g": 16}, CPU, 1000, 4096,
                             {"scan": Scan(), **BUILDERS})
    t = ctx.tables["scan"]
    assert t.seg_end.tolist() == [4, 5, 8] and t.odd.tolist() == [0, 1, 2] and t.n_long == 2
    assert t.seg_end.dtype == torch.int32 and ctx.tables["tiles"].n_tiles == 3
    assert ctx.positions.tolist() == [0, 1, 2, 3, 4, 37, 16, 17, 18]          # the fixed tables are where they were


def test_refusals():
    with pytest.raises(BatchError):
        build_step_context([], {"g": 16}, CPU, 10, 64)
    with pytest.raises(BatchError):                                   # token id outside the vocabulary
        build_step_context([seg("a", 12, 0, 0)], {"g": 16}, CPU, 10, 64)
    with pytest.raises(BatchError):                                   # position beyond the limit
        build_step_context([seg("a", 5, 62, 0)], {"g": 16}, CPU, 10, 64)
    with pytest.raises(BatchError):                                   # wanted index outside the portion
        build_step_context([seg("a", 5, 0, 0, want=[5])], {"g": 16}, CPU, 10, 64)
    with pytest.raises(BatchError):                                   # two segments, one state slot
        build_step_context([seg("a", 2, 0, 0), seg("b", 2, 0, 0)], {"g": 16}, CPU, 10, 64)
