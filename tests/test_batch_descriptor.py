"""The packed step descriptor (CPU): where each array lies, 16-byte alignment of every array, block-table
rows padded with the scratch page, pages already given back replaced by it."""

import torch

from prism_b200.engine.batch import BatchLayout, StepContext, pack_batch


def test_layout_offsets_are_aligned_and_disjoint():
    for T, S, R, W, groups in [(1, 1, 1, 1, [0]), (7, 3, 2, 5, [0, 2]), (33, 4, 33, 9, [1]), (5, 5, 0, 3, [])]:
        lay = BatchLayout(T, S, R, W, groups)
        spans = sorted(lay.off.values())
        for (o, n), (o2, _) in zip(spans, spans[1:]):
            assert o % 4 == 0 and o + n <= o2                  # 4 int32 = 16 bytes; no overlap
        assert spans[-1][0] + spans[-1][1] <= lay.total
        assert set(lay.off) == {"token_ids", "positions", "tok_seg", "seg_start", "cached_len", "q_len",
                                "state_slots", "logit_rows"} | {f"bt{g}" for g in groups}
    lay = BatchLayout(7, 3, 2, 5, [0, 2], {0: 9, 2: 3})
    spans = sorted(lay.off.values())
    for (o, n), (o2, _) in zip(spans, spans[1:]):
        assert o % 4 == 0 and o + n <= o2
    assert lay.off["items0"][1] == 36 and lay.off["items2"][1] == 12 and lay.off["starts0"][1] == 3


def test_pack_and_views():
    # two segments: a decode token of a request that holds 9 tokens, and a 3-token portion after 4 cached ones
    tok, pos, seg_of = [11, 21, 22, 23], [9, 4, 5, 6], [0, 1, 1, 1]
    lay = BatchLayout(4, 2, 2, 4, [0, 1])
    rows = {0: [[5, 2, 7], [3, 1]],            # group 0: all keys
            1: [[-1, -1, 6], [0]]}             # group 1: a window; the first request's early pages were given back
    host = pack_batch(lay, tok, pos, seg_of, [0, 1, 4], [9, 4], [1, 3], [2, 0], [0, 3], rows, {0: 40, 1: 41})
    assert host.dtype == torch.int32 and host.numel() == lay.total
    ctx = StepContext(lay, host, torch.float32, "cpu", None, 64, None, 3, 10)
    assert (ctx.T, ctx.S, ctx.R, ctx.W) == (4, 2, 2, 4) and not ctx.decode_only and ctx.host is None
    assert ctx.token_ids.tolist() == tok and ctx.positions.tolist() == pos and ctx.tok_seg.tolist() == seg_of
    assert ctx.seg_start.tolist() == [0, 1, 4] and ctx.cached_len.tolist() == [9, 4] and ctx.q_len.tolist() == [1, 3]
    assert ctx.state_slots.tolist() == [2, 0] and ctx.logit_rows.tolist() == [0, 3]
    assert ctx.block_tables[0].tolist() == [[5, 2, 7, 40], [3, 1, 40, 40]]
    assert ctx.block_tables[1].tolist() == [[41, 41, 6, 41], [0, 41, 41, 41]]
    assert ctx.decode_work == {}
    # the decode kernel's work items of the leading single-token segment, for group 1; a layout with more places
    # than items marks the rest unused, and the segments after the decoding ones have no items
    import numpy as np
    lay2 = BatchLayout(4, 2, 2, 4, [0, 1], {1: 3})
    items = np.array([[0, 0 | 2 << 16, 9, 0], [0, 1 | 2 << 16, 9, 0]], dtype=np.int32)
    planned = pack_batch(lay2, tok, pos, seg_of, [0, 1, 4], [9, 4], [1, 3], [2, 0], [0, 3], rows, {0: 40, 1: 41},
                         {1: (items, np.array([0 | 2 << 16], dtype=np.int32))})
    ctx2 = StepContext(lay2, planned, torch.float32, "cpu", None, 64, None, 3, 10)
    got_items, got_starts = ctx2.decode_work[1][:2]
    assert got_items.tolist() == items.tolist() + [[-1] * 4] and got_starts.tolist() == [2 << 16, 0]
    assert lay2.off["items1"][0] % 4 == 0 and ctx2.block_tables[1].tolist() == ctx.block_tables[1].tolist()
    # a pure decode step is recognised by its longest segment
    assert StepContext(lay, host, torch.float32, "cpu", None, 64, None, 1, 10).decode_only


def test_rows_longer_than_the_table_are_cut():
    lay = BatchLayout(1, 1, 1, 2, [0])
    host = pack_batch(lay, [1], [0], [0], [0, 1], [0], [1], [0], [0], {0: [[4, 5, 6]]}, {0: 9})
    assert lay.view(host, "bt0").tolist() == [4, 5]
