"""Host-side choices that the kernels' launches rest on, checked without a GPU: how many slices the single-token
attention cuts a sequence into, and when a product normalises its own input."""

import pytest

from sleuth_b200.kernels import ops
from sleuth_b200.parts import linear

SMS = 148


@pytest.mark.parametrize("kv_heads,group", [(8, 2), (2, 4), (1, 16), (4, 40), (16, 1)])
@pytest.mark.parametrize("table_stride", [1, 4, 8, 64, 512])
def test_decode_slices_fill_one_round_and_never_more(kv_heads, group, table_stride):
    row_tiles = (group + 15) // 16
    for n in list(range(1, 70)) + [100, 300]:
        blocks = n * kv_heads * row_tiles
        s = ops.decode_splits(n, kv_heads, group, table_stride, sms=148)
        assert s >= 1
        # a slice holds at least four pages of the longest sequence, unless one slice per pair is all there is
        assert s == 1 or s <= max(1, table_stride // 4) or s == 2
        if blocks <= 2 * SMS:
            # everything runs at once: with three page buffers two blocks fit an SM, with two buffers three
            assert s * blocks <= 3 * SMS
        else:
            assert s == 1 or s * blocks <= 3 * SMS
        # it depends on the batch and the table's width only: the same answer again
        assert s == ops.decode_splits(n, kv_heads, group, table_stride, sms=148)


def test_decode_slices_at_the_benchmark_shapes():
    # 8 kv heads, 2 query heads each, sequences of up to 4,096 keys (64 pages)
    assert ops.decode_splits(1, 8, 2, 64, sms=148) == 16      # capped: four pages a slice
    assert ops.decode_splits(8, 8, 2, 64, sms=148) == 6       # 384 blocks with two page buffers, not 256 with three
    assert ops.decode_splits(12, 8, 2, 64, sms=148) == 3      # 4 for 3 would not pay
    assert ops.decode_splits(16, 8, 2, 64, sms=148) == 3
    assert ops.decode_splits(64, 8, 2, 64, sms=148) == 1


def test_norm_is_fused_only_where_it_was_measured_to_pay():
    assert linear.use_skinny(8, 4096, 1024, norm=True)
    assert linear.use_skinny(1, 4096, 2048, norm=True)
    assert not linear.use_skinny(1, 6144, 4096, norm=True)       # too wide: the norm kernel in front is faster
    assert not linear.use_skinny(16, 4096, 2048, norm=True)      # too many rows for that width
    assert linear.use_skinny(16, 6144, 4096)                     # the plain product still takes it
    assert not linear.use_skinny(linear.SKINNY_ROWS + 1, 1024, 1024)


def test_timeline_groups_block_records_into_launches():
    """Two launches of one kind (the second reuses block numbers), one of another kind in between, out of order."""
    from sleuth_b200.kernels import timeline
    rec = lambda kind, block, enter, go, m2, leave: {"kind": kind, "block": block, "sm": block, "enter": enter,
                                                      "marks": [go, m2, 0], "leave": leave}
    records = [rec("gemm_skinny", 0, 100, 900, 1500, 1700), rec("gemm_skinny", 1, 120, 910, 1600, 1800),
               rec("rmsnorm", 0, 1900, 1950, 0, 2500),
               rec("gemm_skinny", 0, 2000, 2900, 3300, 3500), rec("gemm_skinny", 1, 2600, 2950, 3400, 3600)]
    records.sort(key=lambda r: r["enter"])
    out = timeline.launches(records)
    assert [(L["kind"], L["blocks"]) for L in out] == [("gemm_skinny", 2), ("rmsnorm", 1), ("gemm_skinny", 2)]
    first, norm, second = out
    assert (first["first_enter"], first["last_enter"], first["first_go"], first["last_go"]) == (100, 120, 900, 910)
    assert (first["last_mark2"], first["first_leave"], first["last_leave"]) == (1600, 1700, 1800)
    assert norm["last_mark2"] == 0 and norm["last_leave"] == 2500
    assert (second["first_enter"], second["last_enter"], second["last_leave"]) == (2000, 2600, 3600)
