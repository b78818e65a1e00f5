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
        s = ops.decode_splits(n, kv_heads, group, table_stride)
        assert s >= 1
        # a slice holds at least four pages of the longest sequence, unless one slice per pair is all there is
        assert s == 1 or s <= max(1, table_stride // 4) or s == 2
        if blocks <= 2 * SMS:
            # everything runs at once: with three page buffers two blocks fit an SM, with two buffers three
            assert s * blocks <= 3 * SMS
        else:
            assert s == 1 or s * blocks <= 3 * SMS
        # it depends on the batch and the table's width only: the same answer again
        assert s == ops.decode_splits(n, kv_heads, group, table_stride)


def test_decode_slices_at_the_benchmark_shapes():
    # 8 kv heads, 2 query heads each, sequences of up to 4,096 keys (64 pages)
    assert ops.decode_splits(1, 8, 2, 64) == 16      # capped: four pages a slice
    assert ops.decode_splits(8, 8, 2, 64) == 6       # 384 blocks with two page buffers, not 256 with three
    assert ops.decode_splits(12, 8, 2, 64) == 3      # 4 for 3 would not pay
    assert ops.decode_splits(16, 8, 2, 64) == 3
    assert ops.decode_splits(64, 8, 2, 64) == 1


def test_norm_is_fused_only_where_it_was_measured_to_pay():
    assert linear.use_skinny(8, 4096, 1024, norm=True)
    assert linear.use_skinny(1, 4096, 2048, norm=True)
    assert not linear.use_skinny(1, 6144, 4096, norm=True)       # too wide: the norm kernel in front is faster
    assert not linear.use_skinny(16, 4096, 2048, norm=True)      # too many rows for that width
    assert linear.use_skinny(16, 6144, 4096)                     # the plain product still takes it
    assert not linear.use_skinny(linear.SKINNY_ROWS + 1, 1024, 1024)
