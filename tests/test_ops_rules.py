"""Launch rules of the Python face of the kernels that are plain arithmetic on a step's shape (no GPU needed)."""
from kvad_b200.ops import Ops


def test_decode_key_ranges_keep_a_launch_one_wave():
    sms = 148
    for heads in (1, 3, 12, 16, 25, 40):
        for rows in list(range(1, 70)) + [128, 500]:
            for table_width in (1, 4, 16, 64):
                s = Ops.decode_splits(rows, heads, table_width, n_sms=sms)
                assert 1 <= s <= min(6, table_width)
                if s > 1:
                    assert s * rows * heads <= 2.75 * sms            # more than one range only while that stays one wave
                if s < min(6, table_width):
                    assert (s + 1) * rows * heads > 2.75 * sms       # and as many ranges as fit it
    # the batch sizes the rule was measured at (12 heads): see Ops.decode_splits
    assert [Ops.decode_splits(r, 12, 16, n_sms=sms) for r in (1, 2, 4, 8, 12, 16, 20, 24, 64)] == [6, 6, 6, 4, 2, 2, 1, 1, 1]
    # it depends on the device's size, not on a constant
    assert Ops.decode_splits(8, 12, 16, n_sms=74) == 2
