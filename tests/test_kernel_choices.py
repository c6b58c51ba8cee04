"""Host-side choices in front of the kernels (no GPU needed): how many key splits the decode attention takes."""

import itertools

from tesseract_b200 import kernels


def resident_ctas(head_dim):
    return (2 if head_dim <= 128 else 1) * kernels._SM_COUNT


def test_split_counts_keep_every_cta_resident():
    for seqs, heads, context, head_dim in itertools.product((1, 2, 3, 8, 16, 64, 200), (1, 2, 8), (1, 17, 500, 2184, 32768, 131072),
                                                            (16, 64, 128, 256)):
        splits = kernels.attention_splits(seqs, heads, context, head_dim)
        assert 1 <= splits <= 32
        if splits > 1:
            assert splits * seqs * heads <= resident_ctas(head_dim), (seqs, heads, context, head_dim, splits)
        tiles = -(-context // 16)
        assert splits <= max(1, tiles), "never more splits than tiles of keys"


def test_split_counts_follow_the_measurements():
    # batch 8 of the 1B sizes: four splits as one cluster; batch 64: none; one long sequence: as many as fit
    assert kernels.attention_splits(8, 8, 2184, 64) == 4
    assert kernels.attention_splits(64, 8, 2184, 64) == 1
    assert kernels.attention_splits(1, 8, 131072, 64) == 32
    # wide heads: two CTAs per SM as well, so batch 8 still takes four
    assert kernels.attention_splits(8, 8, 2184, 128) == 4
    # short contexts are not worth a merge
    assert kernels.attention_splits(8, 8, 40, 64) == 1


def test_row_limits_of_the_products():
    assert kernels.DECODE_LINEAR_MAX_ROWS == kernels.DECODE_LINEAR_NORMED_MAX_ROWS == 16
    assert kernels.FUSED_GATE_UP_MIN_ROWS == kernels.DECODE_LINEAR_MAX_ROWS + 1
