"""Launch policies decided on the host (no GPU): how the decode attention splits a sequence's keys."""

from types import SimpleNamespace

import pytest

from dryft_b200.parts.attention import Attention


def _splits(max_kv, n_rows, n_kv=8, sms=148, page=64):
    me = SimpleNamespace(rt=SimpleNamespace(page_size=page, sm_count=sms), n_kv=n_kv, CLUSTER_SPLITS=Attention.CLUSTER_SPLITS)
    return Attention._decode_splits(me, max_kv, n_rows)


@pytest.mark.parametrize("max_kv", [1, 64, 512, 1024, 4096, 8192, 16384, 32768, 131072])
@pytest.mark.parametrize("n_rows", [1, 2, 4, 8, 16, 64])
def test_decode_splits_stay_within_one_block_per_sm_where_the_batch_allows(max_kv, n_rows):
    s = _splits(max_kv, n_rows)
    assert 1 <= s <= 32
    pairs = n_rows * 8
    if pairs * Attention.CLUSTER_SPLITS <= 148:
        # few (row, kv head) pairs: no more blocks than SMs, however long the context
        assert pairs * s <= 148
    if max_kv <= 64:
        assert s == 1


def test_decode_splits_of_a_long_single_sequence():
    assert _splits(32768, 1) == 18      # 144 blocks of 8 kv heads: one per SM, not 32 splits
    assert _splits(16384, 1) == 16
    assert _splits(8192, 1) == 8        # up to eight splits are one cluster
    assert _splits(8192, 8) == 2        # batch 8: 64 pairs, two splits each
    assert _splits(4096, 2) == 4        # 16 clusters: of four blocks, not of eight
    assert _splits(4096, 1) == 8
    assert _splits(512, 64) == 1


def test_products_of_nine_to_sixteen_rows_stay_under_the_shared_memory_cut():
    from dryft_b200.ops import kernels as K
    # up to 8 rows: always the register-streaming product, whatever the width
    assert K.fused_rows_supported(8, 5120, 16, 0, normed=True)
    assert K.fused_rows_supported(1, 8192, 16, 0, normed=True)
    # 9 to 16 rows with the norm on the way in: only widths whose 16 staged rows leave a block under 100 KB
    assert K.small_m_staged_bytes(16, 2560) == 2 * 8704 + 256 + 16 * 2592 * 2 + 1024 <= K.SMALL_M_CUT_BYTES
    assert K.fused_rows_supported(16, 2560, 16, 0, normed=True)
    assert not K.fused_rows_supported(10, 4096, 16, 0, normed=True)   # ten rows would fit, sixteen do not
    assert not K.fused_rows_supported(9, 5120, 16, 0, normed=True)
    # plain activations are not staged: no such limit
    assert K.fused_rows_supported(16, 25600, 16, 0)
    # small_m_max still bounds it
    assert not K.fused_rows_supported(9, 2560, 8, 0, normed=True)
