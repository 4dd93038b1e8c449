"""Rules that choose how a kernel is launched, as far as they are plain arithmetic (no GPU)."""
import pytest

from flyweight_b200.kernels import attention

SM_COUNT = 148


@pytest.mark.parametrize("head_dim", [64, 128])
def test_the_context_slices_of_a_decode_step_cover_the_context_and_bound_a_cta(head_dim):
    """Every choice of ``decode_splits`` covers all tiles, leaves no slice empty, lets no CTA walk more
    than 128 tiles unless the context needs more than 64 slices of them, merges in a cluster only what a
    cluster can hold, and keeps all CTAs resident at once when that is possible at all."""
    resident = SM_COUNT * (5 if head_dim <= 64 else 3)
    for n_kv in (1, 4, 8):
        for n_tokens in (1, 2, 3, 8, 16, 31, 32, 48, 64, 96, 128, 200, 256, 512, 1000):
            for max_tiles in (1, 2, 7, 8, 9, 17, 64, 65, 129, 257, 513, 1000, 1985, 9000):
                splits, per, in_cluster = attention.decode_splits(n_tokens, n_kv, max_tiles, head_dim)
                what = (n_tokens, n_kv, max_tiles, splits, per, in_cluster)
                assert 1 <= splits <= 64 and per >= 1, what
                assert splits * per >= max_tiles > (splits - 1) * per, what          # covered, no empty slice
                assert per <= 128 or splits >= 32, what
                if in_cluster:
                    assert 1 < splits <= 8 and n_tokens * n_kv * splits <= attention.CLUSTER_MERGE_CTAS, what
                pairs = n_tokens * n_kv
                if pairs <= resident and max_tiles <= 128:
                    assert pairs * splits <= resident or splits == 1, what            # one round of the SMs


def test_the_measured_points_of_the_slicing_rule():
    """The choices the rule was fitted to (8 KV heads, head size 64; tiles of 64 keys)."""
    chosen = lambda batch, tiles: attention.decode_splits(batch, 8, tiles)
    assert chosen(8, 65) == (8, 9, True)            # 8 x 4,096 keys: eight slices in a cluster
    assert chosen(16, 65)[0] == 4 and chosen(32, 65)[0] == 2
    assert chosen(48, 65)[0] == 1 and chosen(64, 65)[0] == 1 and chosen(256, 9)[0] == 1
    assert chosen(128, 65)[0] == 2                  # one piece would be 1.4 rounds of the SMs
    assert chosen(8, 513) == (8, 65, True)          # 8 x 32,768 keys
    assert chosen(1, 1985)[0] >= 32 and not chosen(1, 1985)[2]      # one long request: a merge kernel
