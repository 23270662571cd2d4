"""Host-side planning of decode steps: how the keys of a step are split into ranges, and which context bound a
captured decode graph gets.  No GPU needed."""
import pytest

from cisr_b200.engine.batch import CLUSTER_MAX, CTA_TARGET, SPLIT_MIN, SPLIT_QUANTUM, plan_decode_splits
from cisr_b200.engine.graph import MIN_CONTEXT_BUCKET, context_bucket_of


@pytest.mark.parametrize("n_decode", [1, 2, 8, 33, 64, 200])
@pytest.mark.parametrize("kv_heads", [1, 3, 8])
@pytest.mark.parametrize("max_ctx", [1, 63, 64, 257, 4096, 5000, 100_000])
def test_decode_split_plan_covers_the_context_in_whole_ranges(n_decode, kv_heads, max_ctx):
    size, n_splits = plan_decode_splits(n_decode, kv_heads, max_ctx)
    assert size % SPLIT_QUANTUM == 0 and size >= SPLIT_MIN          # ranges start at multiples of 64 keys; a tile per warp
    assert size * n_splits >= max_ctx                                # every key is in a range
    if n_splits <= CLUSTER_MAX:
        assert size * (n_splits - 1) < max_ctx                       # and no range is wholly beyond the context ...
    else:
        assert n_splits % CLUSTER_MAX == 0                           # ... unless ranges were added to fill a cluster
        assert size * (n_splits - CLUSTER_MAX) < max_ctx
    # one wave: not more CTAs than the target unless ranges are already at their smallest
    assert n_decode * kv_heads * -(-max_ctx // size) <= max(CTA_TARGET, n_decode * kv_heads) or size == SPLIT_MIN


def test_the_split_does_not_depend_on_which_requests_share_the_step():
    """Ranges are cut in absolute positions, so a key falls into the same range whatever the other requests are."""
    size_a, _ = plan_decode_splits(8, 3, 4096)
    size_b, _ = plan_decode_splits(8, 3, 4000)
    assert size_a == size_b                                          # same batch, a slightly shorter context: the same cut


@pytest.mark.parametrize("n", [1, 255, 256, 257, 1024, 1025, 1280, 1281, 2048, 2049, 4096, 4097, 65_537])
def test_context_buckets_waste_at_most_a_fifth(n):
    b = context_bucket_of(n)
    assert b >= n and b >= MIN_CONTEXT_BUCKET
    assert context_bucket_of(b) == b                                 # a bucket is its own bucket
    if n > 1024:
        assert (b - n) / b < 0.2
    if n > MIN_CONTEXT_BUCKET:
        assert context_bucket_of(n - 1) <= b                          # monotone


def test_which_tokens_counts_take_the_tcgen05_product():
    """The plain product goes to tcgen05 from one 128-row tile on; the product whose epilogue rotates and writes the
    cache replaces two launches and is taken from 17 tokens on; 16 and fewer belong to the weight-streaming kernels."""
    import torch
    from cisr_b200.ops import kernels as k

    w = torch.zeros(192, 64, dtype=torch.bfloat16)
    for tokens, plain, fused in ((16, False, False), (17, False, True), (127, False, True), (128, True, True), (2048, True, True)):
        a = torch.zeros(tokens, 64, dtype=torch.bfloat16)
        assert k.tcgen05_ok(a, w) is plain and k.tcgen05_ok(a, w, fused=True) is fused, tokens
    assert not k.tcgen05_ok(torch.zeros(256, 64), w)                                   # float32 operands: the library
    assert not k.tcgen05_ok(torch.zeros(256, 60, dtype=torch.bfloat16), w[:, :60])     # rows that are no multiple of 16 bytes
    assert k.tcgen05_rope_ok(64, 32, False) and k.tcgen05_rope_ok(128, 64, False)
    assert not k.tcgen05_rope_ok(64, 16, False) and not k.tcgen05_rope_ok(64, 32, True) and not k.tcgen05_rope_ok(48, 24, False)
