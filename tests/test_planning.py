"""Host-side planning of steps: the launch plan the attention mixer derives from a step's shape (query tiles, the
key ranges of the split decode attention), and which context bound a captured decode graph gets.  No GPU needed."""
import numpy as np
import pytest

from cisr_b200.config import PartSpec
from cisr_b200.engine.batch import HostBatch, unique_planners
from cisr_b200.engine.graph import MIN_CONTEXT_BUCKET, context_bucket_of
from cisr_b200.ops import kernels
from cisr_b200.parts import MIXERS, build_part
from cisr_b200.parts.attention import CLUSTER_MAX, DECODE_RANGE, decode_ranges


def attention(heads=6, kv_heads=2, dim=32):
    import torch
    spec = PartSpec("gqa_attention", {"hidden_size": heads * dim, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": dim,
                                      "window": None, "position": PartSpec("rotary_half", {"theta": 1e4, "dim": dim})})
    return build_part(MIXERS, spec, torch.bfloat16, "mixer")


def host_batch(q_len, ctx_len, bound=None):
    starts = [int(sum(q_len[:i])) for i in range(len(q_len))]
    return HostBatch([f"r{i}" for i in range(len(q_len))], list(range(len(q_len))), starts, list(q_len), list(ctx_len), int(sum(q_len)),
                     [], ctx_bound=bound)


@pytest.mark.parametrize("longest", [1, 63, 64, 255, 256, 257, 4096, 5000, 100_000])
def test_decode_ranges_cover_the_context(longest):
    n = decode_ranges(longest)
    assert n * DECODE_RANGE >= longest                                # every key is in a range
    if n <= CLUSTER_MAX:
        assert (n - 1) * DECODE_RANGE < longest                      # and no range is wholly beyond the context ...
    else:
        assert n % CLUSTER_MAX == 0 and (n - CLUSTER_MAX) * DECODE_RANGE < longest   # ... unless added to fill a cluster


def test_the_split_of_a_request_does_not_depend_on_its_neighbours():
    """Ranges are DECODE_RANGE keys in absolute positions whatever else is in the step: a request's keys are summed in
    the same order alone, beside sixty others, or beside a much longer one (whose extra ranges are empty for it)."""
    mixer = attention()
    alone = mixer.step_plan(host_batch([1], [700]))
    crowd = mixer.step_plan(host_batch([1] * 61, [700] + [90] * 60))
    beside_long = mixer.step_plan(host_batch([1, 1], [700, 9000]))
    assert alone.info["n_splits"] == crowd.info["n_splits"] == 3
    assert beside_long.info["n_splits"] >= 36 and beside_long.info["n_splits"] % CLUSTER_MAX == 0
    assert crowd.info["n_decode"] == 61 and list(crowd.arrays["dec_req"]) == list(range(61))


def test_attention_plan_lists_tiles_longest_first_and_single_tokens_apart():
    mixer = attention()
    plan = mixer.step_plan(host_batch([150, 1, 2, 1], [150, 40, 12, 300]))
    assert plan.info == {"n_tiles": 4, "n_wide": 3, "n_decode": 2, "n_splits": 2}
    assert list(plan.arrays["dec_req"]) == [1, 3]
    tiles = list(zip(plan.arrays["tile_req"], plan.arrays["tile_q0"]))
    assert tiles == [(0, 2 * kernels.PREFILL_TILE), (0, kernels.PREFILL_TILE), (0, 0), (2, 0)]       # a portion's last tile first
    assert list(zip(plan.arrays["wide_req"], plan.arrays["wide_q0"])) == [(0, kernels.WIDE_TILE), (0, 0), (2, 0)]
    assert all(a.dtype == np.int32 for a in plan.arrays.values())


def test_a_plan_made_for_a_bound_serves_every_context_below_it():
    """A captured graph is replayed with other lengths: its plan comes from the bucket, not from the lengths of the day."""
    mixer = attention()
    a = mixer.step_plan(host_batch([1, 1], [10, 20], bound=2048))
    b = mixer.step_plan(host_batch([1, 1], [2000, 5], bound=2048))
    assert a.info == b.info and a.info["n_splits"] == 2048 // DECODE_RANGE
    assert all((a.arrays[k] == b.arrays[k]).all() for k in a.arrays)
    # portions of several tokens are not bounded by it: their tiles depend on their length alone
    c = mixer.step_plan(host_batch([300], [5000], bound=0))
    assert c.info["n_decode"] == 0 and c.info["n_wide"] == 3


def test_layers_with_the_same_geometry_share_one_plan():
    layers = [attention(), attention(), attention(heads=4, kv_heads=4, dim=64)]
    assert len(unique_planners(layers)) == 1           # the plan depends on tile sizes and the range size, not on head counts
    assert unique_planners([object()]) == []


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
