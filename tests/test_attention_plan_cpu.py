"""Host-side decisions of the decode attention and of the captured steps (no GPU needed): how many
CTAs share a single-token row's keys, and which context class a step is replayed from."""
from types import SimpleNamespace

import pytest

from dispec_b200.engine import SeqEntry
from dispec_b200.engine.runner import GRAPH_CONTEXT_CLASSES, ModelRunner
from dispec_b200.ops import tuning as A

SLOTS = 2 * 148  # resident CTA slots of the device the plan is made for (two per SM)


@pytest.mark.parametrize("rows", [1, 2, 3, 8, 31, 64, 256])
@pytest.mark.parametrize("kv_heads", [1, 2, 8])
def test_key_sharing_of_single_token_rows(rows, kv_heads):
    last = 0
    for ctx in (1, 100, 255, 256, 1100, 2048, 4096, 8192, 32768, 131072, 1 << 20):
        splits = A.choose_splits(rows, kv_heads, ctx, SLOTS)
        outer = A.choose_outer(rows, kv_heads, ctx, splits, SLOTS)
        assert 1 <= splits <= A.CLUSTER_MAX_SPLITS and 1 <= outer <= A.MAX_OUTER
        if outer > 1:
            assert splits == A.CLUSTER_MAX_SPLITS  # ranges only on top of a full cluster
            assert ctx // (splits * outer) >= A.OUTER_MIN_KEYS  # and only while a CTA keeps enough keys
            assert rows * kv_heads * splits * outer <= SLOTS
        assert splits * outer >= last  # a longer context is never shared among fewer CTAs
        last = splits * outer
    assert A.choose_splits(0, kv_heads, 4096, SLOTS) == 1 and A.choose_outer(0, kv_heads, 4096, 8, SLOTS) == 1


def test_key_ranges_fill_the_gpu_for_one_long_request():
    splits = A.choose_splits(1, 2, 32768, SLOTS)
    outer = A.choose_outer(1, 2, 32768, splits, SLOTS)
    assert 2 * splits * outer >= SLOTS // 2  # at least one CTA per SM
    assert A.choose_outer(64, 2, 32768, A.choose_splits(64, 2, 32768, SLOTS), SLOTS) == 1  # many rows need none


@pytest.mark.parametrize("limit", [512, 2048, 5000, 40000, 1 << 21])
def test_context_class_of_a_captured_step(limit):
    runner = SimpleNamespace(max_model_len=limit)
    seen = set()
    for n in (1, 2047, 2048, 2049, 8192, 8193, 32768, 40000, 131072, 131073, 600000):
        if n > limit:
            continue
        entries = [SeqEntry("a", [0], 5, [0]), SeqEntry("b", [0], n - 1, [0])]
        bound = ModelRunner._context_class(runner, entries)
        assert n <= bound <= limit  # the class holds the step's longest request
        assert bound == limit or bound in GRAPH_CONTEXT_CLASSES
        smaller = [c for c in GRAPH_CONTEXT_CLASSES if n <= c < limit]
        assert bound == (min(smaller) if smaller else limit)  # and is the smallest that does
        seen.add(bound)
    assert len(seen) <= len(GRAPH_CONTEXT_CLASSES) + 1
