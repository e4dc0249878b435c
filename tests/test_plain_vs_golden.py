"""The plain implementation against logits DiSpec's own runner produced on the CPU
(tests/golden/make_golden.py wrote them; this test needs neither DiSpec nor any model
package)."""
import os

import pytest
import torch

import plain_qwen2 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_matches_reference_runner(name):
    g = torch.load(os.path.join(GOLDEN, f"golden_{name}.pt"))
    weights = plain.random_weights(g["config"], g["seed"], g["std"])
    for ids, whole, split in zip(g["prompts"], g["whole"], g["split"]):
        mine = plain.forward_logits(weights, g["config"], ids)
        assert mine.shape == whole.shape
        assert (mine - whole).abs().max().item() < 2e-6
        if split is not None:
            # the reference's cached, two-portion path agrees with its whole-prompt path
            assert (mine - split).abs().max().item() < 2e-6


def test_float64_truth_is_close():
    g = torch.load(os.path.join(GOLDEN, "golden_b.pt"))
    weights = plain.random_weights(g["config"], g["seed"], g["std"])
    ids = g["prompts"][-1]
    lo = plain.forward_logits(weights, g["config"], ids)
    hi = plain.forward_logits(weights, g["config"], ids, dtype=torch.float64)
    assert (lo.double() - hi).abs().max().item() < 1e-5


def test_sampling_distribution_matches_the_reference():
    """plain.sampling_distribution against the distribution dispec.sampling.logits_to_probs gave
    for the same float64 logits: greedy one-hot, temperature, ties at the k-th value kept by
    top-k, the token that crosses top_p kept, a flat tail.  Where top-p cuts through tokens of
    equal logits, which of them stay depends on the order an unstable sort leaves them in (the
    reference sorts without ``stable``): there the mass per distinct logit value and the number of
    tokens kept are compared, everywhere else every probability."""
    g = torch.load(os.path.join(GOLDEN, "golden_sampling.pt"))
    assert len(g["cases"]) >= 12
    exact = 0
    for (t, k, p), want in zip(g["cases"], g["probs"]):
        for row, ref in zip(g["logits"], want):
            mine = plain.sampling_distribution(row, t, k, p)
            assert int((mine > 0).sum()) == int((ref > 0).sum()), (t, k, p)
            assert (mine.sort().values - ref.sort().values).abs().max().item() < 1e-12, (t, k, p)
            for value in row.unique():
                same = row == value
                assert abs(float(mine[same].sum() - ref[same].sum())) < 1e-12, (t, k, p, float(value))
            if (mine - ref).abs().max().item() < 1e-12:
                exact += 1
            else:  # only a cut through tied tokens may differ
                moved = (mine - ref).abs() > 1e-12
                assert all(int((row == v).sum()) > 1 for v in row[moved].unique()), (t, k, p)
    assert exact >= 60


def streams_agree(weights, config, prompt, got, want, min_margin=1e-4):
    """Compares two greedy streams token by token, teacher-forced on ``want``, and stops at the
    first token whose top-2 margin in the plain implementation is below ``min_margin`` (a tie
    may fall either way, and everything after it differs legitimately).  Returns how many tokens
    were compared."""
    ids = list(prompt)
    for i, (a, b) in enumerate(zip(got, want)):
        last = plain.forward_logits(weights, config, ids)[-1]
        top2 = torch.topk(last, 2).values
        if float(top2[0] - top2[1]) < min_margin:
            return i
        assert a == b, f"token {i}: {a} != {b} (margin {float(top2[0] - top2[1]):.2e})"
        ids.append(b)
    return min(len(got), len(want))


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_greedy_generation_matches_the_reference_scheduler(name):
    """Greedy streams of DiSpec's continuous-batching engine (prompts cut into portions of 16
    under a budget of 32 tokens, 24 pages) against plain whole-sequence generation."""
    g = torch.load(os.path.join(GOLDEN, f"golden_{name}.pt"))
    weights = plain.random_weights(g["config"], g["seed"], g["std"])
    compared = 0
    for prompt, want in zip(g["prompts"], g["streams"]["tokens"]):
        assert len(want) == g["streams"]["new_tokens"]
        mine, _ = plain.greedy_generate(weights, g["config"], prompt, len(want))
        compared += streams_agree(weights, g["config"], prompt, mine, want)
    assert compared >= len(g["prompts"]) * 2
