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
