"""bin/trace_run against the plain implementation: the same requests whole, with the last 32
tokens one by one, in portions of changing size down to two tokens, and mixed (up to four
live, portions beside decoded tokens, few pages so that they are used again, freed pages
filled with NaN), in float32 and in bfloat16, for five tiny configurations."""
import pytest
import torch

import plain_qwen2 as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [5, 17, 33, 70], "b": [1, 9, 40, 64, 131], "c": [3, 50, 97, 150], "d": [2, 45, 100],
           "e": [4, 66, 130, 300]}


def check(name, dtype, tmp_path, cuda_graph=False):
    spec = ru.TINY[name]
    model_dir = str(tmp_path / "model")
    config, weights = ru.make_model_folder(model_dir, name, dtype="bfloat16")
    vocab = config["vocab_size"]
    prompts = {f"p{n}": ru.random_ids(n, vocab, 100 + n) for n in LENGTHS[name]}
    trace, peak = ru.build_four_mode_trace(prompts, spec["page_size"])
    got = ru.run_trace(model_dir, dtype, trace, peak, str(tmp_path / "out"), page_size=spec["page_size"],
                       cuda_graph=cuda_graph)
    refs = {n: plain.forward_logits(weights, config, ids) for n, ids in prompts.items()}
    worst = {}
    for (step, rid, pos), row in got.items():
        mode, pname = rid.split("/")
        ref = refs[pname][pos]
        assert torch.isfinite(row).all(), (step, rid, pos)
        err = (row - ref).abs().max().item()
        scale = max(ref.abs().max().item(), 1e-3)
        key = mode.rstrip("01")
        if err / scale > worst.get(key, (0, None))[0]:
            worst[key] = (err / scale, (step, rid, pos, err))
        if dtype == "float32":
            assert err <= 1e-4, f"first wrong place: step {step} request {rid} position {pos}: {err}"
        else:
            assert err <= 0.03 * scale + 0.02, f"first wrong place: step {step} request {rid} position {pos}: {err}"
            if ref.topk(2).values.diff().abs().item() > 0.1 * scale:
                assert int(row.argmax()) == int(ref.argmax()), (step, rid, pos)
    assert set(worst) == {"whole", "tail", "portions", "mixed"}
    return worst


@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_replay_float32(name, tmp_path):
    check(name, "float32", tmp_path)


@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_replay_bfloat16(name, tmp_path):
    check(name, "bfloat16", tmp_path)


@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_replay_bfloat16_single_token_steps_from_captured_graphs(name, tmp_path):
    """The same with --cuda-graph: the steps made of single tokens only (the last 32 tokens of the
    second mode, and the all-decode steps of the mixed mode) are replayed from captured CUDA
    graphs, which is how serving runs them."""
    check(name, "bfloat16", tmp_path, cuda_graph=True)
