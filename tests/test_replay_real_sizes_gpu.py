"""bin/trace_run at the real layer sizes (Qwen2.5-1.5B, 7B and 14B: head size 128, groups of 6,
7 and 5 query heads per KV head, widths 1536 to 18944, vocabularies of 151,936 and 152,064, tied
and untied) against the plain implementation on the CPU: the four ways of running the same
requests, in float32 and in bfloat16; the bfloat16 run replays its single-token steps from
captured CUDA graphs, as serving does.  Two or three layers only (the layers are the real
ones; there are fewer of them), and the logits of a subset of positions, so that the CPU side
stays in seconds.

The reference checks its runner the same way, against a trusted model in float32, whole and
token by token across a page edge (puneethgv/DiSpec tests/test_qwen3.py:67-89,
tests/test_runner_correctness.py:55-109)."""
import shutil

import pytest
import torch

import plain_qwen2 as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

LENGTHS = [300, 70]


def wanted(length):
    """Positions whose logits are compared: the first tokens, both sides of the first page edges,
    every 41st, and the last 34 (all of the tokens that run one by one, and two before them)."""
    keep = {0, 1, 2, 15, 16, 17, 31, 32, 63, 64, 65, 127, 128, 129, 255, 256, 257}
    keep |= set(range(0, length, 41)) | set(range(max(0, length - 34), length))
    return sorted(p for p in keep if p < length)


@pytest.mark.parametrize("name", ["1.5b", "7b", "14b"])
def test_replay_real_layer_sizes(name, tmp_path):
    spec = ru.REAL_SHAPES[name]
    model_dir = str(tmp_path / "model")
    config, weights = ru.make_real_model_folder(model_dir, name)
    vocab = config["vocab_size"]
    prompts = {f"p{n}": ru.random_ids(n, vocab, 500 + n) for n in LENGTHS}
    rows = {f"p{n}": wanted(n) for n in LENGTHS}
    refs = {}
    for pname, ids in prompts.items():
        logits = plain.forward_logits(weights, config, ids, rows=rows[pname])
        refs[pname] = dict(zip(rows[pname], logits))
    del weights
    trace, peak = ru.build_four_mode_trace(prompts, spec["page_size"], want=lambda pname, pos: pos in refs[pname])
    for dtype in ("float32", "bfloat16"):
        out_dir = str(tmp_path / f"out_{dtype}")
        got = ru.run_trace(model_dir, dtype, trace, peak, out_dir, page_size=spec["page_size"],
                           cuda_graph=dtype == "bfloat16", timeout=900)
        shutil.rmtree(out_dir)
        modes = set()
        for (step, rid, pos), row in sorted(got.items(), key=lambda kv: kv[0]):
            mode, pname = rid.split("/")
            modes.add(mode.rstrip("01"))
            ref = refs[pname][pos]
            assert torch.isfinite(row).all(), (dtype, step, rid, pos)
            err = (row - ref).abs().max().item()
            scale = max(ref.abs().max().item(), 1e-3)
            where = f"{dtype}: first wrong place: step {step} request {rid} position {pos}: {err} (scale {scale})"
            if dtype == "float32":
                assert err <= 1e-4, where
                top2 = ref.topk(2).values
                if (top2[0] - top2[1]).item() > 1e-3:
                    assert int(row.argmax()) == int(ref.argmax()), where
            else:
                assert err <= 0.03 * scale + 0.02, where
                if ref.topk(2).values.diff().abs().item() > 0.1 * scale:
                    assert int(row.argmax()) == int(ref.argmax()), where
        assert modes == {"whole", "tail", "portions", "mixed"}
        del got
