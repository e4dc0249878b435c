"""Run once by hand: pins the plain implementation (tests/plain_qwen2.py) against DiSpec.

    PYTHONPATH=<DiSpec checkout> python tests/golden/make_golden.py

DiSpec's forward (dispec/engine/model_runner.py) borrows its weight modules from a
Qwen2ForCausalLM object of the installed transformers package, exactly as its loader
does (dispec/models/loader.py:18-27).  This script builds that object for the two tiny
configurations below, overwrites every parameter by name with weights drawn by
tests/plain_qwen2.random_weights, and runs DiSpec's own ModelRunner + PagedKVCache on
the CPU in float32: whole prompts, and a prompt cut in two portions (17 + rest) so that
the cached path is taken.  The logits are stored in ``golden_<name>.pt`` together with the
config, the seed and the prompts; tests/test_plain_vs_golden.py regenerates the weights
from the seed and compares the plain implementation with these stored logits, so the
test itself needs neither DiSpec nor transformers.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from plain_qwen2 import random_weights  # noqa: E402

CONFIGS = {
    "a": dict(
        config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
                    hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                    intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                    hidden_act="silu", tie_word_embeddings=True, max_position_embeddings=512,
                    use_sliding_window=False),
        seed=0, std=0.02, page_size=16, prompt_lens=[5, 17, 33]),
    "b": dict(
        config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3,
                    hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                    intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
                    hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=512,
                    use_sliding_window=False),
        seed=1, std=0.05, page_size=8, prompt_lens=[1, 9, 40, 64]),
}


def prompts_for(name, spec):
    g = torch.Generator().manual_seed(1000 + spec["seed"])
    vocab = spec["config"]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in spec["prompt_lens"]]


def main():
    from transformers import Qwen2Config, Qwen2ForCausalLM
    from dispec.engine.model_runner import ModelRunner, SeqMeta
    from dispec.kv.paged_cache import PagedKVCache

    for name, spec in CONFIGS.items():
        cfg = {k: v for k, v in spec["config"].items() if k not in ("architectures", "model_type")}
        model = Qwen2ForCausalLM(Qwen2Config(**cfg)).float().eval()
        model.requires_grad_(False)  # as dispec/models/loader.py:25-26 does
        weights = random_weights(spec["config"], spec["seed"], spec["std"])
        state = model.state_dict()
        with torch.no_grad():
            for key, value in weights.items():
                assert state[key].shape == value.shape, key
                state[key].copy_(value)
        missing = set(state) - set(weights) - {"lm_head.weight"}
        assert not missing, missing
        runner = ModelRunner(model)
        bs = spec["page_size"]
        cache = PagedKVCache.for_model(model.config, 64, bs, torch.float32, "cpu")
        out = {"config": spec["config"], "seed": spec["seed"], "std": spec["std"],
               "prompts": prompts_for(name, spec), "whole": [], "split": []}

        def run(sid, ids, start, table):
            pos = torch.arange(start, start + len(ids))
            slots = cache.slots_for_positions(table.block_ids, pos)
            hidden = runner.forward(torch.tensor(ids), pos, slots,
                                    [SeqMeta(table.block_ids, len(ids), start + len(ids))], cache)
            return runner.logits(hidden).float()

        for sid, ids in enumerate(out["prompts"]):
            table = cache.manager.allocate(sid, len(ids))
            out["whole"].append(run(sid, ids, 0, table))
            cache.manager.free(sid)
            cut = min(17, len(ids) - 1)
            if cut >= 1:
                table = cache.manager.allocate(100 + sid, len(ids))
                first = run(100 + sid, ids[:cut], 0, table)
                rest = run(100 + sid, ids[cut:], cut, table)
                out["split"].append(torch.cat([first, rest]))
                cache.manager.free(100 + sid)
            else:
                out["split"].append(None)
        torch.save(out, os.path.join(HERE, f"golden_{name}.pt"))
        print(name, [tuple(t.shape) for t in out["whole"]], json.dumps(spec["config"])[:60])


if __name__ == "__main__":
    main()
