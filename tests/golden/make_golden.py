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

Two more things are pinned on DiSpec's own output.  ``golden_sampling.pt``: the distribution
``dispec.sampling.logits_to_probs`` draws from, for a dozen (temperature, top_k, top_p) cases
over float64 logits that include ties at the k-th value and a token that crosses top_p.
``golden_<name>.pt["streams"]``: the greedy token streams of DiSpec's
``ContinuousBatchingEngine`` (dispec/sched/scheduler.py) on the CPU in float32 for the
configuration's workload with ``chunk_size=16``, ``max_batch_tokens=32`` and 24 pages, so that
prompts are cut into portions and run beside decoded tokens of other requests.
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
        seed=0, std=0.02, page_size=16, prompt_lens=[5, 17, 33], new_tokens=8),
    "b": dict(
        config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3,
                    hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                    intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
                    hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=512,
                    use_sliding_window=False),
        seed=1, std=0.05, page_size=8, prompt_lens=[1, 9, 40, 64], new_tokens=12),
}


def prompts_for(name, spec):
    g = torch.Generator().manual_seed(1000 + spec["seed"])
    vocab = spec["config"]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in spec["prompt_lens"]]


SAMPLING_CASES = [
    # temperature, top_k, top_p
    (0.0, 0, 1.0), (1.0, 0, 1.0), (0.8, 0, 1.0), (1.7, 5, 1.0), (1.0, 2, 1.0), (1.0, 1, 1.0),
    (1.0, 0, 0.9), (0.6, 0, 0.5), (1.3, 10, 0.7), (1.0, 50, 0.999), (2.5, 3, 0.2), (1.0, 0, 0.05),
]


def sampling_logits():
    """Rows of float64 logits: random ones, three tokens tied at the top (top_k = 2 keeps all
    three), a tie at the k-th value further down, and a flat tail behind one heavy token."""
    g = torch.Generator().manual_seed(77)
    rows = [torch.randn(50, generator=g, dtype=torch.float64) * 2 for _ in range(3)]
    tie_top = torch.full((50,), -5.0, dtype=torch.float64)
    tie_top[[3, 9, 40]] = 2.0
    tie_kth = torch.randn(50, generator=g, dtype=torch.float64)
    tie_kth[[7, 21]] = 3.0
    tie_kth[[30, 31, 32]] = 1.5  # ranks 3 to 5
    heavy = torch.zeros(50, dtype=torch.float64)
    heavy[11] = 4.0
    return torch.stack(rows + [tie_top, tie_kth, heavy])


def golden_sampling():
    from dispec.sampling import SamplingParams, logits_to_probs
    logits = sampling_logits()
    out = {"logits": logits, "cases": SAMPLING_CASES, "probs": []}
    for t, k, p in SAMPLING_CASES:
        out["probs"].append(logits_to_probs(logits.clone(), SamplingParams(temperature=t, top_k=k, top_p=p)))
    torch.save(out, os.path.join(HERE, "golden_sampling.pt"))
    print("sampling", len(SAMPLING_CASES), "cases x", tuple(logits.shape))


def scheduler_streams(model, spec, prompts):
    """Greedy streams of DiSpec's continuous-batching engine under chunked prefill."""
    from dispec.config import KVConfig
    from dispec.sampling import SamplingParams
    from dispec.sched.scheduler import ContinuousBatchingEngine
    eng = ContinuousBatchingEngine(model, kv=KVConfig(block_size=spec["page_size"]), num_blocks=24,
                                   max_batch_tokens=32, chunk_size=16)
    ids = [eng.add_request(p, spec["new_tokens"], SamplingParams(0.0)) for p in prompts]
    eng.run_until_done()
    outs = eng.collect_outputs()
    return {"tokens": [list(outs[i]) for i in ids], "steps": eng.num_steps, "chunk_size": 16,
            "max_batch_tokens": 32, "num_blocks": 24, "new_tokens": spec["new_tokens"]}


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
        out["streams"] = scheduler_streams(model, spec, out["prompts"])
        torch.save(out, os.path.join(HERE, f"golden_{name}.pt"))
        print(name, [tuple(t.shape) for t in out["whole"]], out["streams"]["steps"], "scheduler steps",
              json.dumps(spec["config"])[:60])
    golden_sampling()


if __name__ == "__main__":
    main()
