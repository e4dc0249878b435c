"""Helpers of the replay tests: tiny configurations, model folders, trace building, and a
driver for bin/trace_run."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Two configurations that differ in every size and option, and a third with window layers.
CONFIG_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
                hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                hidden_act="silu", tie_word_embeddings=True, max_position_embeddings=512,
                use_sliding_window=False)
CONFIG_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3,
                hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                intermediate_size=224, vocab_size=384, rope_parameters={"rope_theta": 1000000.0,
                                                                        "rope_type": "default"},
                rms_norm_eps=1e-5, hidden_act="silu", tie_word_embeddings=False,
                max_position_embeddings=1024, use_sliding_window=False)
CONFIG_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=4,
                hidden_size=80, num_attention_heads=10, num_key_value_heads=2, head_dim=48,
                intermediate_size=176, vocab_size=203, rope_theta=50000.0, rms_norm_eps=3e-6,
                hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=2048,
                use_sliding_window=True, sliding_window=24,
                layer_types=["full_attention", "sliding_attention", "sliding_attention",
                             "full_attention"])
# sizes that no fast path takes: a width that is no multiple of 8, an intermediate size that is
# no multiple of 16, one query head per KV head, a prime vocabulary
CONFIG_D = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
                hidden_size=100, num_attention_heads=4, num_key_value_heads=4, head_dim=16,
                intermediate_size=150, vocab_size=211, rope_theta=777.0, rms_norm_eps=2e-6,
                hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=512,
                use_sliding_window=False)
# head size 64: portions of prompts run on the tcgen05 attention kernel, one layer with a window
CONFIG_E = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
                hidden_size=72, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
                intermediate_size=160, vocab_size=300, rope_theta=20000.0, rms_norm_eps=1e-5,
                hidden_act="silu", tie_word_embeddings=True, max_position_embeddings=2048,
                use_sliding_window=True, sliding_window=50,
                layer_types=["sliding_attention", "full_attention"])
TINY = {
    "a": dict(config=CONFIG_A, seed=0, std=0.02, page_size=16),
    "b": dict(config=CONFIG_B, seed=1, std=0.05, page_size=8),
    "c": dict(config=CONFIG_C, seed=7, std=0.04, page_size=16),
    "d": dict(config=CONFIG_D, seed=9, std=0.06, page_size=32),
    "e": dict(config=CONFIG_E, seed=4, std=0.05, page_size=8),
    # configuration A with room for long contexts
    "a_long": dict(config=dict(CONFIG_A, max_position_embeddings=16384), seed=0, std=0.02, page_size=16),
}


def make_model_folder(folder, name, dtype="bfloat16"):
    """Writes the folder with the package's random-weights mode; returns (config dict, weights
    read back with the safetensors library, independent of the package's reader)."""
    from safetensors.torch import load_file

    from dispec_b200.config import load_model_config
    from dispec_b200.weights import write_random_model

    spec = TINY[name]
    cfg = load_model_config(spec["config"])
    overrides = None if spec["config"]["tie_word_embeddings"] else {"lm_head.weight": 0.5}
    write_random_model(cfg, folder, seed=spec["seed"], std=spec["std"], dtype=dtype, overrides=overrides)
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return config, weights


def random_ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Trace:
    """Accumulates steps; remembers which (request, position) each written row belongs to.
    ``want(request id, position) -> bool`` says which positions' logits are asked for
    (default: all)."""

    def __init__(self, want=None):
        self.steps = []
        self.rows = {}  # step -> list of (request, position)
        self._stored = {}
        self._want = want or (lambda rid, pos: True)

    def step(self, entries, end=()):
        """entries: list of (request id, tokens)."""
        n = len(self.steps)
        rec = {"step": n, "entries": [], "end": list(end)}
        rows = []
        for rid, tokens in entries:
            start = self._stored.get(rid, 0)
            want = [i for i in range(len(tokens)) if self._want(rid, start + i)]
            rec["entries"].append({"id": rid, "tokens": list(tokens), "want": want})
            rows += [(rid, start + i) for i in want]
            self._stored[rid] = start + len(tokens)
        for rid in end:
            self._stored.pop(rid, None)
        self.steps.append(rec)
        self.rows[n] = rows
        return n

    def live_tokens(self):
        return dict(self._stored)


def run_trace(model_dir, dtype, trace, max_tokens, out_dir, page_size=16, poison=True, timeout=600,
              cuda_graph=False):
    """Runs bin/trace_run on the trace; returns {(step, request, position): logits row}."""
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    if poison:
        cmd.append("--poison-freed-pages")
    if cuda_graph:
        cmd.append("--cuda-graph")
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    if proc.returncode != 0:
        raise RuntimeError(f"trace_run exited with {proc.returncode}\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
    done = [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")]
    assert [int(ln.split()[1]) for ln in done] == list(range(len(trace.steps))), proc.stdout[-500:]
    out = {}
    for n, rows in trace.rows.items():
        if not rows:
            continue
        data = np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4")
        data = data.reshape(len(rows), -1)
        for row, key in zip(data, rows):
            out[(n, key[0], key[1])] = torch.from_numpy(row.copy())
    return out


def build_four_mode_trace(prompts, page_size, want=None):
    """One trace holding all four ways of running the same requests.

    prompts: {name: token ids}.  Request ids are ``<mode>/<name>``.  ``want(name, position)``
    limits the positions whose logits are asked for.  Returns (trace, max live tokens rounded as
    the program's --max-tokens wants them).
    """
    tr = Trace((lambda rid, pos: want(rid.split("/")[1], pos)) if want else None)
    peak = 0
    unit = max(64, page_size)

    def note_peak():
        nonlocal peak
        live = sum((n + unit - 1) // unit * unit for n in tr.live_tokens().values())
        peak = max(peak, live)

    # 1. each request alone and whole
    for name, ids in prompts.items():
        rid = f"whole/{name}"
        tr.step([(rid, ids)])
        note_peak()
        tr.step([], end=[rid])
    # 2. most of it in one step, the last 32 tokens one by one
    for name, ids in prompts.items():
        rid = f"tail/{name}"
        head = max(len(ids) - 32, 0)
        if head:
            tr.step([(rid, ids[:head])])
        for i in range(head, len(ids)):
            tr.step([(rid, ids[i:i + 1])])
        note_peak()
        tr.step([], end=[rid])
    # 3. portions of changing size, down to two tokens
    sizes = [2, 7, 3, 19, 2, 33, 5, 16, 2, 64, 9]
    for name, ids in prompts.items():
        rid = f"portions/{name}"
        pos, k = 0, 0
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            tr.step([(rid, ids[pos:pos + n])])
            pos += n
            k += 1
        note_peak()
        tr.step([], end=[rid])
    # 4. mixed: up to four live; portions of some beside decoded tokens of others; requests end
    #    and new ones take their pages
    names = list(prompts)
    queue = [(f"mixed{r}/{n}", prompts[n]) for r in range(2) for n in names]
    live = []  # [rid, ids, pos, prefill_until]
    k = 0
    while queue or live:
        while queue and len(live) < 4:
            rid, ids = queue.pop(0)
            live.append([rid, ids, 0, max(len(ids) - 12 - (k % 5), 1)])
        entries, ended = [], []
        for item in live:
            rid, ids, pos, until = item
            if pos < until:
                n = min([5, 2, 11, 17, 3][k % 5], until - pos)
            else:
                n = 1
            k += 1
            # now and then a request sits a step out
            if (k % 7) == 0 and len(live) > 1:
                continue
            entries.append((rid, ids[pos:pos + n]))
            item[2] = pos + n
            if item[2] >= len(ids):
                ended.append(rid)
        tr.step(entries, end=ended)
        note_peak()
        live = [it for it in live if it[0] not in ended]
    return tr, peak


# A few layers of the real layer sizes (fewer layers are not a smaller configuration; smaller
# layers would be): head size 128, groups of 6, 7 and 5 query heads per KV head, the real widths
# and vocabularies, tied and untied heads.
REAL_SHAPES = {
    "1.5b": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3,
                             hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                             intermediate_size=8960, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
                             hidden_act="silu", tie_word_embeddings=True, max_position_embeddings=4096,
                             use_sliding_window=False), seed=2, std=0.02, page_size=16),
    "7b": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
                           hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                           intermediate_size=18944, vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-6,
                           hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=4096,
                           use_sliding_window=False), seed=3, std=0.02, page_size=16),
    "14b": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
                            hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                            intermediate_size=13824, vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-5,
                            hidden_act="silu", tie_word_embeddings=False, max_position_embeddings=4096,
                            use_sliding_window=False), seed=4, std=0.02, page_size=16),
}


def make_real_model_folder(folder, name, device="cuda:0"):
    """A folder of a real layer size, its tensors filled on the device (the counter-based
    generator gives the same bits on either side; the CPU would take minutes here).  Returns
    (config dict, weights read back with the safetensors library as float32)."""
    from safetensors.torch import load_file

    from dispec_b200.config import load_model_config
    from dispec_b200.weights import write_random_model

    spec = REAL_SHAPES[name]
    cfg = load_model_config(spec["config"])
    write_random_model(cfg, folder, seed=spec["seed"], std=spec["std"], dtype="bfloat16", device=device)
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return config, weights
