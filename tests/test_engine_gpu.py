"""Generation through the Python entry points against the plain implementation: greedy and
temperature sampling, chunked prompts mixed with decoding, long decoding, the first tokens of
a sequence, and a pool so small that requests are preempted and recomputed."""
import random

import pytest
import torch

import plain_qwen2 as plain
import replay_util as ru

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ("a", "b", "c", "e"):
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        out[name] = (d,) + ru.make_model_folder(d, name, dtype="bfloat16")
    return out


def load(folder, dtype):
    from dispec_b200 import load_model
    return load_model(folder, dtype, "cuda:0")


def replay_sampling(weights, config, prompt, tokens, params):
    """What the plain implementation would have drawn, teacher-forced with the engine's own
    tokens, from the same stream of uniform numbers.  Returns (tokens, smallest margin)."""
    rng = random.Random(params.seed)
    out, margin = [], 1.0
    ids = list(prompt)
    for tok in tokens:
        logits = plain.forward_logits(weights, config, ids)[-1]
        if params.temperature <= 0:
            top2 = torch.topk(logits, 2).values
            margin = min(margin, float(top2[0] - top2[1]))
            out.append(int(logits.argmax()))
        else:
            u = min(rng.random(), 1.0 - 2.0 ** -24)
            probs = plain.sampling_distribution(logits, params.temperature, params.top_k, params.top_p)
            cdf = probs.cumsum(-1)
            want = plain.draw_inverse_cdf(probs, u)
            margin = min(margin, float((cdf - u * cdf[-1]).abs().min()))
            out.append(want)
        ids.append(tok)
    return out, margin


def assert_tokens_within_margin(weights, config, prompt, tokens, params, rel=0.03, floor=0.02):
    """Every token of a bfloat16 stream, teacher-forced: equal to the plain implementation's, or
    the plain decision at that position is closer than bfloat16 can resolve (greedy: top-2 gap
    below 2 * (rel * largest logit + floor); sampled: the uniform number lies within that mass of
    an edge of the cumulative distribution)."""
    rng = random.Random(params.seed)
    ids = list(prompt)
    for i, tok in enumerate(tokens):
        logits = plain.forward_logits(weights, config, ids)[-1]
        reach = 2 * (rel * logits.abs().max().item() + floor)
        if params.temperature <= 0:
            top2 = torch.topk(logits, 2).values
            assert tok == int(logits.argmax()) or float(top2[0] - top2[1]) < reach, (i, tok)
        else:
            u = min(rng.random(), 1.0 - 2.0 ** -24)
            probs = plain.sampling_distribution(logits, params.temperature, params.top_k, params.top_p)
            want = plain.draw_inverse_cdf(probs, u)
            cdf = probs.cumsum(-1)
            # a logit error e moves cumulative masses by at most about e / T of the mass
            edge = float((cdf - u * cdf[-1]).abs().min())
            assert tok == want or edge < reach / max(params.temperature, 1e-3), (i, tok, want, edge)
        ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_through_llm_engine(folders, name, dtype):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders[name]
    engine = LLMEngine(load(folder, dtype), num_blocks=64)
    for n in ([5, 17, 33] if name == "a" else [1, 9, 40]):
        prompt = ru.random_ids(n, config["vocab_size"], 300 + n)
        got = engine.generate(prompt, 8, SamplingParams(temperature=0.0))
        want, margin = replay_sampling(weights, config, prompt, got, SamplingParams())
        if dtype == "float32":
            assert margin > 1e-4 and got == want
        else:
            scale = 0.03 * plain.forward_logits(weights, config, prompt).abs().max().item() + 0.02
            assert got == want or margin < 2 * scale
    assert engine.runner.cache.num_free_pages() == 64


def test_long_decoding_float32(folders):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders["a"]
    engine = LLMEngine(load(folder, "float32"), num_blocks=64)
    prompt = ru.random_ids(3, config["vocab_size"], 1)
    got = engine.generate(prompt, 260, SamplingParams())
    assert len(got) == 260
    # logits of the whole generated sequence, computed once by the plain implementation
    logits = plain.forward_logits(weights, config, prompt + got)
    for i, tok in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        top2 = torch.topk(row, 2)
        if float(top2.values[0] - top2.values[1]) > 1e-4:
            assert int(top2.indices[0]) == tok, i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_continuous_batching_chunked_mixed_greedy_and_temperature(folders, dtype):
    """Config B's workload: prompts of 1, 9, 40, 64 tokens, portions of 16 mixed with decoding,
    12 new tokens each, greedy and temperature 0.8 side by side."""
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["b"]
    engine = ContinuousBatchingEngine(load(folder, dtype), KVConfig(block_size=8), num_blocks=48,
                                      max_batch_tokens=32, chunk_size=16)
    reqs = []
    for i, n in enumerate([1, 9, 40, 64, 9, 40]):
        prompt = ru.random_ids(n, config["vocab_size"], 400 + i)
        params = SamplingParams(temperature=0.8 if i % 2 else 0.0, top_k=40 if i == 3 else 0,
                                top_p=0.9 if i == 5 else 1.0, seed=50 + i)
        reqs.append((engine.add_request(prompt, 12, params), prompt, params))
    engine.run_until_done()
    out = engine.collect_outputs()
    assert engine.num_prefill_tokens == 1 + 9 + 40 + 64 + 9 + 40
    for rid, prompt, params in reqs:
        got = out[rid]
        assert len(got) == 12
        want, margin = replay_sampling(weights, config, prompt, got, params)
        if dtype == "float32":
            assert got == want or margin < 1e-5, (rid, got, want, margin)
        else:
            # teacher-forced on the engine's own tokens, so every position is compared on its own:
            # a token may differ only where the plain margin (top-2 gap, or the distance of the
            # uniform number from an edge of the cumulative distribution) is within bfloat16's reach
            assert_tokens_within_margin(weights, config, prompt, got, params)
    assert engine.runner.cache.num_free_pages() == 48


def test_head_size_64_chunked_prompts_beside_decoding(folders):
    """The configuration whose portions of prompts run on the tcgen05 attention kernel (one
    layer with a window of 50): prompts longer than a key tile, cut into portions of 48 beside
    decoded tokens, greedy, against the plain implementation."""
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    from dispec_b200.ops import attention as A
    folder, config, weights = folders["e"]
    assert A.tcgen05_supported(config["head_dim"], 3, 8, torch.bfloat16)
    engine = ContinuousBatchingEngine(load(folder, "bfloat16"), KVConfig(block_size=8), num_blocks=160,
                                      max_batch_tokens=64, chunk_size=48)
    reqs = []
    for i, n in enumerate([150, 7, 260, 97]):
        prompt = ru.random_ids(n, config["vocab_size"], 600 + i)
        reqs.append((engine.add_request(prompt, 10, SamplingParams()), prompt))
    engine.run_until_done()
    out = engine.collect_outputs()
    for rid, prompt in reqs:
        got = out[rid]
        want, margin = replay_sampling(weights, config, prompt, got, SamplingParams())
        scale = 0.03 * plain.forward_logits(weights, config, prompt).abs().max().item() + 0.02
        assert got == want or margin < 2 * scale, (rid, got, want, margin)
    assert engine.runner.cache.num_free_pages() == 160


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_steps_give_the_same_tokens_as_waiting_for_every_step(folders, dtype):
    """Step n + 1 launched before the tokens of step n are read (tokens fed on the device, end of
    sequence seen one step late) against the engine that waits for every step: the same outputs,
    with ends of sequence in mid-stream, temperature sampling, portions of prompts and arrivals
    while others decode."""
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["b"]
    model = load(folder, dtype)
    prompts = [ru.random_ids(n, config["vocab_size"], 700 + i) for i, n in enumerate([1, 9, 40, 64, 9, 23])]

    def run(overlap, eos):
        engine = ContinuousBatchingEngine(model, KVConfig(block_size=8), num_blocks=64, max_batch_tokens=32,
                                          chunk_size=16, overlap=overlap)
        ids = []
        for i, p in enumerate(prompts[:4]):
            params = SamplingParams(temperature=0.7 if i % 2 else 0.0, top_k=20 if i == 1 else 0, seed=90 + i)
            ids.append(engine.add_request(p, 14, params, eos_id=eos.get(i)))
        for _ in range(5):
            engine.step()
        for i, p in enumerate(prompts[4:], start=4):  # arrive while the others decode
            ids.append(engine.add_request(p, 14, SamplingParams(seed=90 + i), eos_id=eos.get(i)))
        engine.run_until_done()
        out = engine.collect_outputs()
        assert engine.runner.cache.num_free_pages() == 64
        assert not engine.has_work()
        return [out[i] for i in ids], engine.num_steps

    free_run, _ = run(False, {})
    eos, cut = {}, {}
    for i, toks in enumerate(free_run):  # a token in mid-stream that did not occur before it
        for k in range(2, 11):
            if toks[k] not in toks[:k]:
                eos[i], cut[i] = toks[k], k + 1
                break
    assert len(eos) >= 2, "too few requests can stop in mid-stream with these weights"
    waited, steps_waited = run(False, eos)
    overlapped, steps_overlapped = run(True, eos)
    assert waited == overlapped
    for i, tok in eos.items():
        assert waited[i] == free_run[i][:cut[i]] and waited[i][-1] == tok
    assert steps_overlapped >= steps_waited


@pytest.mark.parametrize("seed", [0, 1])
def test_overlapped_steps_under_page_pressure_random_workload(folders, seed):
    """Thirty requests of random lengths, ends of sequence and priorities through a pool so small
    that requests are preempted and recomputed, arriving in three waves: overlapped steps against
    waiting for every step, in 32-bit so that equal means equal."""
    import random as pyrandom
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["a"]
    model = load(folder, "float32")
    rnd_ = pyrandom.Random(seed)
    reqs = []
    for i in range(30):
        n = rnd_.randrange(1, 40)
        reqs.append(dict(prompt=ru.random_ids(n, config["vocab_size"], 900 + 31 * seed + i),
                         max_new=rnd_.randrange(1, 24), eos=rnd_.choice([None, None, rnd_.randrange(config["vocab_size"])]),
                         temperature=rnd_.choice([0.0, 0.0, 0.9]), priority=rnd_.choice([0, 0, 1]), wave=i % 3))

    def run(overlap):
        engine = ContinuousBatchingEngine(model, KVConfig(block_size=16), num_blocks=14, max_batch_tokens=48,
                                          chunk_size=16, max_num_seqs=8, overlap=overlap)
        ids = {}
        for wave in range(3):
            for i, r in enumerate(reqs):
                if r["wave"] == wave:
                    ids[i] = engine.add_request(r["prompt"], r["max_new"],
                                                SamplingParams(temperature=r["temperature"], seed=70 + i),
                                                eos_id=r["eos"], priority=r["priority"])
            for _ in range(7):
                engine.step()
        engine.run_until_done()
        out = engine.collect_outputs()
        assert engine.runner.cache.num_free_pages() == 14 and not engine.has_work()
        engine.runner.cache.check()
        return [out[ids[i]] for i in range(len(reqs))], engine.num_preemptions

    waited, pre_waited = run(False)
    overlapped, pre_overlapped = run(True)
    assert waited == overlapped
    assert pre_waited > 0 and pre_overlapped > 0, "the pool was meant to be too small"
    for r, toks in zip(reqs, waited):
        assert 1 <= len(toks) <= r["max_new"]
        if r["eos"] is not None and r["eos"] in toks:
            assert toks.index(r["eos"]) == len(toks) - 1


def test_no_leak_between_identical_requests(folders):
    from dispec_b200 import ContinuousBatchingEngine, SamplingParams
    folder, config, _ = folders["a"]
    engine = ContinuousBatchingEngine(load(folder, "bfloat16"), num_blocks=64, max_batch_tokens=64,
                                      chunk_size=16)
    prompt = ru.random_ids(21, config["vocab_size"], 7)
    ids = [engine.add_request(prompt, 48, SamplingParams()) for _ in range(3)]
    engine.run_until_done()
    out = engine.collect_outputs()
    assert out[ids[0]] == out[ids[1]] == out[ids[2]] and len(out[ids[0]]) == 48


def test_small_pool_preempts_and_recomputes_with_the_same_tokens(folders):
    from dispec_b200 import ContinuousBatchingEngine, SamplingParams
    folder, config, weights = folders["a"]
    model = load(folder, "float32")
    prompts = [ru.random_ids(n, config["vocab_size"], 500 + n) for n in (16, 16, 30)]
    outs = []
    for blocks in (64, 5):  # 5 pages of 16: the three requests cannot all stay
        engine = ContinuousBatchingEngine(model, num_blocks=blocks, max_batch_tokens=64, poison=True)
        ids = [engine.add_request(p, 24, SamplingParams(temperature=0.7, seed=i)) for i, p in enumerate(prompts)]
        engine.run_until_done()
        outs.append([engine.collect_outputs()[i] for i in ids])
        if blocks == 5:
            assert engine.num_preemptions >= 1
        assert engine.runner.cache.num_free_pages() == blocks
        engine.runner.check_device()
    for roomy, tight, p in zip(outs[0], outs[1], prompts):
        if roomy != tight:  # only a draw on a knife's edge may differ
            want, margin = replay_sampling(weights, config, p, tight, SamplingParams(temperature=0.7))
            assert margin < 1e-5


def test_first_tokens_of_a_sequence(folders):
    """Positions 0, 1, 2: one token at a time from an empty cache."""
    from dispec_b200.engine import ModelRunner, SeqEntry
    folder, config, weights = folders["b"]
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 0.05)):
        runner = ModelRunner(load(folder, dtype), page_size=8, num_pages=4, max_num_seqs=2)
        ids = ru.random_ids(3, config["vocab_size"], 9)
        ref = plain.forward_logits(weights, config, ids)
        runner.admit("s")
        for i, t in enumerate(ids):
            row = runner.step([SeqEntry("s", [t], i, [0])])[0].cpu()
            assert (row - ref[i]).abs().max().item() < tol * max(1.0, ref[i].abs().max().item())


def test_step_refuses_bad_input(folders):
    from dispec_b200.cache import OutOfPagesError
    from dispec_b200.engine import ModelRunner, SeqEntry
    folder, config, _ = folders["a"]
    runner = ModelRunner(load(folder, "float32"), page_size=16, num_pages=2, max_num_seqs=2)
    runner.admit("s")
    with pytest.raises(ValueError, match="start at position"):
        runner.step([SeqEntry("s", [1, 2], 5, [])])
    with pytest.raises(ValueError, match="token id"):
        runner.step([SeqEntry("s", [1, 9999], 0, [])])
    with pytest.raises(KeyError):
        runner.step([SeqEntry("nobody", [1], 0, [])])
    with pytest.raises(OutOfPagesError):
        runner.step([SeqEntry("s", list(range(40)), 0, [])])
    assert runner.step([SeqEntry("s", [1, 2, 3], 0, [])]).shape == (0, config["vocab_size"])


def test_captured_decode_steps_match_eager_steps(folders):
    """All-decode steps replayed from a captured graph (padded to 1, 2, 4 rows) give the logits of
    the eager path, while requests come and go."""
    from dispec_b200.engine import ModelRunner, SeqEntry
    folder, config, weights = folders["c"]
    model = load(folder, "bfloat16")
    prompts = {r: ru.random_ids(n, config["vocab_size"], 600 + n) for r, n in (("x", 37), ("y", 12), ("z", 70))}
    results = []
    for graphs in (False, True):
        runner = ModelRunner(model, page_size=16, num_pages=24, max_num_seqs=4, cuda_graph=graphs, poison=True)
        rows = []
        pos = {}
        for r, p in prompts.items():
            runner.admit(r)
            runner.step([SeqEntry(r, p[:-8], 0, [])])
            pos[r] = len(p) - 8
        live = ["x", "y", "z"]
        for i in range(8):
            if i == 5:
                runner.release("y")
                live.remove("y")
            entries = [SeqEntry(r, [prompts[r][pos[r]]], pos[r], [0]) for r in live]
            rows.append(runner.step(entries).float().cpu().clone())
            for r in live:
                pos[r] += 1
        if graphs:
            assert {bucket for bucket, _ in runner._graphs} == {2, 4}
        runner.check_device()
        results.append(torch.cat(rows))
    refs = {r: plain.forward_logits(weights, config, p) for r, p in prompts.items()}
    scale = max(v.abs().max().item() for v in refs.values())
    assert (results[0] - results[1]).abs().max().item() < 0.03 * scale
    # and both are right: the first decoded row of x
    assert (results[1][0] - refs["x"][len(prompts["x"]) - 8]).abs().max().item() < 0.03 * scale + 0.02


def test_captured_decode_steps_follow_the_context_into_the_next_class(tmp_path):
    """One request decoded from 2,041 to 2,056 tokens: the captured step changes, at 2,048, to the
    one laid out for longer contexts, which cuts the row's keys into ranges merged by a second
    kernel.  The logits stay those of the eager path and of the plain implementation."""
    from dispec_b200.engine import ModelRunner, SeqEntry
    from dispec_b200.ops import attention as A
    folder = str(tmp_path)
    config, weights = ru.make_model_folder(folder, "a_long", dtype="bfloat16")
    model = load(folder, "bfloat16")
    n, tail = 2056, 16
    ids = ru.random_ids(n, config["vocab_size"], 77)
    results = []
    for graphs in (False, True):
        runner = ModelRunner(model, page_size=16, num_pages=600, max_num_seqs=2, cuda_graph=graphs,
                             poison=True)
        runner.admit("r")
        runner.step([SeqEntry("r", ids[:n - tail], 0, [])])
        rows = [runner.step([SeqEntry("r", [ids[i]], i, [0])]).float().cpu().clone() for i in range(n - tail, n)]
        if graphs:
            assert set(runner._graphs) == {(1, 2048), (1, 8192)}
        runner.check_device()
        results.append(torch.cat(rows))
    kvh = config["num_key_value_heads"]
    assert A.choose_outer(1, kvh, 8192, A.choose_splits(1, kvh, 8192)) > 1  # the second class does cut
    ref = plain.forward_logits(weights, config, ids)[n - tail:]
    scale = ref.abs().max().item()
    assert (results[0] - results[1]).abs().max().item() < 0.03 * scale
    assert (results[1] - ref).abs().max().item() < 0.03 * scale + 0.02


@pytest.mark.parametrize("sizes", [
    # the layer sizes of Qwen2.5-1.5B, 7B and 14B (groups of 6, 7 and 5 heads per KV head)
    dict(num_hidden_layers=3, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
         intermediate_size=8960, vocab_size=151936, rms_norm_eps=1e-6, tie_word_embeddings=True),
    dict(num_hidden_layers=2, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
         intermediate_size=18944, vocab_size=152064, rms_norm_eps=1e-6, tie_word_embeddings=False),
    dict(num_hidden_layers=2, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
         intermediate_size=13824, vocab_size=152064, rms_norm_eps=1e-5, tie_word_embeddings=False),
], ids=["1.5b", "7b", "14b"])
def test_recorded_layer_sizes_bfloat16_against_the_32_bit_path(sizes):
    """A few layers of the family's real sizes, random weights: a 700-token prompt in two portions
    and six decoded tokens (captured steps in bfloat16), the serving kernels against the true
    32-bit path."""
    from dispec_b200 import load_model_config
    from dispec_b200.engine import ModelRunner, SeqEntry
    from dispec_b200.weights import load_random_model
    cfg = load_model_config(dict(
        architectures=["Qwen2ForCausalLM"], model_type="qwen2", head_dim=128, rope_theta=1000000.0,
        hidden_act="silu", max_position_embeddings=4096, use_sliding_window=False, **sizes))
    ids = ru.random_ids(706, sizes["vocab_size"], 5)
    got = {}
    for dtype in ("float32", "bfloat16"):
        model = load_random_model(cfg, 2, 0.02, dtype, "cuda:0")
        runner = ModelRunner(model, page_size=16, num_pages=64, max_num_seqs=4, cuda_graph=dtype == "bfloat16")
        runner.admit("r")
        runner.step([SeqEntry("r", ids[:512], 0, [])])
        rows = [runner.step([SeqEntry("r", ids[512:700], 512, [187])]).float().cpu().clone()]
        for i in range(700, 706):
            rows.append(runner.step([SeqEntry("r", [ids[i]], i, [0])]).float().cpu().clone())
        runner.check_device()
        got[dtype] = torch.cat(rows)
        del runner, model
        torch.cuda.empty_cache()
    ref, out = got["float32"], got["bfloat16"]
    scale = ref.abs().max().item()
    assert torch.isfinite(out).all() and scale > 0.5
    assert (out - ref).abs().max().item() < 0.03 * scale + 0.02
    # the same next token wherever the 32-bit path is sure of it
    top2 = ref.topk(2, dim=-1).values
    sure = (top2[:, 0] - top2[:, 1]) > 2 * (0.03 * scale + 0.02)
    assert torch.equal(out.argmax(-1)[sure], ref.argmax(-1)[sure])


def test_command_line_generate_and_random(tmp_path):
    """`python -m dispec_b200 random` writes a folder that `generate` serves; greedy output equals
    the plain implementation's."""
    import json
    import os
    import subprocess
    import sys
    from safetensors.torch import load_file
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(ru.CONFIG_B))
    out_dir = tmp_path / "model"
    env = dict(os.environ, PYTHONPATH=ru.ROOT)
    subprocess.run([sys.executable, "-m", "dispec_b200", "random", "--config", str(cfg_path), "--out", str(out_dir),
                    "--seed", "5", "--std", "0.08"], check=True, env=env, cwd=ru.ROOT)
    proc = subprocess.run([sys.executable, "-m", "dispec_b200", "generate", "--model", str(out_dir), "--dtype", "float32",
                           "--prompt-ids", "5,17,3,99", "--prompt-ids", "7 8 9", "--max-new", "6", "--block-size", "8",
                           "--num-blocks", "32", "--max-batch-tokens", "16", "--chunk-size", "4"],
                          check=True, env=env, cwd=ru.ROOT, capture_output=True, text=True)
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert [ln["prompt_tokens"] for ln in lines] == [4, 3]
    weights = {k: v.float() for k, v in load_file(str(out_dir / "model.safetensors")).items()}
    config = json.load(open(out_dir / "config.json"))
    for ln, prompt in zip(lines, ([5, 17, 3, 99], [7, 8, 9])):
        want, gaps = plain.greedy_generate(weights, config, prompt, 6)
        n = next((i for i, g in enumerate(gaps) if g < 1e-4), 6)
        assert ln["output_ids"][:n] == want[:n]
    # the same model without a folder: random weights filled on the device from the configuration and
    # the seed, with the other spellings of the cache options
    proc2 = subprocess.run([sys.executable, "-m", "dispec_b200", "generate", "--random", str(cfg_path), "--weights-seed", "5",
                            "--std", "0.08", "--dtype", "float32", "--prompt-ids", "5,17,3,99", "--prompt-ids", "7 8 9",
                            "--max-new", "6", "--page-size", "8", "--num-pages", "32", "--max-batch-tokens", "16",
                            "--chunk-size", "4"], check=True, env=env, cwd=ru.ROOT, capture_output=True, text=True)
    assert [json.loads(ln) for ln in proc2.stdout.splitlines() if ln.startswith("{")] == lines
    # and the replay program as a sub-command
    step = {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3, 99], "want": [3]}], "end": ["a"]}
    proc3 = subprocess.run([sys.executable, "-m", "dispec_b200", "replay", "--model", str(out_dir), "--dtype", "float32",
                            "--out", str(tmp_path / "logits"), "--max-tokens", "64", "--page-size", "8"],
                           input=json.dumps(step) + "\n", check=True, env=env, cwd=ru.ROOT, capture_output=True, text=True)
    assert proc3.stdout.split() == ["done", "0"]
    import numpy as np
    row = torch.from_numpy(np.fromfile(tmp_path / "logits" / "0.f32", dtype="<f4"))
    assert (row - plain.forward_logits(weights, config, [5, 17, 3, 99])[-1]).abs().max().item() < 1e-4


# -------------------------------------------- anchored on the reference scheduler's own output

@pytest.mark.parametrize("name", ["a", "b"])
def test_engine_streams_match_the_reference_scheduler(name, tmp_path):
    """Greedy token streams that DiSpec's own ContinuousBatchingEngine produced on the CPU in
    float32 (stored by tests/golden/make_golden.py: portions of 16 under a budget of 32 tokens, 24
    pages) against this engine in float32 with the same settings and the same weights, token by
    token up to the first position whose top-2 margin is below 1e-4."""
    import json
    import os
    from test_plain_vs_golden import GOLDEN, streams_agree
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams, load_model
    from dispec_b200.weights import write_safetensors
    g = torch.load(os.path.join(GOLDEN, f"golden_{name}.pt"))
    weights = plain.random_weights(g["config"], g["seed"], g["std"])
    with open(tmp_path / "config.json", "w") as f:
        json.dump(g["config"], f)
    write_safetensors(str(tmp_path / "model.safetensors"), weights)
    st = g["streams"]
    page = 16 if name == "a" else 8
    for overlap in (False, True):
        engine = ContinuousBatchingEngine(load_model(str(tmp_path), "float32", "cuda:0"), KVConfig(block_size=page),
                                          num_blocks=st["num_blocks"], max_batch_tokens=st["max_batch_tokens"],
                                          chunk_size=st["chunk_size"], overlap=overlap)
        ids = [engine.add_request(p, st["new_tokens"], SamplingParams(0.0)) for p in g["prompts"]]
        engine.run_until_done()
        out = engine.collect_outputs()
        compared = 0
        for rid, prompt, want in zip(ids, g["prompts"], st["tokens"]):
            assert len(out[rid]) == len(want)
            compared += streams_agree(weights, g["config"], prompt, out[rid], want)
        assert compared >= 2 * len(ids)
        if not overlap:
            assert engine.num_steps == st["steps"]  # the same schedule as the reference's, step for step
        assert engine.runner.cache.num_free_pages() == st["num_blocks"]


# ------------------------------------- bfloat16, captured graphs, overlap and preemption together

@pytest.mark.parametrize("seed", [0, 1])
def test_bfloat16_graphs_and_overlap_under_page_pressure(folders, seed):
    """The random thirty-request workload through a pool so small that requests are preempted and
    recomputed, in bfloat16 with captured decode steps: overlapped steps against waiting for every
    step, and every token against the plain implementation where its margin allows."""
    import random as pyrandom
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["b"]
    model = load(folder, "bfloat16")
    rnd_ = pyrandom.Random(100 + seed)
    reqs = []
    for i in range(30):
        n = rnd_.randrange(1, 40)
        reqs.append(dict(prompt=ru.random_ids(n, config["vocab_size"], 1900 + 31 * seed + i),
                         max_new=rnd_.randrange(1, 24), eos=rnd_.choice([None, None, rnd_.randrange(config["vocab_size"])]),
                         temperature=rnd_.choice([0.0, 0.0, 0.9]), priority=rnd_.choice([0, 0, 1]), wave=i % 3))

    def run(overlap):
        engine = ContinuousBatchingEngine(model, KVConfig(block_size=8), num_blocks=28, max_batch_tokens=48,
                                          chunk_size=16, max_num_seqs=8, overlap=overlap, cuda_graph=True, poison=True)
        assert engine.runner.cuda_graph
        ids = {}
        for wave in range(3):
            for i, r in enumerate(reqs):
                if r["wave"] == wave:
                    ids[i] = engine.add_request(r["prompt"], r["max_new"],
                                                SamplingParams(temperature=r["temperature"], seed=70 + i),
                                                eos_id=r["eos"], priority=r["priority"])
            for _ in range(7):
                engine.step()
        engine.run_until_done()
        out = engine.collect_outputs()
        assert engine.runner.cache.num_free_pages() == 28 and not engine.has_work()
        engine.runner.cache.check()
        engine.runner.check_device()
        assert engine.runner._graphs, "no step was replayed from a captured graph"
        return [out[ids[i]] for i in range(len(reqs))], engine.num_preemptions

    waited, pre_waited = run(False)
    overlapped, pre_overlapped = run(True)
    assert pre_waited > 0 and pre_overlapped > 0, "the pool was meant to be too small"
    for i, (r, toks, toks2) in enumerate(zip(reqs, waited, overlapped)):
        params = SamplingParams(temperature=r["temperature"], seed=70 + i)
        for stream in (toks, toks2):
            assert 1 <= len(stream) <= r["max_new"]
            if r["eos"] is not None and r["eos"] in stream:
                assert stream.index(r["eos"]) == len(stream) - 1
        assert_tokens_within_margin(weights, config, r["prompt"], toks, params)
        if toks2 != toks:  # the same kernels on the same inputs: only a preemption at another step
            assert_tokens_within_margin(weights, config, r["prompt"], toks2, params)  # may change a near-tie


# ------------------------------------------------------------- more than 64 requests at once

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live", [65, 100, 130])
def test_many_live_requests(folders, live, dtype):
    """65, 100 and 130 requests decoding side by side: more single-token rows than the few-row
    matrix product takes (they go to the many-row product), and the captured steps of 128 and 256
    padded rows.  Greedy, against the plain implementation."""
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["b"]
    engine = ContinuousBatchingEngine(load(folder, dtype), KVConfig(block_size=8), num_blocks=live * 4 + 8,
                                      max_batch_tokens=4096, max_num_seqs=256, cuda_graph=True)
    prompts = [ru.random_ids(1 + (7 * i) % 19, config["vocab_size"], 3000 + i) for i in range(live)]
    ids = [engine.add_request(p, 6, SamplingParams()) for p in prompts]
    engine.step()
    assert len(engine.running) + len(engine.finished) == live  # every request is live after one step
    engine.run_until_done()
    out = engine.collect_outputs()
    if dtype == "bfloat16":
        assert any(bucket >= 128 for bucket, _ in engine.runner._graphs), engine.runner._graphs.keys()
    for rid, prompt in list(zip(ids, prompts))[::3]:
        got = out[rid]
        assert len(got) == 6
        if dtype == "float32":
            want, margin = replay_sampling(weights, config, prompt, got, SamplingParams())
            assert got == want or margin < 1e-4, (rid, got, want, margin)
        else:
            assert_tokens_within_margin(weights, config, prompt, got, SamplingParams())
    assert engine.runner.cache.num_free_pages() == live * 4 + 8
    engine.runner.check_device()
