"""Command line of the engine: ``python -m dispec_b200 <command>``.

Option names follow the reference's scripts where it has them: ``--model``, ``--max-new``,
``--concurrency``, ``--repeats``, ``--temperature`` (puneethgv/DiSpec bench/throughput.py:44-48,
bench/dispec_bench.py:68-72), ``--lengths``, ``--label`` (bench/prefill_bench.py:21-26); sampling
and cache options carry the names of its dataclasses (dispec/config.py:31-51: ``top_p``,
``top_k``, ``seed``, ``block_size``) and constructor arguments (dispec/sched/scheduler.py:61-63:
``num_blocks``, ``max_batch_tokens``, ``chunk_size``).  Token ids in, token ids out: the
tokenizer is not part of the engine.

    generate        generate from prompts given as token ids (--model DIR, or --random CONFIG for
                    random weights filled on the device)
    random          write a model folder with random weights from a config.json and a seed
    replay          feed given token ids step by step and write logits (the program of bin/trace_run)
    throughput      continuous-batching throughput at several concurrency levels
    prefill-bench   time to first token for prompts of given lengths
    env-check       what the engine needs, and whether it is there
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time


def _engine_args(ap, random_weights=False):
    if random_weights:
        src = ap.add_mutually_exclusive_group(required=True)
        src.add_argument("--model", help="folder with config.json and model.safetensors")
        src.add_argument("--random", metavar="CONFIG", help="a config.json (or a folder holding one): the model "
                         "gets random weights, filled on the device")
        ap.add_argument("--weights-seed", type=int, default=None, help="seed of --random (default: --seed)")
        ap.add_argument("--std", type=float, default=0.02, help="standard deviation of --random")
    else:
        ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--block-size", "--page-size", dest="block_size", type=int, default=16,
                    help="tokens per cache page")
    ap.add_argument("--num-blocks", "--num-pages", dest="num_blocks", type=int, default=2048,
                    help="pages per cache group")
    ap.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--chunk-size", type=int, default=None, help="largest prompt portion per step")
    ap.add_argument("--no-cuda-graph", action="store_true", help="run decode steps without graph replay")
    ap.add_argument("--device", default="cuda:0")


def _make_engine(args):
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, load_model
    if getattr(args, "random", None):
        from dispec_b200 import load_model_config, load_random_model
        seed = args.seed if args.weights_seed is None else args.weights_seed
        model = load_random_model(load_model_config(args.random), seed, args.std, args.dtype, args.device)
    else:
        model = load_model(args.model, args.dtype, args.device)
    return ContinuousBatchingEngine(model, KVConfig(block_size=args.block_size), num_blocks=args.num_blocks,
                                    max_batch_tokens=args.max_batch_tokens, chunk_size=args.chunk_size,
                                    cuda_graph=not args.no_cuda_graph), model


def _parse_prompts(args, vocab):
    prompts = []
    for text in args.prompt_ids or []:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            for line in f:
                line = line.strip()
                if line:
                    prompts.append(json.loads(line) if line.startswith("[") else [int(t) for t in line.replace(",", " ").split()])
    if args.random_prompts:
        import torch
        g = torch.Generator().manual_seed(args.seed)
        for n in args.random_prompts:
            prompts.append(torch.randint(0, vocab, (n,), generator=g).tolist())
    if not prompts:
        raise SystemExit("generate: give --prompt-ids, --prompt-file or --random-prompts")
    return prompts


def cmd_generate(args) -> int:
    from dispec_b200 import SamplingParams
    engine, model = _make_engine(args)
    prompts = _parse_prompts(args, model.spec.vocab_size)
    ids = []
    for i, p in enumerate(prompts):
        params = SamplingParams(args.temperature, args.top_p, args.top_k, seed=args.seed + i)
        ids.append(engine.add_request(p, args.max_new, params, eos_id=args.eos_id))
    t0 = time.perf_counter()
    engine.run_until_done()
    dt = time.perf_counter() - t0
    out = engine.collect_outputs()
    for rid, p in zip(ids, prompts):
        print(json.dumps({"id": rid, "prompt_tokens": len(p), "output_ids": out[rid]}))
    n = sum(len(out[r]) for r in ids)
    print(f"# {n} tokens in {dt:.3f}s ({n / dt:.1f} tok/s), {engine.num_steps} steps, "
          f"{engine.num_preemptions} preemptions", file=sys.stderr)
    return 0


def cmd_random(args) -> int:
    from dispec_b200 import load_model_config, write_random_model
    cfg = load_model_config(args.config)
    write_random_model(cfg, args.out, seed=args.seed, std=args.std, dtype=args.dtype)
    print(args.out)
    return 0


def cmd_throughput(args) -> int:
    import torch
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams, load_model
    model = load_model(args.model, args.dtype, args.device)
    g = torch.Generator().manual_seed(0)
    for c in args.concurrency:
        runs = []
        for _ in range(args.repeats + 1):  # the first run warms up
            eng = ContinuousBatchingEngine(model, KVConfig(block_size=args.block_size),
                                           num_blocks=args.num_blocks, max_batch_tokens=args.max_batch_tokens,
                                           chunk_size=args.chunk_size, cuda_graph=not args.no_cuda_graph)
            for _ in range(c):
                eng.add_request(torch.randint(0, model.spec.vocab_size, (args.prompt_len,), generator=g).tolist(),
                                args.max_new, SamplingParams(0.0))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.run_until_done()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            runs.append(sum(len(v) for v in eng.collect_outputs().values()) / dt)
            del eng
        runs = runs[1:]
        print(f"  concurrency={c:>3}: {statistics.median(runs):.1f} tok/s  (runs {', '.join(f'{r:.1f}' for r in runs)})")
    return 0


def cmd_prefill_bench(args) -> int:
    import torch
    from dispec_b200 import load_model
    from dispec_b200.engine import ModelRunner, SeqEntry
    model = load_model(args.model, args.dtype, args.device)
    lengths = [int(x) for x in args.lengths.split(",")]
    runner = ModelRunner(model, page_size=args.block_size,
                         num_pages=(max(lengths) + args.block_size - 1) // args.block_size + 8, max_num_seqs=2)
    points = []
    for n in lengths:
        g = torch.Generator().manual_seed(n)
        ids = torch.randint(0, min(model.spec.vocab_size, 100_000), (n,), generator=g).tolist()
        ts = []
        for r in range(args.repeats + 2):
            runner.admit("p")
            torch.cuda.synchronize()
            t = time.perf_counter()
            runner.step([SeqEntry("p", ids, 0, [n - 1])])
            torch.cuda.synchronize()
            ts.append((time.perf_counter() - t) * 1000)
            runner.release("p")
        ms = statistics.median(ts[2:])
        points.append({"n_tokens": n, "dispec_b200_ms": ms})
        print(f"{n:>7} {ms:>8.2f}ms {n / ms * 1000:>10.0f} tok/s", flush=True)
    print("RESULT_JSON " + json.dumps({"kind": "prefill", "label": args.label, "model": args.model,
                                       "gpu": torch.cuda.get_device_name(), "points": points}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dispec_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate from prompts given as token ids")
    _engine_args(g, random_weights=True)
    g.add_argument("--prompt-ids", action="append", help="one prompt as token ids: '5,17,3' (repeatable)")
    g.add_argument("--prompt-file", help="one prompt per line: ids separated by spaces/commas, or a JSON list")
    g.add_argument("--random-prompts", type=int, nargs="+", help="lengths of uniform random prompts")
    g.add_argument("--max-new", type=int, default=256, help="new tokens per request (max_new_tokens)")
    g.add_argument("--temperature", type=float, default=0.0, help="0 means greedy")
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0, help="0 means off")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--eos-id", type=int, default=None, help="stop a request after this token")
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("random", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json (or a folder holding one)")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r.set_defaults(fn=cmd_random)

    t = sub.add_parser("throughput", help="continuous-batching throughput sweep")
    _engine_args(t)
    t.add_argument("--max-new", type=int, default=96)
    t.add_argument("--concurrency", type=int, nargs="+", default=[6, 16, 32])
    t.add_argument("--repeats", type=int, default=3, help="runs per concurrency; median reported")
    t.add_argument("--prompt-len", type=int, default=32, help="length of the synthetic prompts")
    t.set_defaults(fn=cmd_throughput)

    p = sub.add_parser("prefill-bench", help="time to first token for prompts of given lengths")
    _engine_args(p)
    p.add_argument("--lengths", default="512,1024,2048,4096,8192")
    p.add_argument("--repeats", type=int, default=5)
    p.add_argument("--label", default="")
    p.set_defaults(fn=cmd_prefill_bench)

    rp = sub.add_parser("replay", add_help=False,
                        help="trace replay: steps on standard input, logits to files (options as bin/trace_run)")
    rp.set_defaults(fn=None)

    e = sub.add_parser("env-check", help="what the engine needs, and whether it is there")
    e.set_defaults(fn=lambda a: __import__("dispec_b200.env_check", fromlist=["main"]).main())

    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":  # the replay program parses its own options
        from dispec_b200.engine.replay import main as replay_main
        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    from dispec_b200.config.model_config import ConfigError
    from dispec_b200.registry import RegistryError
    try:
        return args.fn(args)
    except (ConfigError, RegistryError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    except ValueError as e:  # WeightError, SafetensorsError and refused requests
        if type(e).__name__ in ("WeightError", "SafetensorsError"):
            print(f"error: {e}", file=sys.stderr)
            return 2
        raise


if __name__ == "__main__":
    sys.exit(main())
