"""Trace replay: feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch through the engine's own model, step function, cache
manager and kernels (this program has no forward pass, cache or loader of its own and
samples nothing).  For a step that wants logits, ``<out>/<step>.f32`` holds them as
little-endian float32 [wanted places, vocab], in the order of the entries and of ``want``.
After every step a line ``done <step>`` is printed and flushed.  ``end`` lists requests whose
pages are given back after the step.  The cache pools hold ``--max-tokens`` tokens (each live
request's length rounded up to a multiple of 64, or of the page size where that is larger), so
pages are used again.  ``--cuda-graph`` replays steps made of single tokens only from captured
CUDA graphs, as serving does (bfloat16 only; other steps and float32 run eagerly either way).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="tokens the cache pools hold (live requests, each rounded up to pages)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="replay all-single-token steps from captured CUDA graphs (bfloat16)")
    ap.add_argument("--max-requests", type=int, default=8, help="requests live at a time")
    ap.add_argument("--poison-freed-pages", action="store_true",
                    help="fill pages with NaN when they are given back (shows reads of stale data)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 3
    from dispec_b200.engine import ModelRunner, SeqEntry
    from dispec_b200.weights import load_model

    if args.page_size < 1:
        print("trace_run: --page-size must be positive", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    print(f"trace_run: loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    model = load_model(args.model, args.dtype, args.device)
    # --max-tokens counts every live request rounded up to 64 tokens; a page size that does not
    # divide 64 can leave each request's last page partly outside that count: one page of slack each
    num_pages = max(1, (args.max_tokens + args.page_size - 1) // args.page_size)
    if 64 % args.page_size:
        num_pages += args.max_requests
    runner = ModelRunner(model, page_size=args.page_size, num_pages=num_pages,
                         max_num_seqs=args.max_requests, poison=args.poison_freed_pages,
                         cuda_graph=args.cuda_graph)
    print(f"trace_run: {num_pages} pages of {args.page_size} tokens per cache group "
          f"({len(model.cache_groups)} group(s)); ready", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if not runner.cache.has(rid):
                runner.admit(rid)
            entries.append(SeqEntry(rid, list(e["tokens"]), runner.cache.num_tokens(rid),
                                    list(e.get("want", []))))
        logits = runner.step(entries)
        if logits.shape[0]:
            # (a captured step returns a view of the graph's output buffer: copied out here, before the next step)
            host = logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            host.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        runner.check_device(f"step {step}")
        for rid in rec.get("end", []):
            runner.release(rid)
        print(f"done {step}", flush=True)
    return 0
