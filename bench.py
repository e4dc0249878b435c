#!/usr/bin/env python3
"""Benchmark of the engine: decoded tokens a second on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests (Qwen2.5-1.5B layer sizes, random weights
N(0, 0.02) from seed 2, 1024-token random prompts, page size 16, context limit 4096).  W warm-up
steps, then exactly K steps between two device synchronisations, timed with CUDA events; each
step feeds back the tokens the previous step chose (argmax), read on the host.  One JSON line
goes to standard output:

  value      decoded tokens a second, step function + argmax driven directly
  e2e        the same through ContinuousBatchingEngine (scheduler, sampler, pinned staging):
             host token ids in, host token ids out, wall clock
  prefill    one 2,048-token prompt in one step: tokens a second and the fraction of the bf16 peak
  roofline   bytes a decode step must read (every weight once + the live requests' cache)
             divided by its time, against the measured copy bandwidth
  points     decode at batch 1, 64 and 128 (with the fraction of the copy bandwidth), one request at
             32,768 tokens of context, and, for the Qwen2.5-7B and 14B layer sizes with every layer
             of each, decode at batch 1 / 8 / 64 and the 2,048-token prefill with their fractions

Peaks come from MEASURED_PEAKS.json beside this file when present ("of measured"), else the
fallback 6.65 TB/s and 1.59 PFLOP/s ("of fallback").  ``--impl reference`` runs the unmodified
reference (installed under baseline/_ref) through its own ContinuousBatchingEngine on the same
shapes.  With --gpus above 1 it prints one line saying so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-1.5B layer sizes (the benchmark's configuration, not the package's)
BENCH_CONFIG = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=1536,
    num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=8960,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, hidden_act="silu",
    tie_word_embeddings=True, max_position_embeddings=4096, use_sliding_window=False)
# the two larger shapes of the same family (bench.py --shape 7b|14b); seeds as listed beside them
OTHER_SHAPES = {
    "7b": (dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                intermediate_size=18944, vocab_size=152064, rms_norm_eps=1e-6, tie_word_embeddings=False), 3),
    "14b": (dict(num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                 intermediate_size=13824, vocab_size=152064, rms_norm_eps=1e-5, tie_word_embeddings=False), 4),
}
SEED, STD = 2, 0.02
BATCH, PROMPT_LEN, NEW_TOKENS, CONTEXT_LEN, PAGE_SIZE = 8, 1024, 256, 4096, 16
PREFILL_TOKENS = 2048
LONG_CONTEXT = 32768  # an extra point: decoding one request at this context length


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons while a region is timed: through NVML (a read takes
    well under a millisecond, so that a timed region of a few tens of milliseconds still gets ten
    samples and more), or through nvidia-smi where the NVML binding is missing.  Only reads."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, period_s: float = 0.002):
        self.samples = []  # [sm_mhz, sm_max_mhz, {reason: bool}]
        self.period_s = period_s
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            self._max = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001 - fall back to nvidia-smi
            self._nvml = None

    def _read_nvml(self):
        n = self._nvml
        mhz = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
        bits = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle) if hasattr(
            n, "nvmlDeviceGetCurrentClocksEventReasons") else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        masks = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        return [mhz, self._max, {k: bool(bits & m) for k, m in masks.items()}]

    def _read_smi(self):
        out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
        if not out:
            return None
        f = [x.strip() for x in out[0].split(",")]
        return [int(f[0]), int(f[1]), {n: v.lower().startswith("active") for n, v in zip(self.NAMES, f[2:])}]

    def _run(self):
        while not self._stop.is_set():
            try:
                sample = self._read_nvml() if self._nvml else self._read_smi()
                if sample:
                    self.samples.append(sample)
            except Exception:  # noqa: BLE001 - sampling must never break the run
                pass
            self._stop.wait(self.period_s if self._nvml else 0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self) -> dict:
        mhz = [s[0] for s in self.samples]
        mx = [s[1] for s in self.samples]
        reasons = sorted({n for s in self.samples for n, on in s[2].items() if on})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(mhz),
                "source": "nvml" if self._nvml else "nvidia-smi"}


def bench_config(shape: str, cfg_dict: dict, layers: int, full_layers: int, context_len: int, seed: int,
                 weight_bytes: int, peaks_source: str) -> dict:
    """The ``config`` of the JSON line: every size by name, flat, the same keys in both arms."""
    return {
        "model": f"Qwen2.5-{shape.upper()} shape", "layers": layers, "layers_full": full_layers,
        "hidden": cfg_dict["hidden_size"], "heads": cfg_dict["num_attention_heads"],
        "kv_heads": cfg_dict["num_key_value_heads"], "head_dim": cfg_dict["head_dim"],
        "intermediate": cfg_dict["intermediate_size"], "vocab": cfg_dict["vocab_size"],
        "tied": cfg_dict["tie_word_embeddings"], "global_batch": BATCH, "seq_len": PROMPT_LEN,
        "context_len": context_len, "new_tokens": NEW_TOKENS, "page_size": PAGE_SIZE,
        "parallelism": "single GPU", "weights": f"random N(0,{STD}) seed {seed}",
        "l2": "no flush: each step reads %.2f GB of weights, above the 126 MB L2" % (weight_bytes / 1e9),
        "peaks": "of " + peaks_source,
    }


def random_prompts(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def model_bytes_and_flops(cfg: dict, layers: int):
    h, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, KVH, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (H + 2 * KVH) * D * h + (H + 2 * KVH) * D + H * D * h + 3 * I * h + 2 * h
    weight_bytes = 2 * (layers * per_layer + V * h + h)  # lm_head (tied or not) read once
    kv_bytes_per_token = 2 * layers * KVH * D * 2
    matmul_params = layers * ((H + 2 * KVH) * D * h + H * D * h + 3 * I * h)

    def prefill_flops(T):
        return 2 * T * matmul_params + layers * 2 * H * D * T * T + 2 * V * h

    return weight_bytes, kv_bytes_per_token, prefill_flops


# ------------------------------------------------------------------------------ our arm

def decode_direct(runner, prompts, steps, warmup, max_batch_tokens=8192, clocks=None):
    """Step function + argmax, no scheduler: returns (ms per step, launches in the timed region,
    mean context length over the timed steps).  ``clocks``: a ClockSampler that runs during the
    timed steps only."""
    import torch
    from dispec_b200 import ops
    from dispec_b200.engine import SeqEntry
    from dispec_b200.ops.library import LaunchCounter
    ids = [f"r{i}" for i in range(len(prompts))]
    for rid in ids:
        runner.admit(rid)
    last = {}
    pending = [(rid, p, 0) for rid, p in zip(ids, prompts)]
    while pending:  # prefill, untimed: whole prompts side by side, longer ones in portions
        batch, used = [], 0
        while pending and used < max_batch_tokens:
            rid, p, done = pending.pop(0)
            n = min(len(p) - done, max_batch_tokens - used)
            if done + n < len(p):
                batch.append(SeqEntry(rid, p[done:done + n], done, []))
                pending.insert(0, (rid, p, done + n))
            else:
                batch.append(SeqEntry(rid, p[done:], done, [n - 1]))
            used += n
        toks = ops.argmax(runner.step(batch)).tolist()
        for e, t in zip([e for e in batch if e.want], toks):
            last[e.req_id] = t
    pos = {rid: len(p) for rid, p in zip(ids, prompts)}
    # Each step takes its tokens from the previous step's result on the device and copies its own
    # result to pinned host memory; the host reads that copy one step later, while the next step
    # runs (the engine's overlapped steps, without the scheduler).
    state = {"tokens": torch.tensor([last[rid] for rid in ids], dtype=torch.int32, device=runner.device),
             "pending": None}
    host = [torch.empty(len(ids), dtype=torch.int32, pin_memory=True) for _ in range(2)]

    def one_step():
        entries = [SeqEntry(rid, [0], pos[rid], [0], feed_row=i) for i, rid in enumerate(ids)]
        toks = ops.argmax(runner.step(entries, feed_tokens=state["tokens"]))
        turn = runner.num_steps & 1
        host[turn].copy_(toks, non_blocking=True)  # device -> host copy of the result
        ev = torch.cuda.Event()
        ev.record()
        previous, state["pending"], state["tokens"] = state["pending"], (host[turn], ev), toks
        if previous is not None:
            previous[1].synchronize()
            for rid, t in zip(ids, previous[0].tolist()):
                last[rid] = t
        for rid in ids:
            pos[rid] += 1

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    ctx0 = statistics.mean(pos.values())
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = LaunchCounter.n
    if clocks is not None:
        clocks.__enter__()
    start.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.__exit__()
    ms = start.elapsed_time(end) / steps
    launches = LaunchCounter.n - n0
    mean_ctx = (ctx0 + statistics.mean(pos.values())) / 2
    for rid in ids:
        runner.release(rid)
    return ms, launches, mean_ctx


def decode_e2e(model, prompts, steps, warmup, num_blocks, max_model_len=None):
    """Through the public entry point: host token ids in, host token ids out."""
    import torch
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    engine = ContinuousBatchingEngine(model, KVConfig(block_size=PAGE_SIZE), num_blocks=num_blocks,
                                      max_batch_tokens=8192, max_num_seqs=max(len(prompts), 8),
                                      max_model_len=max_model_len)
    for p in prompts:
        # (room for the steps in which the other prompts are still being read)
        engine.add_request(p, warmup + steps + 8 + len(prompts), SamplingParams(0.0))
    while engine.waiting or engine.prefilling:
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert len(engine.running) == len(prompts)
    h2d = engine.runner.staging.last_bytes
    return len(prompts) * steps / dt, dt / steps * 1000, h2d, 4 * len(prompts)


def prefill_time(runner, prompt, repeats=5):
    import torch
    from dispec_b200.engine import SeqEntry
    ts = []
    for _ in range(repeats + 2):
        runner.admit("p")
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        runner.step([SeqEntry("p", prompt, 0, [len(prompt) - 1])])
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
        runner.release("p")
    return statistics.median(ts[2:])


def measure_shape(shape: str, args, pk: dict) -> dict:
    """Decode at batch 1, 8 and 64 and a 2,048-token prefill for one of the larger shapes, with
    every layer of the shape: tokens a second and the fraction of the measured roofline."""
    import torch
    from dispec_b200 import load_model_config
    from dispec_b200.engine import ModelRunner
    from dispec_b200.weights import load_random_model
    cfg_dict = dict(BENCH_CONFIG)
    cfg_dict.update(OTHER_SHAPES[shape][0])
    seed = OTHER_SHAPES[shape][1]
    layers = cfg_dict["num_hidden_layers"]
    t0 = time.time()
    model = load_random_model(load_model_config(cfg_dict), seed, STD, "bfloat16", "cuda:0")
    torch.cuda.synchronize()
    print(f"bench: {shape} model ({layers} layers) filled on the device in {time.time() - t0:.1f}s",
          file=sys.stderr, flush=True)
    weight_bytes, kv_per_token, prefill_flops = model_bytes_and_flops(cfg_dict, layers)
    steps, warmup = max(20, min(args.steps, 50)), max(3, args.warmup // 2)
    per_req = (PROMPT_LEN + NEW_TOKENS + steps + warmup + PAGE_SIZE) // PAGE_SIZE + 1
    out = {f"{shape}_layers": layers}
    for b in (1, 8, 64):
        r = ModelRunner(model, page_size=PAGE_SIZE, num_pages=max(b * per_req, 160), max_num_seqs=max(b, 8),
                        cuda_graph=True)
        ms, _, ctx = decode_direct(r, random_prompts(b, PROMPT_LEN, cfg_dict["vocab_size"], 13 + b), steps, warmup)
        out[f"{shape}_decode_b{b}"] = round(b * 1000.0 / ms, 1)
        out[f"{shape}_decode_b{b}_hbm_frac"] = round(
            (weight_bytes + b * ctx * kv_per_token) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        if b == 1:
            pms = prefill_time(r, random_prompts(1, PREFILL_TOKENS, cfg_dict["vocab_size"], 12)[0], repeats=3)
            out[f"{shape}_prefill"] = round(PREFILL_TOKENS / pms * 1000.0, 1)
            out[f"{shape}_prefill_frac"] = round(prefill_flops(PREFILL_TOKENS) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        del r
        torch.cuda.empty_cache()
    del model
    torch.cuda.empty_cache()
    return out


def mma_issue_rate() -> dict:
    """Cycles one thread needs per tcgen05.mma (128 x N x 16), for 1, 2 and 4 issuing threads."""
    import ctypes
    import torch
    from dispec_b200.ops import library as L
    out = torch.zeros(3, dtype=torch.int64, device="cuda:0")
    table = {}
    for n in (16, 64, 128):
        for issuers in (1, 2, 4):
            for _ in range(2):  # the second run is warm
                L.check(L.core().dsp_selftest_mma_issue_rate(n, issuers, 200, ctypes.c_void_p(out.data_ptr()),
                                                             L.stream_handle()))
            issue, done, ok = out.tolist()
            table[f"n{n}_issuers{issuers}"] = {"cycles_per_mma_per_thread": round(issue / 800, 1),
                                               "cycles_per_mma_overall": round(done / 800 / issuers, 1), "ok": bool(ok)}
    return {"only": "mma-rate", "shape_of_one_product": "128 x N x 16, bfloat16, operands in shared memory", "table": table}


def tma_ingest_rate() -> dict:
    """Bytes a clock that one SM takes in from the L2 by TMA, by the size of a request: boxes of
    64 of k x 128 rows x 1, 2 or 3 blocks of k (16, 32, 48 KB), one to four requests per ring slot."""
    import ctypes
    import torch
    from dispec_b200.ops import library as L
    from dispec_b200.ops import tuning
    ctas = tuning.sm_count(torch.device("cuda:0"))
    rows, iters = 20480, 2000
    matrix = torch.zeros((rows, 1536), dtype=torch.bfloat16, device="cuda:0")
    cycles = torch.zeros(ctas, dtype=torch.int64, device="cuda:0")
    ok = torch.ones(1, dtype=torch.int32, device="cuda:0")
    table = {}
    for stages, boxes, k_blocks in ((6, 1, 1), (6, 2, 1), (3, 4, 1), (3, 1, 2), (3, 2, 2), (2, 2, 3)):
        for _ in range(2):  # the second run is warm
            L.check(L.core().dsp_selftest_tma_rate(L.ptr(matrix), rows, stages, boxes, k_blocks, ctas, iters,
                                                   L.ptr(cycles), L.ptr(ok), L.stream_handle()))
        torch.cuda.synchronize()
        per_slot = float(cycles.double().mean()) / iters
        table[f"{boxes}_requests_of_{16 * k_blocks}KB_ring_of_{stages}"] = {
            "cycles_per_slot": round(per_slot), "bytes_per_clock_and_sm": round(boxes * k_blocks * 16384 / per_slot, 1),
            "ok": bool(int(ok.item()))}
    return {"only": "tma-rate", "ctas": ctas, "source": "a 20,480 x 1,536 bfloat16 matrix in the L2, row tiles in turn",
            "table": table}


def attention_prefill_times() -> dict:
    """The attention kernel for portions of prompts alone: one prompt, causal, by head counts,
    length and how its pages lie in the pool (one after the other, as a pool that is not
    fragmented hands them out, or scattered).  CUDA events over 20 launches, tile lists built once."""
    import torch
    from dispec_b200.ops import attention as A
    from dispec_b200.ops import library as L
    dev = torch.device("cuda:0")
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    rows = []
    for H, KVH, D, T, page in ((12, 2, 128, 2048, 16), (28, 4, 128, 2048, 16), (40, 8, 128, 2048, 16),
                               (14, 2, 64, 2048, 16), (12, 2, 128, 8192, 16), (12, 2, 128, 32768, 16),
                               (12, 2, 128, 8192, 64)):
        G, n = H // KVH, (T + page - 1) // page
        gen = torch.Generator(device=dev).manual_seed(0)
        q = torch.randn(T, H * D, device=dev, generator=gen).bfloat16()
        times = {}
        for order in ("consecutive", "scattered"):
            ids = torch.arange(n, device=dev) if order == "consecutive" else torch.randperm(n + 4, device=dev, generator=gen)[:n]
            kp = torch.randn(n + 4, KVH, page, D, device=dev, generator=gen).bfloat16()
            vp = torch.randn(n + 4, KVH, page, D, device=dev, generator=gen).bfloat16()
            table = ids.int().view(1, -1).contiguous()
            starts = lambda per: (i32([0] * len(range(0, T, per))), i32(list(range(0, T, per))), len(range(0, T, per)))
            small, big = starts(A.tokens_per_tile(G)), starts(A.prefill_tokens_per_tile(G))
            out = torch.zeros_like(q)
            q_start, ctx_len = i32([0, T]), i32([T])
            run = lambda: A.paged_attention_tiles(q, H * D, kp, vp, table, q_start, ctx_len, small[0], small[1],
                                                  small[2], 0, out, H, KVH, D, 0, D ** -0.5, 1, big)
            for _ in range(3):
                run()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                run()
            e1.record()
            torch.cuda.synchronize()
            L.raise_on_device_error("attention for portions of prompts")
            times[order] = e0.elapsed_time(e1) / 20 * 1000
        flops = 4 * H * D * T * (T + 1) / 2
        rows.append({"heads": H, "kv_heads": KVH, "head_dim": D, "tokens": T, "page": page,
                     "us_pages_consecutive": round(times["consecutive"], 1), "us_pages_scattered": round(times["scattered"], 1),
                     "tflops_consecutive": round(flops / times["consecutive"] / 1e6), "tflops_scattered": round(flops / times["scattered"] / 1e6)})
    return {"only": "attn-prefill", "rows": rows}


def decode_timeline(args) -> dict:
    """Where the time of a decode step's kernels goes: the weight-streaming products and the
    single-token attention of a captured step (few layers of the recorded shape) record the global
    timer at points of every CTA's life; needs a build with DISPEC_B200_STAMPS=1 (set before the
    package is imported, which main() does for this mode).  Microseconds, mean over CTAs / slowest CTA."""
    import ctypes
    import numpy as np
    import torch
    from dispec_b200 import load_model_config
    from dispec_b200.engine import ModelRunner, SeqEntry
    from dispec_b200.ops import library as L
    from dispec_b200.weights import load_random_model
    batch, layers = args.batch, args.layers or 4
    cfg = dict(BENCH_CONFIG, num_hidden_layers=layers)
    model = load_random_model(load_model_config(cfg), SEED, STD, "bfloat16", "cuda:0")
    runner = ModelRunner(model, page_size=PAGE_SIZE, num_pages=batch * 90, max_num_seqs=max(batch, 8), cuda_graph=True)
    ids = [f"r{i}" for i in range(batch)]
    for rid, p in zip(ids, random_prompts(batch, PROMPT_LEN, cfg["vocab_size"], 11)):
        runner.admit(rid)
        runner.step([SeqEntry(rid, p, 0, [])])
    core, attn = L.core(), L.attention_library(cfg["head_dim"])
    a_ctl = getattr(attn, f"dsp_attn_stamps_control_d{cfg['head_dim']}")
    a_log = getattr(attn, f"dsp_attn_stamps_log_d{cfg['head_dim']}")
    a_read = getattr(attn, f"dsp_attn_stamps_read_d{cfg['head_dim']}")
    core.dsp_gemm_stream_stamps_control.restype = ctypes.c_long
    a_ctl.restype = ctypes.c_long
    core.dsp_gemm_stream_stamps_control(1)
    a_ctl(1)
    pos = PROMPT_LEN
    for _ in range(6):  # the captured step is replayed last: its launches' stamps are the ones read
        runner.step([SeqEntry(rid, [5], pos, [0]) for rid in ids])
        pos += 1
    torch.cuda.synchronize()

    def read(control, log_fn, read_fn, width):
        log = (ctypes.c_long * (4096 * width))()
        n = log_fn(log, 4096)
        used = control(0)
        buf = (ctypes.c_ulonglong * max(used, 1))()
        read_fn(buf, ctypes.c_long(used))
        stamps = np.frombuffer(buf, dtype=np.uint64).astype(np.int64)
        return [tuple(log[i * width + j] for j in range(width)) for i in range(n)], stamps

    g_launches, g = read(core.dsp_gemm_stream_stamps_control, core.dsp_gemm_stream_stamps_log,
                         core.dsp_gemm_stream_stamps_read, 4)
    a_launches, a = read(a_ctl, a_log, a_read, 2)

    def phase(s, first, last):
        m = (s[:, first] > 0) & (s[:, last] > 0)
        v = (s[m, last] - s[m, first]) / 1000.0
        return [round(float(v.mean()), 2), round(float(v.max()), 2)] if m.any() else None

    kinds = {(cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]: "qkv",
             2 * cfg["intermediate_size"]: "gate_up", cfg["vocab_size"]: "head"}
    products, prev_end = {}, None
    for base, ctas, N, K in g_launches[-(4 * layers + 1):][4:]:  # the first layer follows the embedding: left out
        s = g[base:base + ctas * 12].reshape(ctas, 12)
        name = kinds.get(N, "o_proj" if K == cfg["num_attention_heads"] * cfg["head_dim"] else "down")
        row = {"ctas": int(ctas),
               "end_of_previous_product_to_wait": round(float(s[:, 1].min() - prev_end) / 1000.0, 2) if prev_end else None,
               "wait_to_first_stage": phase(s, 1, 2), "first_stage_to_last_product_issued": phase(s, 2, 3),
               "last_w_requested_to_last_product": phase(s, 7, 3), "last_product_issued_to_accumulator": phase(s, 3, 4),
               "accumulator_to_cluster_barrier": phase(s, 4, 11),
               "accumulator_to_partials_arrived": phase(s, 4, 5), "partials_arrived_to_rows_stored": phase(s, 5, 9),
               "accumulator_to_end": phase(s, 4, 6), "wait_to_end": phase(s, 1, 6)}
        prev_end = s[:, 6].max()
        products.setdefault(name, []).append(row)
    attention = []
    for base, ctas in a_launches[-layers:][1:]:
        s = a[base:base + ctas * 12].reshape(ctas, 12)
        # the cluster merges by sending rows to their owners (the shape of this run takes that path)
        attention.append({"ctas": int(ctas), "wait_to_q_ready": phase(s, 2, 3), "q_ready_to_warp0_done": phase(s, 3, 4),
                          "warp0_done_to_cta_done": phase(s, 4, 5), "cta_done_to_rows_merged": phase(s, 5, 8),
                          "rows_merged_to_sent": phase(s, 8, 6), "sent_to_all_arrived": phase(s, 6, 7),
                          "all_arrived_to_end": phase(s, 7, 9), "wait_to_end": phase(s, 2, 9)})
    return {"only": "timeline", "batch": batch, "layers": layers, "unit": "us, [mean over CTAs, slowest CTA]",
            "products": {k: v[-1] for k, v in products.items()}, "attention": attention[-1] if attention else None}


def run_ours(args) -> dict:
    import torch
    from dispec_b200 import load_model_config
    from dispec_b200.engine import ModelRunner
    from dispec_b200.weights import load_random_model

    if args.only == "mma-rate":
        return mma_issue_rate()
    if args.only == "attn-prefill":
        return attention_prefill_times()
    if args.only == "tma-rate":
        return tma_ingest_rate()
    if args.only == "timeline":
        return decode_timeline(args)
    cfg_dict = dict(BENCH_CONFIG)
    seed = SEED
    if args.shape != "1.5b":
        cfg_dict.update(OTHER_SHAPES[args.shape][0])
        seed = OTHER_SHAPES[args.shape][1]
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    layers = cfg_dict["num_hidden_layers"]
    cfg = load_model_config(cfg_dict)
    t0 = time.time()
    model = load_random_model(cfg, seed, STD, "bfloat16", "cuda:0")
    print(f"bench: model ready in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
    pk = peaks()
    weight_bytes, kv_per_token, prefill_flops = model_bytes_and_flops(cfg_dict, layers)
    prompt_len = args.context if args.only == "decode" and args.context else PROMPT_LEN
    pages_per_req = (prompt_len + NEW_TOKENS + args.steps + args.warmup + PAGE_SIZE) // PAGE_SIZE + 1
    vocab = cfg_dict["vocab_size"]

    # more steps than the recorded context length has room for: the engine's limit is raised (and said)
    longest = prompt_len + args.steps + args.warmup + 64
    over = longest if longest > cfg_dict["max_position_embeddings"] else None

    def runner_for(batch, per_req=pages_per_req, max_len=over):
        return ModelRunner(model, page_size=PAGE_SIZE, num_pages=max(batch * per_req, 160),
                           max_num_seqs=max(batch, 8), cuda_graph=True, max_model_len=max_len)

    if args.max_key_ranges:
        from dispec_b200.ops import tuning
        tuning.MAX_OUTER = args.max_key_ranges
    if args.only == "decode":
        r = runner_for(args.batch, max_len=2 * args.context + args.steps + args.warmup if args.context else over)
        ms, launches, ctx = decode_direct(r, random_prompts(args.batch, prompt_len, vocab, 11), args.steps, args.warmup)
        step_bytes = weight_bytes + args.batch * ctx * kv_per_token
        return {"only": "decode", "shape": args.shape, "batch": args.batch, "layers": layers,
                "ms_per_step": round(ms, 4), "tok_s": round(args.batch * 1000.0 / ms, 1),
                "gpu_launches": launches, "mean_ctx": ctx,
                "hbm_frac": round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
    if args.only == "prefill":
        r = runner_for(1)
        pms = prefill_time(r, random_prompts(1, PREFILL_TOKENS, vocab, 12)[0], repeats=max(1, args.steps))
        return {"only": "prefill", "shape": args.shape, "layers": layers, "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                "tok_s": round(PREFILL_TOKENS / pms * 1000.0, 1),
                "frac": round(prefill_flops(PREFILL_TOKENS) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    # headline: batch 8
    runner = runner_for(BATCH)
    prompts = random_prompts(BATCH, PROMPT_LEN, vocab, 11)
    clocks = ClockSampler()
    ms, launches, mean_ctx = decode_direct(runner, prompts, args.steps, args.warmup, clocks=clocks)
    value = BATCH * 1000.0 / ms
    step_bytes = weight_bytes + BATCH * mean_ctx * kv_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9
    # prefill of 2,048 tokens
    pms = prefill_time(runner, random_prompts(1, PREFILL_TOKENS, vocab, 12)[0])
    pflops = prefill_flops(PREFILL_TOKENS)
    del runner
    torch.cuda.empty_cache()
    e2e_value, e2e_ms, h2d, d2h = decode_e2e(model, prompts, args.steps, args.warmup, BATCH * pages_per_req + 64, over)
    points = {}
    for b in (1, 64, 128):  # 128: beyond the rows of the few-row product (its chunks and the many-row product)
        r = runner_for(b)
        steps = max(20, min(args.steps, 100))
        bms, _, bctx = decode_direct(r, random_prompts(b, PROMPT_LEN, vocab, 13 + b), steps, max(3, args.warmup // 2))
        points[f"decode_b{b}"] = round(b * 1000.0 / bms, 1)
        points[f"decode_b{b}_hbm_frac"] = round((weight_bytes + b * bctx * kv_per_token) / (bms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        del r
        torch.cuda.empty_cache()
    # beyond the recorded configuration: one request with a long context (its keys are shared among
    # several clusters and merged by a second kernel)
    steps = max(20, min(args.steps, 100))
    r = runner_for(1, (LONG_CONTEXT + steps + 64) // PAGE_SIZE + 2, 2 * LONG_CONTEXT)
    bms, _, _ = decode_direct(r, random_prompts(1, LONG_CONTEXT, vocab, 31), steps, max(3, args.warmup // 2))
    points[f"decode_b1_ctx{LONG_CONTEXT}"] = round(1000.0 / bms, 1)
    del r
    torch.cuda.empty_cache()
    from dispec_b200.ops import library
    libraries = [os.path.basename(p) for p in library.loaded_libraries()]
    if args.shape == "1.5b" and not args.layers and not args.no_other_shapes:
        # the two larger shapes of the family, every layer of each: decode at batch 1 / 8 / 64, prefill
        del model
        torch.cuda.empty_cache()
        for shape in ("7b", "14b"):
            points.update(measure_shape(shape, args, pk))
    return {
        "metric": "decode_tokens_per_s", "value": round(value, 1), "unit": "tok/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": bench_config(args.shape, cfg_dict, layers, full_layers, max(CONTEXT_LEN, over or 0), seed,
                               weight_bytes, pk["source"]),
        "clocks": clocks.summary(),
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / pms * 1000.0, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pms, 3), "frac": round(pflops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "kernel_libraries": libraries,
    }


# ------------------------------------------------------------------------- reference arm

def run_reference(args) -> dict:
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "dispec")):
        return {"impl": "reference", "unavailable": "baseline/_ref is absent (the reference was not installed)"}
    sys.path.insert(0, ref)
    try:
        import torch
        from transformers import Qwen2Config, Qwen2ForCausalLM
        from dispec.sampling import SamplingParams
        from dispec.sched.scheduler import ContinuousBatchingEngine
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:200]}
    cfg = {k: v for k, v in BENCH_CONFIG.items() if k not in ("architectures", "model_type")}
    torch.manual_seed(SEED)
    with torch.device("cuda"):
        model = Qwen2ForCausalLM(Qwen2Config(**cfg)).to(torch.bfloat16)
    model.eval()
    model.requires_grad_(False)
    pages = BATCH * ((PROMPT_LEN + NEW_TOKENS + args.steps + args.warmup) // PAGE_SIZE + 2) + 64
    weight_bytes, _, _ = model_bytes_and_flops(BENCH_CONFIG, cfg["num_hidden_layers"])
    longest = PROMPT_LEN + args.steps + args.warmup + 64
    over = longest if longest > BENCH_CONFIG["max_position_embeddings"] else None
    eng = ContinuousBatchingEngine(model, num_blocks=pages, max_batch_tokens=8192,
                                   attn_backend="triton", fuse=True)
    for p in random_prompts(BATCH, PROMPT_LEN, cfg["vocab_size"], 11):
        eng.add_request(p, args.warmup + args.steps + 8, SamplingParams(0.0))
    while eng.waiting or eng.prefilling:
        eng.step()
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    with ClockSampler() as clocks:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        s.record()
        for _ in range(args.steps):
            eng.step()
        e.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    ms = s.elapsed_time(e) / args.steps
    return {
        "metric": "decode_tokens_per_s", "value": round(BATCH * 1000.0 / ms, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "reference",
        "config": bench_config("1.5b", BENCH_CONFIG, cfg["num_hidden_layers"], cfg["num_hidden_layers"],
                               max(CONTEXT_LEN, over or 0), SEED, weight_bytes, peaks()["source"]),
        "path": "dispec ContinuousBatchingEngine(attn_backend=triton, fuse=True); weights from the model "
                "library's own initialiser (normal, std 0.02) under torch.manual_seed",
        "clocks": clocks.summary(),
        "e2e": {"value": round(BATCH * args.steps / wall, 1), "unit": "tok/s"},
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (recorded)")
    ap.add_argument("--shape", choices=["1.5b", "7b", "14b"], default="1.5b",
                    help="layer sizes: Qwen2.5-1.5B (the default and the recorded configuration), 7B or 14B")
    ap.add_argument("--only", choices=["decode", "prefill", "timeline", "mma-rate", "tma-rate", "attn-prefill"], default=None,
                    help="profiling aid: run one phase only and print a short line; timeline: where the time of the "
                         "decode step's products and attention goes (a build with timestamps); mma-rate: cycles per "
                         "tcgen05.mma for one to four issuing threads; tma-rate: bytes a clock an SM takes in from "
                         "the L2 by TMA, by the size of a request; attn-prefill: the attention kernel for portions of prompts "
                         "alone, by shape, length and the order of the pages")
    ap.add_argument("--batch", type=int, default=BATCH, help="batch of the --only decode phase")
    ap.add_argument("--max-key-ranges", type=int, default=0,
                    help="profiling aid: cap on the key ranges per decoded row beyond one cluster (1: none)")
    ap.add_argument("--context", type=int, default=0,
                    help="prompt length of the --only decode phase (default: the recorded configuration's)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--no-other-shapes", action="store_true",
                    help="skip the 7B and 14B points of the default run (shorter run while developing)")
    args = ap.parse_args()
    if args.only == "timeline":
        os.environ["DISPEC_B200_STAMPS"] = "1"  # before the package builds or loads its libraries
    globals()["PAGE_SIZE"] = args.page_size
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    try:
        line = run_reference(args) if args.impl == "reference" else run_ours(args)
    except Exception as e:  # noqa: BLE001
        if args.impl == "reference":
            line = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}
        else:
            raise
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
