"""Greedy, temperature, top-k and top-p sampling, with the reference's names and meanings
(puneethgv/DiSpec dispec/sampling.py:15-75).

The distribution is the reference's: logits / T, top-k keeping ties with the k-th value,
top-p dropping a token once the mass before it (descending order) exceeds top_p, softmax,
one draw.  The draw itself is an inverse CDF at a uniform number taken from a per-request
``random.Random(seed)``, one number per sampled token, so that a request's tokens do not
depend on what else is in the batch and a CPU implementation can replay them; the
reference draws with torch.multinomial from the global generator (dispec/sampling.py:62-67,
dispec/sched/scheduler.py:217-218) and applies the first request's parameters to the
whole batch, which this engine does not imitate.
"""
from __future__ import annotations

import random
from dataclasses import dataclass

import torch

from dispec_b200 import ops

_BELOW_ONE = 1.0 - 2.0 ** -24


@dataclass
class SamplingParams:
    temperature: float = 0.0  # <= 0: greedy (argmax)
    top_p: float = 1.0
    top_k: int = 0  # 0: off
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


def make_rng(params: SamplingParams, generator=None) -> random.Random:
    if isinstance(generator, random.Random):
        return generator
    if isinstance(generator, int):
        return random.Random(generator)
    return random.Random(params.seed)


class Sampler:
    """Samples one token per logits row, each row with its own parameters and generator."""

    def __init__(self, device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: list, rngs: list) -> list[int]:
        if logits.shape[0] == 0:
            return []
        return self.sample_device(logits, params, rngs).tolist()

    @torch.inference_mode()
    def sample_device(self, logits: torch.Tensor, params: list, rngs: list) -> torch.Tensor:
        """The same draw, left on the device (int32 [n]): the caller reads it when it needs it."""
        n = logits.shape[0]
        assert len(params) == n and len(rngs) == n
        if n == 0:
            return torch.empty((0,), dtype=torch.int32, device=logits.device)
        if all(p.greedy for p in params):
            return ops.argmax(logits)
        host = torch.empty((4, n), dtype=torch.float32, pin_memory=True)
        for i, (p, rng) in enumerate(zip(params, rngs)):
            host[0, i] = p.temperature
            host[1, i] = float(p.top_k)
            host[2, i] = p.top_p
            host[3, i] = 0.0 if p.greedy else min(rng.random(), _BELOW_ONE)
        dev = host.to(self.device, non_blocking=True)
        top_k = dev[1].to(torch.int32)
        return ops.sample(logits, dev[0].contiguous(), top_k, dev[2].contiguous(), dev[3].contiguous())


def sample(logits: torch.Tensor, params: SamplingParams, generator=None) -> torch.Tensor:
    """Logits (n, vocab) -> token ids (n,), every row with the same parameters
    (dispec/sampling.py:70-75).  ``generator``: a ``random.Random`` or an int seed."""
    logits = logits.to(torch.float32)
    if logits.dim() == 1:
        logits = logits[None]
    if params.greedy:
        return ops.argmax(logits).to(torch.long)
    rng = make_rng(params, generator)
    ids = Sampler(logits.device).sample(logits, [params] * logits.shape[0], [rng] * logits.shape[0])
    return torch.tensor(ids, dtype=torch.long, device=logits.device)
