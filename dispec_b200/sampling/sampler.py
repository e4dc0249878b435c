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

    def __init__(self, device, capacity: int = 256):
        self.device = device
        # temperature, top_k (as int32 bits), top_p and the uniform number of every row: pinned host
        # buffers used in turn (a copy may still be on its way when the next step is prepared) and one
        # device buffer; nothing is allocated per step
        self._capacity = 0
        self._host: list = []
        self._events: list = []
        self._dev = None
        self._turn = 0
        self._grow(capacity)

    def _grow(self, n: int) -> None:
        cap = max(n, 2 * self._capacity)
        self._host = [torch.empty((4, cap), dtype=torch.float32, pin_memory=True) for _ in range(3)]
        self._events = [None, None, None]
        self._dev = torch.empty((4, cap), dtype=torch.float32, device=self.device)
        self._capacity = cap

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
        if n > self._capacity:
            self._grow(n)
        self._turn = (self._turn + 1) % len(self._host)
        if self._events[self._turn] is not None:
            self._events[self._turn].synchronize()
        host = self._host[self._turn]
        rows = host.numpy()
        top_k = rows[1].view("int32")
        for i, (p, rng) in enumerate(zip(params, rngs)):
            rows[0, i] = p.temperature
            top_k[i] = p.top_k
            rows[2, i] = p.top_p
            rows[3, i] = 0.0 if p.greedy else min(rng.random(), _BELOW_ONE)
        dev = self._dev
        dev[:, :n].copy_(host[:, :n], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._events[self._turn] = event
        return ops.sample(logits, dev[0, :n], dev[1, :n].view(torch.int32), dev[2, :n], dev[3, :n])


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
