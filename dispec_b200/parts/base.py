"""Interfaces of the parts a decoder is assembled from.

A part owns its sizes and constants (constructor arguments), declares the tensors it
needs (``tensor_specs``), receives them once (``load``) and runs on a flat batch of
tokens described by a ``StepContext``.  No part knows which model it is in: what it
needs from outside arrives as an argument (another part object, a cache view, a state
view).

Roles and their required methods:

* ``Norm.forward(ctx, x, rows=None) -> y`` and
  ``Norm.forward_add(ctx, residual, delta) -> y`` (adds ``delta`` into ``residual`` in
  place in 32-bit, then normalises the sum).
* ``PositionEncoding.rotation() -> Rotation(inv_freq, rotary_dim) | None`` and
  ``PositionEncoding.score_scale() -> float``: what the attention mixer asks of it.
* ``Mixer.forward(ctx, x, cache, state) -> y``; ``cache_need()`` says which named tensors
  a call of this mixer keeps per token in the paged cache (or None), ``state_need()`` what
  fixed-size per-request state (or None).
* ``FeedForward.forward(ctx, x) -> y``.
* ``Block.forward(ctx, x, cache, state) -> x``: the arrangement of two norms, a mixer
  and a feed-forward with their residual sums.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from dispec_b200.cache.manager import CacheTensor, key_value_tensors  # noqa: F401  (CacheTensor re-exported)


@dataclass(frozen=True)
class TensorSpec:
    """Shape and storage class of one tensor a part needs.

    ``dtype``: "model" follows the engine (bfloat16, or float32 on the 32-bit path);
    "float32" stays 32-bit in every mode; "int32" is an integer table.
    ``init`` tells the random-weights mode how to draw it: "normal" is N(0, std),
    "one_plus_normal" is 1 + N(0, std) (gains), "zeros" is 0.
    """
    shape: tuple[int, ...]
    dtype: str = "model"
    init: str = "normal"


@dataclass(frozen=True)
class PartSpec:
    """Declarative description of one part: registered kind, constructor parameters,
    and the checkpoint tensor name behind each of the part's local tensor names."""
    role: str
    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    tensors: dict[str, str] = field(default_factory=dict)  # local name -> checkpoint name


@dataclass(frozen=True)
class CacheNeed:
    """What one mixer call keeps per token in the paged cache: a tuple of named tensors
    (``CacheTensor(name, num_heads, width)``), each with its own heads and width.  Ordinary
    attention keeps two of equal shape, "key" and "value" (``CacheNeed.key_value``); a mixer
    that caches one latent tensor, or keys and values of different widths, lists those instead
    and finds them by name in ``LayerCacheView.tensors``.  ``window`` 0: every token stays;
    W > 0: only the last W positions are ever read, older pages can be given back."""
    tensors: tuple
    window: int = 0

    @classmethod
    def key_value(cls, num_kv_heads: int, head_dim: int, window: int = 0) -> "CacheNeed":
        return cls(key_value_tensors(num_kv_heads, head_dim), window)


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state of one mixer call: a tensor of ``shape`` per live
    request, zeroed when a request is admitted."""
    shape: tuple[int, ...]
    dtype: str = "float32"


class Part:
    role = ""
    kind = ""
    # False for a part whose forward decides things on the host from the step's values (such a
    # part cannot be replayed from a captured graph; the runner then runs every step eagerly)
    graph_safe = True

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors")


class Norm(Part):
    def forward(self, ctx, x, rows=None):
        raise NotImplementedError

    def forward_add(self, ctx, residual, delta):
        raise NotImplementedError


@dataclass(frozen=True)
class Rotation:
    """Rotation of query and key heads: the pair (i, i + rotary_dim/2) of every head is turned
    by the angle position * inv_freq[i]; dimensions from ``rotary_dim`` on pass unchanged."""
    inv_freq: Any  # float32 [rotary_dim / 2] on the device
    rotary_dim: int


class PositionEncoding(Part):
    """What a mixer asks of its position encoding.  ``rotation()``: how it turns queries and
    keys before the scores (None: not at all).  ``score_scale()``: a factor the encoding puts on
    the attention scores beside the mixer's own scale.  ``prepare(device)`` (optional) builds
    device tables once the weights are loaded.  An encoding of another kind (an offset added to
    the stream, a bias on the scores) adds a method of its own and is consumed by a mixer that
    knows that method; the built-in attention mixer uses the two below."""

    def rotation(self) -> Rotation | None:
        return None

    def score_scale(self) -> float:
        return 1.0


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def tokens_per_attention_tile(self):
        """Query tokens per attention tile this mixer wants listed in the batch: an int, a tuple
        of them (one tile list each), or None."""
        return None

    def forward(self, ctx, x, cache, state):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x):
        raise NotImplementedError


class Block(Part):
    def forward(self, ctx, x, pending, cache, state):
        raise NotImplementedError
