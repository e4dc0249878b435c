"""Token embedding (row gather, no scaling: puneethgv/DiSpec dispec/engine/model_runner.py:63,199)
and the output head (logits = h W^T, no bias, 32-bit logits; :66,228-231)."""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.parts.base import Part, TensorSpec
from dispec_b200.registry import register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx):
        return ops.embed(self.weight, ctx.token_ids)


@register_part("head", "linear_head")
class LinearHead(Part):
    """A tied head names the embedding's checkpoint tensor; the loader then hands both parts
    the same device tensor."""

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, h):
        return ops.linear(h, self.weight, out_dtype=torch.float32)
