"""Dense SwiGLU feed-forward: down( silu(h Wg^T) * (h Wu^T) ), gate and up as one fused
product (puneethgv/DiSpec dispec/engine/model_runner.py:112,222-226), no biases."""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.parts.base import FeedForward, TensorSpec
from dispec_b200.registry import register_part


@register_part("feed_forward", "swiglu")
class SwiGLUFeedForward(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def load(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def forward(self, ctx, x):
        gate_up = ops.linear(x, self.w_gate_up)
        return ops.linear(ops.swiglu(gate_up), self.w_down)
