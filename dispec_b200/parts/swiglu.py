"""Dense SwiGLU feed-forward: down( silu(h Wg^T) * (h Wu^T) ), gate and up as one fused
product (puneethgv/DiSpec dispec/engine/model_runner.py:112,222-226), no biases."""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import gemm as gemm_ops
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
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        i, h = self.intermediate_size, self.hidden_size
        # gate and up rows alternate in blocks of 16 when the width allows, so that one warp of the
        # decoding kernel holds both halves of an output and applies the activation itself
        self.block = gemm_ops.SWIGLU_BLOCK if i % gemm_ops.SWIGLU_BLOCK == 0 else 0
        if self.block:
            b = self.block
            self.w_gate_up = torch.stack([gate.view(i // b, b, h), up.view(i // b, b, h)],
                                         dim=1).reshape(2 * i, h).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    adds_residual = True
    takes_deferred_norm = True

    def forward(self, ctx, x, residual=None, then_norm=None):
        """``residual``: added by the last product (32-bit sum, rounded once), so that the sum
        comes back.  ``x`` may be a norm still to be applied (``NormedRows``), and ``then_norm``
        the (weight, eps) of the norm that reads the result: then (result, NormedRows) comes back."""
        if self.block and gemm_ops.gate_up_swiglu_supported(x, self.w_gate_up):
            act = gemm_ops.linear_gate_up_swiglu(x, self.w_gate_up)
        else:
            act = ops.swiglu(ops.linear(x, self.w_gate_up), block=self.block)
        return ops.linear(act, self.w_down, residual=residual, out=residual, then_norm=then_norm)
