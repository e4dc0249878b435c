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
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    fuses_norm_and_residual = True

    def forward(self, ctx, x, pre_norm=None, residual=None):
        """``pre_norm`` / ``residual``: as for the attention mixer.  With few rows the activation
        is applied on the way into the down projection instead of by a kernel of its own."""
        if pre_norm is not None:
            gain, eps = pre_norm.as_linear_prologue()
            gate_up = gemm_ops.linear_rms_norm(x, gain, eps, self.w_gate_up)
        else:
            gate_up = ops.linear(x, self.w_gate_up)
        if gemm_ops.fused_prologue_supported(gate_up, self.w_down):
            return gemm_ops.linear_swiglu(gate_up, self.w_down, residual=residual, out=residual)
        return ops.linear(ops.swiglu(gate_up), self.w_down, residual=residual, out=residual)
