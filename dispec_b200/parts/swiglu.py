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

    fuses_norm_and_residual = True

    def forward(self, ctx, x, pre_norm=None, residual=None):
        """``pre_norm``: x is not normalised yet, the norm is applied on the way into the first
        product.  ``residual``: added by the last product, so that the sum comes back."""
        norm = pre_norm.as_linear_prologue() if pre_norm is not None else None
        if self.block and gemm_ops.gate_up_swiglu_supported(x, self.w_gate_up) and (
                norm is None or x.shape[0] <= gemm_ops.FUSED_MAX_ROWS):
            act = gemm_ops.linear_gate_up_swiglu(x, self.w_gate_up, norm)
        else:
            if norm is not None:
                gate_up = gemm_ops.linear_rms_norm(x, norm[0], norm[1], self.w_gate_up)
            else:
                gate_up = ops.linear(x, self.w_gate_up)
            act = ops.swiglu(gate_up, block=self.block)
        return ops.linear(act, self.w_down, residual=residual, out=residual)
