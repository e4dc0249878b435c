"""Grouped-query attention over the paged cache.

q, k, v = h W^T + b (one fused product, rows ordered q, k, v: puneethgv/DiSpec
dispec/engine/model_runner.py:104-118,131-136); rotation of q and k and the write of k, v
into the pages (:145-148); scores scaled by ``scale`` (default head_dim**-0.5, :72), key b
visible to the query at position p iff b <= p (and b > p - window for a window layer), softmax
and weighted sum in 32-bit (:160-183 and dispec/engine/triton_attn.py:59-95); output
projection without bias (:158,185).
"""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import attention as attn_ops
from dispec_b200.parts.base import CacheNeed, Mixer, TensorSpec
from dispec_b200.registry import register_part


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position_encoding, window: int = 0, scale: float | None = None,
                 out_bias: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.qkv_bias = qkv_bias
        self.out_bias = out_bias
        self.window = window
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        if not self.scale > 0.0:
            raise ValueError(f"the attention scale must be positive, got {self.scale}")
        self.position_encoding = position_encoding
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def tensor_specs(self):
        h, d = self.hidden_size, self.head_dim
        specs = {
            "q_proj.weight": TensorSpec((self.num_heads * d, h)),
            "k_proj.weight": TensorSpec((self.num_kv_heads * d, h)),
            "v_proj.weight": TensorSpec((self.num_kv_heads * d, h)),
            "o_proj.weight": TensorSpec((h, self.num_heads * d)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = TensorSpec((self.num_heads * d,))
            specs["k_proj.bias"] = TensorSpec((self.num_kv_heads * d,))
            specs["v_proj.bias"] = TensorSpec((self.num_kv_heads * d,))
        if self.out_bias:
            specs["o_proj.bias"] = TensorSpec((h,))
        return specs

    def load(self, tensors):
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors.get("o_proj.bias")

    def cache_need(self):
        return CacheNeed.key_value(self.num_kv_heads, self.head_dim, self.window)

    def tokens_per_attention_tile(self):
        group = self.num_heads // self.num_kv_heads
        small = attn_ops.tokens_per_tile(group)
        if small and self.head_dim in (64, 128):
            return (small, attn_ops.prefill_tokens_per_tile(group))  # portions of prompts: 128-row tiles
        return small

    adds_residual = True
    takes_deferred_norm = True

    def forward(self, ctx, x, cache, state, residual=None, then_norm=None):
        """``residual``: added by the last product (32-bit sum, rounded once), so that the sum
        comes back.  ``x`` may be a norm still to be applied (``NormedRows``), and ``then_norm``
        the (weight, eps) of the norm that reads the result: then (result, NormedRows) comes back."""
        H, KVH, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = ops.linear(x, self.w_qkv, self.b_qkv)
        rot = self.position_encoding.rotation()
        inv_freq, rotary_dim = (rot.inv_freq, rot.rotary_dim) if rot is not None else (None, 0)
        scale = self.scale * self.position_encoding.score_scale()
        # single tokens come first in the batch: when their attention kernel rotates q and k itself and
        # stores the new key and value, the rotation kernel runs on the portions of prompts only
        n_dec = ctx.num_decode_seqs
        fused = None
        if attn_ops.decode_rope_fusable(ctx, H, KVH, D, rotary_dim, qkv.dtype):
            fused = (inv_freq, rotary_dim, cache.write)
        first = n_dec if fused else 0
        if qkv.shape[0] > first:
            ops.rope_kv_store(qkv[first:], ctx.positions[first:], ctx.seq_of_token[first:], cache.page_table,
                              cache.key_pool if cache.write else None,
                              cache.value_pool if cache.write else None,
                              inv_freq, H, KVH, D, rotary_dim, write_kv=cache.write)
        out = torch.empty((qkv.shape[0], H * D), dtype=qkv.dtype, device=qkv.device)
        attn_ops.paged_attention(ctx, qkv, qkv.stride(0), cache, out, H, KVH, D, self.window,
                                 scale, fused_rope=fused)
        return ops.linear(out, self.w_o, self.b_o, residual=residual, out=residual, then_norm=then_norm)
