"""Rotary position encoding, "default" type: inv_freq[i] = theta^(-2i/rotary_dim), angle =
position * inv_freq[i] in 32-bit, pairs (i, i + rotary_dim/2) rotated (half-split layout).
puneethgv/DiSpec dispec/engine/model_runner.py:35-44,121-124; the table formula in 32-bit at
dispec/kv/transfer.py:50-58.  The reference rounds the cos/sin tables to the model type and
rotates in that type; here angles, cos, sin and the rotation are 32-bit and the result is
rounded once."""
from __future__ import annotations

import torch

from dispec_b200.parts.base import PositionEncoding, Rotation
from dispec_b200.registry import register_part


@register_part("position_encoding", "rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={head_dim}")
        self.inv_freq = None

    def prepare(self, device):
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(torch.float32).to(device)

    def rotation(self):
        if self.inv_freq is None:
            raise RuntimeError("the rotary encoding was not prepared (load the model first)")
        return Rotation(self.inv_freq, self.rotary_dim)


@register_part("position_encoding", "none")
class NoPositionEncoding(PositionEncoding):
    """Keys and queries go to the scores as they are (``rotation()`` is None)."""
