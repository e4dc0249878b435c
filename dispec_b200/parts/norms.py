"""RMSNorm.  y = w * round(x * rsqrt(mean(x^2) + eps)): 32-bit statistics, the normalised
value rounded to the storage type before the gain is applied (the order the reference's
borrowed module was measured to use; applied at puneethgv/DiSpec
dispec/engine/model_runner.py:215,218,220)."""
from __future__ import annotations

from dispec_b200 import ops
from dispec_b200.ops import gemm as gemm_ops
from dispec_b200.parts.base import Norm, TensorSpec
from dispec_b200.registry import register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = hidden_size
        self.eps = eps
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.hidden_size,), init="one_plus_normal")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, x, rows=None):
        return ops.rms_norm(x, self.weight, self.eps, rows=rows)

    def deferred(self, x):
        """This norm of ``x`` as an input that its consumer applies (a product takes it apart
        where it can, see ``ops.gemm.NormedRows``; otherwise the norm kernel runs there)."""
        return gemm_ops.NormedRows(x, self.weight, self.eps)

    def after_product(self):
        """(weight, eps) for a product that writes the rows this norm reads (``linear(then_norm=)``)."""
        return self.weight, self.eps

    def forward_add(self, ctx, residual, delta, rows=None):
        """Norm of residual + delta (32-bit sum).  Without ``rows`` the sum replaces ``residual``."""
        return ops.rms_norm(residual, self.weight, self.eps, delta=delta, rows=rows,
                            write_back=rows is None)
