"""Norms over the hidden size, fused with the residual sum that precedes them: RMSNorm
(snowllm/ops/norm.py:11-30; snowllm/models/lfm2/layers.py:99-104) and Dynamic Tanh, which computes no
statistics at all: tanh(alpha * x) * weight + bias with one learned number alpha."""
from __future__ import annotations

from ..ops import kernels
from .base import Part
from .registry import register_norm
from .spec import INIT_BIAS, INIT_ONES, KEEP_SMALL, TensorSpec


class RMSNorm(Part):
    libraries = ("elementwise",)
    fusable_rms = True     # x * rsqrt(mean(x^2) + eps) * weight over the whole width: what a part that fuses
                           # the norm before it into its own first kernel may take over (weight, eps)

    def __init__(self, dtype, names, *, size: int, eps: float):
        super().__init__(dtype, names)
        self.size, self.eps = size, eps
        self.weight = None

    def declare(self, has):
        return [TensorSpec("weight", self.names["weight"], (self.size,), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, residual, delta=None, rows=None):
        """``residual += delta`` in float, then the norm of the sum in the compute dtype.  With
        ``rows`` (int32 row numbers) only those rows come out and the residual stays untouched."""
        return kernels.add_rmsnorm(residual, delta, self.weight, self.eps, self.dtype, rows=rows)

    def add_normed(self, ctx, residual, y):
        """``residual += norm(y)`` for a sublayer's float output ``y`` (the norm on the output side);
        returns the new residual in the compute dtype (the residual itself when that is float)."""
        same = residual.dtype == self.dtype
        x = kernels.norm_add(residual, y, self.weight, self.eps, self.dtype, want_x=not same)
        return residual if same else x


class DynamicTanh(Part):
    """tanh(alpha * x) * weight + bias, elementwise, in float: no mean, no variance, no eps.  Tensors:
    ``weight`` [size], ``bias`` [size], ``alpha`` (one number)."""
    libraries = ("sublayer",)
    fusable_rms = False

    def __init__(self, dtype, names, *, size: int):
        super().__init__(dtype, names)
        self.size = size
        self.weight = self.bias = self.alpha = None

    def declare(self, has):
        n = self.names
        return [TensorSpec("weight", n["weight"], (self.size,), INIT_ONES, KEEP_SMALL),
                TensorSpec("bias", n["bias"], (self.size,), INIT_BIAS, KEEP_SMALL),
                TensorSpec("alpha", n["alpha"], (), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.weight, self.bias, self.alpha = tensors["weight"], tensors["bias"], tensors["alpha"]

    def forward(self, ctx, residual, delta=None, rows=None):
        """``residual += delta`` in float (a tensor, an ``ExpertSum`` or the ``DeltaSum`` of a layer whose
        two sublayers ran side by side), then the norm of the sum in the compute dtype.  With ``rows`` only
        those rows come out and the residual stays untouched."""
        return kernels.add_dyt(residual, delta, self.weight, self.bias, self.alpha, self.dtype, rows=rows)


register_norm("rmsnorm", RMSNorm)
register_norm("dyt", DynamicTanh)
