"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * weight`` in float32, the weight
multiplying after the normalisation (python/stride_worker/layers.py:24-35)."""

from __future__ import annotations

from ..csrc import ops
from .base import Norm, TensorDecl, register_part


class RMSNorm(Norm):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.eps = float(spec.eps)
        self.width = int(spec.width)
        self.weight = None
        self._name = spec.prefix + "weight"

    def declare(self):
        return {self._name: TensorDecl((self.width,), "vector")}

    def bind(self, weights):
        self.weight = weights[self._name]

    def named_tensors(self):
        return {self._name: self.weight}

    def fold_inputs(self):
        return self.weight, self.eps

    def apply(self, residual, pending, out, rows=None):
        ops.add_rmsnorm(residual, pending, self.weight, out, self.eps, rows=rows)      # sum, write-back and norm in one kernel


register_part("norm", "rmsnorm", RMSNorm)
