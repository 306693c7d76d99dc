"""RMSNorm, fused with the residual addition that precedes it.

out = x / sqrt(mean(x^2) + eps) * w with x = residual (+ delta); reduced in
float32.  src/model/math.rs:28-50.
"""
from __future__ import annotations

from typing import List

from ..config.spec import NormSpec
from ..kernels import ops
from ..weights.loader import VECTOR, TensorDecl
from .base import Part, register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    def __init__(self, spec: NormSpec, name: str, tensors: dict, mctx):
        self.spec, self.weight = spec, tensors[name]

    @classmethod
    def tensor_decls(cls, spec: NormSpec, name: str) -> List[TensorDecl]:
        return [TensorDecl(name, (spec.size,), VECTOR)]

    @property
    def fusable(self) -> bool:
        """Whether products may apply this norm in their own prologue and epilogue (parts.base.NormedInput)."""
        return not self.spec.unit_offset

    def apply(self, residual, delta, out, rows=None):
        """residual[float32] += delta (kept when rows is None); out = norm of the sum.
        With ``rows`` only those rows are normed, into out[0..len(rows))."""
        ops.add_rmsnorm(residual, delta, self.weight, self.spec.eps, out, rows, self.spec.unit_offset)
