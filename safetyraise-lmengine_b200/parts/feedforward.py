"""Gated dense feed-forward: down(act(gate(x)) * up(x)), SiLU as the activation.
src/model/native.rs:552-557, src/model/math.rs:11-22."""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import FeedForwardSpec
from ..errors import Unsupported
from ..kernels import ops
from ..weights.loader import MATRIX, TensorDecl
from .base import Part, register_feed_forward
from .linear import Linear


@register_feed_forward("gated_dense")
class GatedDense(Part):
    def __init__(self, spec: FeedForwardSpec, prefix: str, tensors: dict, mctx):
        if spec.activation != "silu":
            raise Unsupported(f"activation {spec.activation!r} is not implemented")
        self.spec = spec
        p = prefix + "mlp."
        # gate rows then up rows: one projection whose output the SwiGLU kernel halves
        self.gate_up = Linear(torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]],
                                        dim=0).contiguous(), p + "gate_up")
        self.down = Linear(tensors[p + "down_proj.weight"], p + "down_proj")

    @classmethod
    def tensor_decls(cls, spec: FeedForwardSpec, prefix: str) -> List[TensorDecl]:
        p = prefix + "mlp."
        return [TensorDecl(p + "gate_proj.weight", (spec.intermediate_size, spec.hidden_size), MATRIX),
                TensorDecl(p + "up_proj.weight", (spec.intermediate_size, spec.hidden_size), MATRIX),
                TensorDecl(p + "down_proj.weight", (spec.hidden_size, spec.intermediate_size), MATRIX)]

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        gu = self.gate_up(ctx, x, "ffn.gate_up")
        h = ctx.workspace.get("ffn.h", x.shape[0], self.spec.intermediate_size, ctx.dtype)
        ops.swiglu(gu, h)
        return self.down(ctx, h, "ffn.down")
