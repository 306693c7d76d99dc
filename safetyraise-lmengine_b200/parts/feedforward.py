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
        p, nm = prefix, spec.names
        gate, up = tensors[p + nm.gate], tensors[p + nm.up]
        I, H = gate.shape
        # One projection for gate and up.  For the tensor-core kernels the rows are interleaved in
        # blocks of 16 (8 gate rows, then the 8 up rows of the same features) so that the product's
        # epilogue holds both halves of a feature and writes silu(gate) * up directly; otherwise gate
        # rows then up rows, and a SwiGLU kernel halves the output.
        self.fused = (I % 8 == 0 and gate.dtype == torch.bfloat16 and mctx.dtype == torch.bfloat16
                      and H % 8 == 0 and not mctx.options.get("unfused_swiglu", False))
        if self.fused:
            w = torch.stack([gate.view(I // 8, 8, H), up.view(I // 8, 8, H)], dim=1).reshape(2 * I, H)
        else:
            w = torch.cat([gate, up], dim=0)
        self.gate_up = Linear(w.contiguous(), p + "gate_up")
        self.down = Linear(tensors[p + nm.down], p + nm.down)

    @classmethod
    def tensor_decls(cls, spec: FeedForwardSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, spec.names
        return [TensorDecl(p + nm.gate, (spec.intermediate_size, spec.hidden_size), MATRIX),
                TensorDecl(p + nm.up, (spec.intermediate_size, spec.hidden_size), MATRIX),
                TensorDecl(p + nm.down, (spec.hidden_size, spec.intermediate_size), MATRIX)]

    def can_fuse(self, ctx) -> bool:
        return self.fused and self.gate_up.can_fuse(ctx, ctx.T) and self.down.can_fuse(ctx, ctx.T)

    def forward_fused(self, ctx, nx, residual: torch.Tensor, next_norm):
        """forward for a lazily normalised input; the down projection adds into the residual stream and
        prepares the input of the part behind ``next_norm`` (None: nothing follows)."""
        h = ctx.workspace.get("ffn.h", ctx.T, self.spec.intermediate_size, ctx.dtype)
        self.gate_up.from_normed(ctx, nx, h, swiglu8=True)
        return self.down.into_residual(ctx, h, residual, next_norm, "f")

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        h = ctx.workspace.get("ffn.h", x.shape[0], self.spec.intermediate_size, ctx.dtype)
        if self.fused and ops.can_fuse_swiglu(x.dtype, self.gate_up.weight):
            ops.gemm(x, self.gate_up.weight, h, swiglu8=True)
        else:
            gu = self.gate_up(ctx, x, "ffn.gate_up")
            ops.swiglu(gu, h)
        return self.down(ctx, h, "ffn.down")
