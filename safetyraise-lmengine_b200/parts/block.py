"""Pre-norm residual block: r = x + mixer(norm(x)); x' = r + ff(norm(r)).
src/model/native.rs:526-562.

The residual stream is a float32 tensor updated in place.  A block does not add
its feed-forward output itself: it returns it as *pending*, and the next norm
(the next block's, or the final one) adds it in the same kernel that norms.
"""
from __future__ import annotations

from typing import List

from ..config.spec import LayerSpec, RunStep
from ..weights.loader import TensorDecl
from .base import FEED_FORWARDS, MIXERS, NORMS, Block, NormedInput, lookup, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec: LayerSpec, tensors: dict, mctx):
        p = spec.weight_prefix
        self.spec = spec
        self.mixer_norm = lookup(NORMS, spec.mixer_norm.kind, "norm")(spec.mixer_norm, p + spec.mixer_norm_name,
                                                                      tensors, mctx)
        self.ff_norm = lookup(NORMS, spec.feed_forward_norm.kind, "norm")(spec.feed_forward_norm,
                                                                          p + spec.feed_forward_norm_name, tensors, mctx)
        self.mixer = lookup(MIXERS, spec.mixer.kind, "mixer")(spec.mixer, p, tensors, mctx)
        self.feed_forward = lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward")(
            spec.feed_forward, p, tensors, mctx)
        self.hidden = spec.mixer_norm.size
        self.replayable = all(getattr(part, "replayable", True)
                              for part in (self.mixer_norm, self.ff_norm, self.mixer, self.feed_forward))

    @classmethod
    def tensor_decls(cls, spec: LayerSpec, prefix: str = "") -> List[TensorDecl]:
        p = spec.weight_prefix
        return (lookup(NORMS, spec.mixer_norm.kind, "norm").tensor_decls(spec.mixer_norm, p + spec.mixer_norm_name)
                + lookup(MIXERS, spec.mixer.kind, "mixer").tensor_decls(spec.mixer, p)
                + lookup(NORMS, spec.feed_forward_norm.kind, "norm").tensor_decls(spec.feed_forward_norm,
                                                                                 p + spec.feed_forward_norm_name)
                + lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward").tensor_decls(
                    spec.feed_forward, p))

    def fuses(self, ctx) -> bool:
        """Whether this block runs its norms inside the products around them for this step: both parts
        offer forward_fused and the step is small enough for the kernels that carry the fusions."""
        return (getattr(self.mixer_norm, "fusable", False) and getattr(self.ff_norm, "fusable", False)
                and hasattr(self.mixer, "forward_fused") and hasattr(self.feed_forward, "forward_fused")
                and self.mixer.can_fuse(ctx) and self.feed_forward.can_fuse(ctx)
                and not ctx.options.get("unfused_norms", False))

    def prepared_input_norm(self, ctx):
        """This block takes its input already multiplied by its first norm's weight when it fuses."""
        return self.mixer_norm if self.fuses(ctx) else None

    def forward(self, ctx, residual, pending, run_step: RunStep, next_block=None):
        """See parts.base.Block.  When this block runs its norms inside the products around them and the
        block behind it takes a prepared input, the down projection's epilogue prepares it."""
        T = residual.shape[0]
        if self.fuses(ctx):
            asks = getattr(next_block, "prepared_input_norm", None)      # None behind the last block
            next_norm = asks(ctx) if asks is not None else None
            if isinstance(pending, NormedInput):
                nx = pending
            else:
                n = ctx.workspace.get("block.normed", T, self.hidden, ctx.dtype)
                self.mixer_norm.apply(residual, pending, n)
                nx = NormedInput(n, None, self.hidden, self.mixer_norm.spec.eps)
            nx = self.mixer.forward_fused(ctx, nx, run_step, residual, self.ff_norm)
            return self.feed_forward.forward_fused(ctx, nx, residual, next_norm)
        assert not isinstance(pending, NormedInput), "a prepared input was handed to a block that did not ask for one"
        n = ctx.workspace.get("block.normed", T, self.hidden, ctx.dtype)
        self.mixer_norm.apply(residual, pending, n)
        mixed = self.mixer.forward(ctx, n, run_step)
        self.ff_norm.apply(residual, mixed, n)
        return self.feed_forward.forward(ctx, n)
