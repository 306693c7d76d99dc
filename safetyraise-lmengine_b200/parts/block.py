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
from .base import FEED_FORWARDS, MIXERS, NORMS, Part, lookup, register_block


@register_block("pre_norm")
class PreNormBlock(Part):
    MIXER_NORM, FF_NORM = "input_layernorm.weight", "post_attention_layernorm.weight"

    def __init__(self, spec: LayerSpec, tensors: dict, mctx):
        p = spec.weight_prefix
        self.spec = spec
        self.mixer_norm = lookup(NORMS, spec.mixer_norm.kind, "norm")(spec.mixer_norm, p + self.MIXER_NORM,
                                                                      tensors, mctx)
        self.ff_norm = lookup(NORMS, spec.feed_forward_norm.kind, "norm")(spec.feed_forward_norm,
                                                                          p + self.FF_NORM, tensors, mctx)
        self.mixer = lookup(MIXERS, spec.mixer.kind, "mixer")(spec.mixer, p, tensors, mctx)
        self.feed_forward = lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward")(
            spec.feed_forward, p, tensors, mctx)
        self.hidden = spec.mixer_norm.size

    @classmethod
    def tensor_decls(cls, spec: LayerSpec, prefix: str = "") -> List[TensorDecl]:
        p = spec.weight_prefix
        return (lookup(NORMS, spec.mixer_norm.kind, "norm").tensor_decls(spec.mixer_norm, p + cls.MIXER_NORM)
                + lookup(MIXERS, spec.mixer.kind, "mixer").tensor_decls(spec.mixer, p)
                + lookup(NORMS, spec.feed_forward_norm.kind, "norm").tensor_decls(spec.feed_forward_norm,
                                                                                 p + cls.FF_NORM)
                + lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward").tensor_decls(
                    spec.feed_forward, p))

    def forward(self, ctx, residual, pending, run_step: RunStep):
        T = residual.shape[0]
        n = ctx.workspace.get("block.normed", T, self.hidden, ctx.dtype)
        self.mixer_norm.apply(residual, pending, n)
        mixed = self.mixer.forward(ctx, n, run_step)
        self.ff_norm.apply(residual, mixed, n)
        return self.feed_forward.forward(ctx, n)
