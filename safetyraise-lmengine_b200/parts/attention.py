"""Attention over the paged cache with grouped query heads.

Per step: fused q/k/v projection, per-head RMSNorm of q and k (if the
specification has one), position encoding, append of k and v to the pages,
causal attention over everything the request has in the cache, output
projection.  src/model/native.rs:565-648.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import PAGED_ALL, PAGED_WINDOW
from ..config.spec import AttentionSpec, RunStep
from ..errors import Unsupported
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import POSITION_ENCODINGS, ROTATION, CacheNeed, Part, lookup, register_mixer
from .linear import Linear


@register_mixer("paged_attention")
class PagedAttention(Part):
    def __init__(self, spec: AttentionSpec, prefix: str, tensors: dict, mctx):
        if spec.bias:
            raise Unsupported("attention with bias is not implemented")
        self.spec = spec
        p, nm = prefix, spec.names
        # q, k and v rows stacked: one projection, one read of the input
        self.qkv = Linear(torch.cat([tensors[p + nm.q], tensors[p + nm.k], tensors[p + nm.v]],
                                    dim=0).contiguous(), p + "qkv")
        self.out = Linear(tensors[p + nm.o], p + nm.o)
        self.q_norm_w = tensors[p + nm.q_norm] if spec.qk_norm else None
        self.k_norm_w = tensors[p + nm.k_norm] if spec.qk_norm else None
        self.eps = spec.qk_norm.eps if spec.qk_norm else 1.0
        self.position = None
        if spec.position is not None:
            self.position = lookup(POSITION_ENCODINGS, spec.position.kind, "position encoding")(
                spec.position, mctx)
            if getattr(self.position, "applies", ROTATION) != ROTATION:
                raise Unsupported(f"position encoding {spec.position.kind!r} acts on "
                                  f"{self.position.applies!r}; this attention applies rotations of q and k only")
        self.options = mctx.options

    @classmethod
    def tensor_decls(cls, spec: AttentionSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, spec.names
        qd, kvd = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        decls = [TensorDecl(p + nm.q, (qd, spec.hidden_size), MATRIX),
                 TensorDecl(p + nm.k, (kvd, spec.hidden_size), MATRIX),
                 TensorDecl(p + nm.v, (kvd, spec.hidden_size), MATRIX),
                 TensorDecl(p + nm.o, (spec.hidden_size, qd), MATRIX)]
        if spec.qk_norm:
            decls += [TensorDecl(p + nm.q_norm, (spec.head_dim,), VECTOR),
                      TensorDecl(p + nm.k_norm, (spec.head_dim,), VECTOR)]
        return decls

    @classmethod
    def cache_need_of(cls, s: AttentionSpec) -> CacheNeed:
        return CacheNeed(PAGED_WINDOW if s.window else PAGED_ALL, s.kv_heads, s.head_dim, s.window)

    def can_fuse(self, ctx) -> bool:
        return self.qkv.can_fuse(ctx, ctx.T) and self.out.can_fuse(ctx, ctx.T)

    def forward_fused(self, ctx, nx, run_step: RunStep, residual: torch.Tensor, next_norm):
        """The same as forward for a lazily normalised input, with the output projection adding into the
        residual stream and preparing the input of the part behind ``next_norm``."""
        qkv = ctx.workspace.get("attn.qkv", ctx.T, self.qkv.out_features, ctx.dtype)
        self.qkv.from_normed(ctx, nx, qkv)
        attended = self._attend(ctx, qkv, run_step)
        return self.out.into_residual(ctx, attended, residual, next_norm, "a", early=False)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        qkv = self.qkv(ctx, x, "attn.qkv")
        return self.out(ctx, self._attend(ctx, qkv, run_step), "attn.proj", early=False)

    def _attend(self, ctx, qkv: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        s = self.spec
        T = qkv.shape[0]
        k_pool, v_pool, group = ctx.cache.kv_of_entry(run_step.cache)
        # how the encoding turns q and k is the encoding's to say (pairing, rotary fraction): the kernels take it
        rot = self.position.rotation(ctx) if self.position is not None else None
        attended = ctx.workspace.get("attn.out", T, s.heads * s.head_dim, ctx.dtype)
        if ops.attention_from_projection(ctx, qkv, k_pool, v_pool, attended, ctx.block_tables[group], self.q_norm_w,
                                         self.k_norm_w, self.eps, rot, run_step.writes_cache, s.heads,
                                         s.kv_heads, s.head_dim, k_pool.shape[2], s.softmax_scale, s.window or 0):
            return attended
        q = ctx.workspace.get("attn.q", T, s.heads * s.head_dim, ctx.dtype)
        ops.qk_norm_rope_append(qkv, q, k_pool, v_pool, self.q_norm_w, self.k_norm_w, self.eps,
                                rot.cos if rot else None, rot.sin if rot else None, ctx.kv_slot[group], s.heads,
                                s.kv_heads, s.head_dim, rot.pairs if rot else 0, write_kv=run_step.writes_cache,
                                interleaved=bool(rot and rot.interleaved))
        ops.paged_attention(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], s.heads, s.kv_heads,
                            s.head_dim, k_pool.shape[2], s.softmax_scale, s.window or 0)
        return attended
