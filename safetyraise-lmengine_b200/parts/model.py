"""The decoder: embedding, blocks in their run order, final norm, output head.

Built from a ``ModelSpec`` alone; which architecture the spec came from does
not matter here.  src/model/native.rs:156-312.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List

import torch

from ..cache.manager import FIXED_STATE, CacheGroupSpec
from ..config.spec import ModelSpec
from ..errors import ConfigError
from ..kernels import ops
from ..weights.loader import MATRIX, TABLE, TensorDecl, load_tensors
from .base import BLOCKS, NORMS, ModelContext, lookup
from .linear import Linear


def tensor_decls(spec: ModelSpec) -> List[TensorDecl]:
    decls = [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), TABLE)]
    for layer in spec.layers:
        decls += lookup(BLOCKS, layer.block, "block").tensor_decls(layer)
    decls += lookup(NORMS, spec.final_norm.kind, "norm").tensor_decls(spec.final_norm, spec.final_norm_name)
    if not spec.tie_word_embeddings:
        decls.append(TensorDecl(spec.head_name, (spec.vocab_size, spec.hidden_size), MATRIX))
    return decls


class DecoderModel:
    def __init__(self, spec: ModelSpec, mctx: ModelContext, source):
        self.spec, self.mctx = spec, mctx
        tensors = load_tensors(source, tensor_decls(spec), mctx.dtype, mctx.device)
        self.embed = tensors[spec.embed_name]
        self.blocks = [lookup(BLOCKS, layer.block, "block")(layer, tensors, mctx) for layer in spec.layers]
        self.final_norm = lookup(NORMS, spec.final_norm.kind, "norm")(spec.final_norm, spec.final_norm_name,
                                                                      tensors, mctx)
        # tied: the head IS the embedding table (same storage), src/model/native.rs:171-179
        self.head = Linear(self.embed if spec.tie_word_embeddings else tensors[spec.head_name], "lm_head")
        for step in spec.run_order:
            if not 0 <= step.layer < len(self.blocks):
                raise ConfigError(f"run order names layer {step.layer}, the model has {len(self.blocks)}")
        self.bad_flag = torch.zeros(1, dtype=torch.int32, device=mctx.device)
        # decode steps may be replayed from CUDA graphs only if no part plans on the host
        self.replayable = all(getattr(b, "replayable", True) for b in self.blocks) and \
            getattr(self.final_norm, "replayable", True)

    def cache_groups(self) -> List[CacheGroupSpec]:
        """Run steps with equal needs share a group; each group gets pages (or state) of its own."""
        by_need: "OrderedDict[object, list]" = OrderedDict()
        owner_need = {}
        for step in self.spec.run_order:
            need = self.blocks[step.layer].mixer.cache_need()
            if need.kind == "none":
                continue
            if step.writes_cache:
                if step.cache in owner_need:
                    raise ConfigError(f"cache entry {step.cache} is written by two run steps")
                owner_need[step.cache] = need
                by_need.setdefault(need, []).append(step.cache)
        for step in self.spec.run_order:
            need = self.blocks[step.layer].mixer.cache_need()
            if need.kind != "none" and not step.writes_cache and owner_need.get(step.cache) != need:
                raise ConfigError(f"a run step reads cache entry {step.cache}, which no step with the "
                                  f"same needs writes")
        groups = []
        for i, (need, entries) in enumerate(by_need.items()):
            groups.append(CacheGroupSpec(name=f"g{i}:{need.kind}", kind=need.kind, entries=tuple(entries),
                                         kv_heads=need.kv_heads, head_dim=need.head_dim, window=need.window,
                                         state_shape=need.state_shape, state_dtype=need.state_dtype))
        return groups

    def forward(self, ctx) -> torch.Tensor:
        """Runs the tokens of ``ctx``; returns float32 logits [len(ctx.logit_rows), vocab]."""
        H = self.spec.hidden_size
        residual = ctx.workspace.get("residual", ctx.T, H, torch.float32)
        ops.embed_gather(ctx.token_ids, self.embed, residual, self.bad_flag)
        pending = None
        order = self.spec.run_order
        for i, step in enumerate(order):
            block = self.blocks[step.layer]
            # a block may hand the next one its input already multiplied by that block's norm weight,
            # if both run their norms inside the products (decode steps of a few tokens)
            nxt = self.blocks[order[i + 1].layer] if i + 1 < len(order) else None
            next_norm = None
            if nxt is not None and hasattr(block, "fuses") and hasattr(nxt, "fuses") and block.fuses(ctx) \
                    and nxt.fuses(ctx):
                next_norm = nxt.mixer_norm
            pending = block.forward(ctx, residual, pending, step, next_norm) if hasattr(block, "fuses") \
                else block.forward(ctx, residual, pending, step)
        R = ctx.logit_rows.shape[0]
        logits = ctx.workspace.get("logits", R, self.spec.vocab_size, torch.float32, reserve=64)
        if R == 0:          # nothing wanted: the step only had to fill the cache
            return logits
        hn = ctx.workspace.get("final.normed", R, H, ctx.dtype, reserve=64)
        self.final_norm.apply(residual, pending, hn, rows=ctx.logit_rows)
        self.head.into(ctx, hn, logits)
        return logits

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def walk(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                key = obj.untyped_storage().data_ptr()
                if key not in seen:
                    seen.add(key)
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, (list, tuple)):
                for o in obj:
                    walk(o)
            elif hasattr(obj, "__dict__"):
                for k, o in vars(obj).items():
                    if k not in ("mctx", "spec", "options"):
                        walk(o)
        walk(self)
        return total
