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
from .base import (BLOCKS, EMBEDDING, FAULT_ACTIVATION, FAULT_TOKEN, NORMS, POSITION_ENCODINGS, STATUS_WORDS,
                   ModelContext, lookup)
from .linear import Linear


def tensor_decls(spec: ModelSpec) -> List[TensorDecl]:
    decls = [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), TABLE)]
    if spec.embed_position is not None:
        decls += lookup(POSITION_ENCODINGS, spec.embed_position.kind, "position encoding").tensor_decls(
            spec.embed_position, spec.embed_position_name)
    for layer in spec.layers:
        decls += lookup(BLOCKS, layer.block, "block").tensor_decls(layer)
    decls += lookup(NORMS, spec.final_norm.kind, "norm").tensor_decls(spec.final_norm, spec.final_norm_name)
    if not spec.tie_word_embeddings:
        decls.append(TensorDecl(spec.head_name, (spec.vocab_size, spec.hidden_size), MATRIX))
    return decls


def cache_groups_of(spec: ModelSpec) -> List[CacheGroupSpec]:
    """What a model of this specification needs from the cache manager, from the specification alone.
    Run steps with equal needs share a group; each group gets pages (or state) of its own."""
    from .base import MIXERS
    need_of = lambda step: lookup(MIXERS, spec.layers[step.layer].mixer.kind, "mixer").cache_need_of(
        spec.layers[step.layer].mixer)
    by_need: "OrderedDict[object, list]" = OrderedDict()
    owner_need = {}
    for step in spec.run_order:
        need = need_of(step)
        if need.kind == "none":
            continue
        if step.writes_cache:
            if step.cache in owner_need:
                raise ConfigError(f"cache entry {step.cache} is written by two run steps")
            owner_need[step.cache] = need
            by_need.setdefault(need, []).append(step.cache)
    for step in spec.run_order:
        need = need_of(step)
        if need.kind != "none" and not step.writes_cache and owner_need.get(step.cache) != need:
            raise ConfigError(f"a run step reads cache entry {step.cache}, which no step with the "
                              f"same needs writes")
    groups = []
    for i, (need, entries) in enumerate(by_need.items()):
        groups.append(CacheGroupSpec(name=f"g{i}:{need.kind}", kind=need.kind, entries=tuple(entries),
                                     kv_heads=need.kv_heads, head_dim=need.head_dim, window=need.window,
                                     state_shape=need.state_shape, state_dtype=need.state_dtype))
    return groups


class DecoderModel:
    def __init__(self, spec: ModelSpec, mctx: ModelContext, source):
        self.spec, self.mctx = spec, mctx
        tensors = load_tensors(source, tensor_decls(spec), mctx.dtype, mctx.device)
        self.embed = tensors[spec.embed_name]
        self.embed_position = None
        if spec.embed_position is not None:
            cls = lookup(POSITION_ENCODINGS, spec.embed_position.kind, "position encoding")
            if getattr(cls, "applies", None) != EMBEDDING:
                raise ConfigError(f"position encoding {spec.embed_position.kind!r} does not add to the embedding")
            self.embed_position = cls(spec.embed_position, mctx, tensors, spec.embed_position_name)
        self.blocks = [lookup(BLOCKS, layer.block, "block")(layer, tensors, mctx) for layer in spec.layers]
        self.final_norm = lookup(NORMS, spec.final_norm.kind, "norm")(spec.final_norm, spec.final_norm_name,
                                                                      tensors, mctx)
        # tied: the head IS the embedding table (same storage), src/model/native.rs:171-179
        self.head = Linear(self.embed if spec.tie_word_embeddings else tensors[spec.head_name], "lm_head")
        for step in spec.run_order:
            if not 0 <= step.layer < len(self.blocks):
                raise ConfigError(f"run order names layer {step.layer}, the model has {len(self.blocks)}")
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=mctx.device)   # when a step brings none
        # decode steps may be replayed from CUDA graphs only if no part plans on the host
        self.replayable = all(getattr(b, "replayable", True) for b in self.blocks) and \
            getattr(self.final_norm, "replayable", True) and getattr(self.embed_position, "replayable", True)

    def cache_groups(self) -> List[CacheGroupSpec]:
        return cache_groups_of(self.spec)

    def forward(self, ctx) -> torch.Tensor:
        """Runs the tokens of ``ctx``; returns float32 logits [len(ctx.logit_rows), vocab]."""
        H = self.spec.hidden_size
        residual = ctx.workspace.get("residual", ctx.T, H, torch.float32)
        status = ctx.status if ctx.status is not None else self.status
        ops.embed_gather(ctx.token_ids, self.embed, residual, status[FAULT_TOKEN:FAULT_TOKEN + 1])
        if self.embed_position is not None:
            self.embed_position.add_to_embedding(ctx, residual)
        pending = None
        order = self.spec.run_order
        for i, step in enumerate(order):
            nxt = self.blocks[order[i + 1].layer] if i + 1 < len(order) else None
            pending = self.blocks[step.layer].forward(ctx, residual, pending, step, nxt)
        # NaN and infinity stay in a residual stream that is only ever added to, and every key or value
        # a step writes is read by its own token: one look at the end covers every block
        # (src/model/native.rs:276-278, src/engine/state.rs:56-58)
        ops.check_finite(residual, pending if isinstance(pending, torch.Tensor) else None,
                         status[FAULT_ACTIVATION:FAULT_ACTIVATION + 1])
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
