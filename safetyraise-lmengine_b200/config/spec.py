"""Typed specifications of a model: what the parts are built from.

A ``ModelSpec`` is a list of ``LayerSpec`` (each names its mixer, feed-forward
and norms by ``kind`` plus their sizes and constants) and a *run order*: the
list of steps a forward takes.  A step names the layer whose weights it uses
and the cache entry it writes or reads, so a layer may run twice, and a layer
may read the cache another layer wrote.  Nothing here knows an architecture:
readers such as ``config/qwen3.py`` fill these records from config.json keys.

Counterpart of ModelSpec/AttentionSpec/RopeSpec/LayerKind in the reference
(src/model/spec.rs:9-78), generalised so that every layer carries its own
part specifications.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    kind: str            # registry key in parts.NORMS
    size: int
    eps: float
    unit_offset: bool = False   # weight + 1 (not used by Qwen3: src/model/native.rs:534)


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # registry key in parts.POSITION_ENCODINGS
    theta: float = 0.0   # the fields of a rotary encoding; another kind adds its own in a subclass
    rotary_dim: int = 0
    head_dim: int = 0


@dataclass(frozen=True)
class AttentionNames:
    """Tensor names of an attention mixer, each appended to its layer's ``weight_prefix``."""
    q: str = "self_attn.q_proj.weight"
    k: str = "self_attn.k_proj.weight"
    v: str = "self_attn.v_proj.weight"
    o: str = "self_attn.o_proj.weight"
    q_norm: str = "self_attn.q_norm.weight"
    k_norm: str = "self_attn.k_norm.weight"


@dataclass(frozen=True)
class GatedDenseNames:
    """Tensor names of a gated dense feed-forward, each appended to its layer's ``weight_prefix``."""
    gate: str = "mlp.gate_proj.weight"
    up: str = "mlp.up_proj.weight"
    down: str = "mlp.down_proj.weight"


@dataclass(frozen=True)
class MixerSpec:
    """Common header of every mixer specification."""
    kind: str            # registry key in parts.MIXERS


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    qk_norm: Optional[NormSpec] = None      # per-head norm of q and k before the position encoding
    position: Optional[PositionSpec] = None
    softmax_scale: float = 0.0
    window: Optional[int] = None            # None: every earlier key is visible
    bias: bool = False
    names: AttentionNames = AttentionNames()


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str            # registry key in parts.FEED_FORWARDS
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    names: GatedDenseNames = GatedDenseNames()   # read by the gated dense part; other kinds name their own


@dataclass(frozen=True)
class LayerSpec:
    block: str                               # registry key in parts.BLOCKS
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    weight_prefix: str                       # e.g. "model.layers.3."
    mixer_norm_name: str = "input_layernorm.weight"              # appended to weight_prefix
    feed_forward_norm_name: str = "post_attention_layernorm.weight"


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order."""
    layer: int                 # index into ModelSpec.layers: whose weights run
    cache: int                 # cache entry (per-step key/value or state storage) it uses
    writes_cache: bool = True  # False: reads what another step wrote under ``cache``


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position_embeddings: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunStep, ...]
    final_norm: NormSpec
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...] = ()
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    embed_position: Optional[PositionSpec] = None   # an encoding that adds to the embedded tokens (none in Qwen3)
    embed_position_name: str = "model.embed_positions.weight"
    extra: dict = field(default_factory=dict, compare=False)

    def to_json(self) -> dict:
        return asdict(self)

    @property
    def num_cache_entries(self) -> int:
        return 1 + max(s.cache for s in self.run_order) if self.run_order else 0
