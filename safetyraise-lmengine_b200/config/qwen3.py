"""Qwen3 dense decoder: config.json keys -> ModelSpec.

Keys, defaults and rejections follow ModelSpec::from_hf and validate of the
reference (src/model/spec.rs:136-488) for the family ``qwen3``.
"""
from __future__ import annotations

import math

from ..errors import ConfigError, Unsupported
from .spec import (AttentionSpec, FeedForwardSpec, LayerSpec, ModelSpec, NormSpec,
                   PositionSpec, RunStep)

ARCHITECTURE = "Qwen3ForCausalLM"
MODEL_TYPE = "qwen3"
MAX_LAYERS = 4096                     # src/model/spec.rs:203-206


def _positive_int(cfg: dict, key: str, default=None) -> int:
    if key not in cfg or cfg[key] is None:
        if default is None:
            raise ConfigError(f"config.json: missing required key {key!r}")
        return default
    v = cfg[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {key!r} must be a positive integer, got {v!r}")
    return v


def _positive_float(cfg: dict, key: str, default: float) -> float:
    v = cfg.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ConfigError(f"config.json: {key!r} must be a finite positive number, got {v!r}")
    return float(v)


def _boolean(cfg: dict, key: str, default: bool) -> bool:
    v = cfg.get(key)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: {key!r} must be true or false, got {v!r}")
    return v


def _eos_ids(text: dict, root: dict, vocab: int):
    v = text.get("eos_token_id", root.get("eos_token_id"))     # src/model/spec.rs:301-324
    if v is None:
        return ()
    ids = v if isinstance(v, list) else [v]
    out = []
    for t in ids:
        if isinstance(t, bool) or not isinstance(t, int) or t < 0 or t >= vocab:
            raise ConfigError(f"config.json: eos_token_id {t!r} is not a token of the vocabulary")
        out.append(t)
    return tuple(out)


def adapt_source(source):
    """A checkpoint that holds its text model as ``model.language_model.*`` is read under the plain
    ``model.*`` names; the output head keeps its name (src/model/native.rs:156-165)."""
    if "model.language_model.embed_tokens.weight" in set(source.names()):
        from ..weights.loader import PrefixedSource
        return PrefixedSource(source, "model.", "model.language_model.")
    return source


def read_spec(root: dict) -> ModelSpec:
    text = root.get("text_config", root)                       # src/model/spec.rs:137
    if text.get("model_type") != MODEL_TYPE:
        raise ConfigError(f"config.json: model_type {text.get('model_type')!r} does not match "
                          f"architecture {ARCHITECTURE}")
    act = text.get("hidden_act")
    if act is not None and act != "silu":                      # src/model/spec.rs:169-175
        raise Unsupported(f"hidden_act {act!r}: only 'silu' is implemented")
    if _boolean(text, "use_sliding_window", False):            # src/model/spec.rs:176-178
        raise Unsupported("use_sliding_window: Qwen3 with a sliding window is not implemented")
    if _boolean(text, "attention_bias", False) or _boolean(text, "attn_output_gate", False):
        raise Unsupported("attention_bias / attn_output_gate must be false for Qwen3")

    hidden = _positive_int(text, "hidden_size")
    heads = _positive_int(text, "num_attention_heads")
    if text.get("head_dim") is not None:
        head_dim = _positive_int(text, "head_dim")
    else:
        if hidden % heads:
            raise ConfigError("config.json: hidden_size is not a multiple of num_attention_heads "
                              "and head_dim is not given")
        head_dim = hidden // heads
    kv_heads = _positive_int(text, "num_key_value_heads", heads)
    if heads % kv_heads:
        raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of "
                          f"num_key_value_heads {kv_heads}")
    n_layers = _positive_int(text, "num_hidden_layers")
    if n_layers > MAX_LAYERS:
        raise ConfigError(f"config.json: num_hidden_layers {n_layers} exceeds {MAX_LAYERS}")
    kinds = text.get("layer_types")
    if kinds is not None:
        if not isinstance(kinds, list) or len(kinds) != n_layers:
            raise ConfigError("config.json: layer_types must list one kind per layer")
        for k in kinds:
            if k != "full_attention":
                raise Unsupported(f"layer_types entry {k!r}: Qwen3 dense has full_attention only")
    intermediate = _positive_int(text, "intermediate_size")
    vocab = _positive_int(text, "vocab_size")
    if vocab > 0xFFFFFFFF:
        raise ConfigError("config.json: vocab_size exceeds 32 bits")
    max_pos = _positive_int(text, "max_position_embeddings")
    eps = _positive_float(text, "rms_norm_eps", 1e-6)

    rp, rs = text.get("rope_parameters"), text.get("rope_scaling")
    if rp is not None and rs is not None and rp != rs:         # src/model/spec.rs:241-248
        raise ConfigError("config.json: rope_parameters and rope_scaling disagree")
    rope = rp if rp is not None else rs
    if rope is not None:
        if not isinstance(rope, dict):
            raise ConfigError("config.json: rope parameters must be an object")
        kind = rope.get("rope_type", rope.get("type", "default"))
        if kind != "default":
            raise Unsupported(f"rope scaling {kind!r}: only unscaled RoPE is implemented")
        if "factor" in rope and rope["factor"] != 1.0:
            raise Unsupported("rope scaling factor other than 1.0 is not implemented")
    rope_src = rope if rope is not None else text
    if "mrope_section" in rope_src:
        raise Unsupported("mrope_section: multi-axis positions are not implemented (text only)")
    fraction = _positive_float(rope_src, "partial_rotary_factor",
                               _positive_float(text, "partial_rotary_factor", 1.0))
    if fraction > 1.0:
        raise ConfigError("config.json: partial_rotary_factor exceeds 1")
    rotary_dim = int(head_dim * fraction)
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ConfigError(f"config.json: rotary dimension {rotary_dim} must be even and positive")
    theta = _positive_float(rope_src, "rope_theta", _positive_float(text, "rope_theta", 1e6))

    tie = _boolean(text, "tie_word_embeddings", _boolean(root, "tie_word_embeddings", False))
    eos = _eos_ids(text, root, vocab)

    for a, b, what in ((vocab, hidden, "embedding"), (intermediate, hidden, "feed-forward"),
                       (heads * head_dim, hidden, "attention projection")):
        if a * b * 4 >= 1 << 63:                               # src/model/spec.rs:479-487
            raise ConfigError(f"config.json: {what} size overflows")

    position = PositionSpec("rotary_half", theta, rotary_dim, head_dim)
    qk_norm = NormSpec("rmsnorm", head_dim, eps)
    layers = []
    for i in range(n_layers):
        layers.append(LayerSpec(
            block="pre_norm",
            mixer=AttentionSpec(kind="paged_attention", hidden_size=hidden, heads=heads,
                                kv_heads=kv_heads, head_dim=head_dim, qk_norm=qk_norm,
                                position=position, softmax_scale=1.0 / math.sqrt(head_dim),
                                window=None, bias=False),
            feed_forward=FeedForwardSpec("gated_dense", hidden, intermediate, "silu"),
            mixer_norm=NormSpec("rmsnorm", hidden, eps),
            feed_forward_norm=NormSpec("rmsnorm", hidden, eps),
            weight_prefix=f"model.layers.{i}.",
        ))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=hidden, vocab_size=vocab,
        max_position_embeddings=max_pos, layers=tuple(layers),
        run_order=tuple(RunStep(i, i, True) for i in range(n_layers)),
        final_norm=NormSpec("rmsnorm", hidden, eps), tie_word_embeddings=tie,
        eos_token_ids=eos,
    )
