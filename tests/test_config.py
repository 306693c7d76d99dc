"""Configuration reading and the registry (no GPU)."""
import copy

import pytest
from conftest import TINY_A, TINY_B

from safetyraise_lmengine_b200 import ARCHITECTURES, spec_from_config
from safetyraise_lmengine_b200.errors import ConfigError, Unsupported


def test_registry_has_qwen3():
    assert "Qwen3ForCausalLM" in ARCHITECTURES


def test_reads_every_size_from_config():
    a, b = spec_from_config(TINY_A), spec_from_config(TINY_B)
    assert (a.hidden_size, a.vocab_size, len(a.layers), a.tie_word_embeddings) == (64, 256, 2, True)
    assert (b.hidden_size, b.vocab_size, len(b.layers), b.tie_word_embeddings) == (96, 384, 3, False)
    ma, mb = a.layers[0].mixer, b.layers[0].mixer
    assert (ma.heads, ma.kv_heads, ma.head_dim, ma.position.theta, ma.qk_norm.eps) == (4, 2, 16, 1e4, 1e-6)
    assert (mb.heads, mb.kv_heads, mb.head_dim, mb.position.theta, mb.qk_norm.eps) == (6, 1, 32, 1e6, 1e-5)
    assert mb.heads * mb.head_dim != b.hidden_size
    assert b.eos_token_ids == (7, 9) and a.eos_token_ids == ()
    assert a.layers[1].feed_forward.intermediate_size == 128
    assert [s.layer for s in b.run_order] == [0, 1, 2]
    assert a.max_position_embeddings == 128


def test_defaults():
    cfg = copy.deepcopy(TINY_A)
    for k in ("head_dim", "num_key_value_heads", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        cfg.pop(k)
    s = spec_from_config(cfg)
    m = s.layers[0].mixer
    assert m.head_dim == 16 and m.kv_heads == 4                      # src/model/spec.rs:190-200
    assert m.position.theta == 1e6 and s.final_norm.eps == 1e-6     # src/model/spec.rs:283-293,365
    assert s.tie_word_embeddings is False


def test_rope_theta_in_rope_parameters():
    cfg = dict(TINY_A, rope_parameters={"rope_type": "default", "rope_theta": 5e5})
    assert spec_from_config(cfg).layers[0].mixer.position.theta == 5e5


@pytest.mark.parametrize("patch, err", [
    ({"architectures": ["NoSuchModel"]}, Unsupported),
    ({"architectures": ["Qwen3ForCausalLM", "X"]}, ConfigError),
    ({"model_type": "qwen2"}, ConfigError),
    ({"num_key_value_heads": 3}, ConfigError),
    ({"num_key_value_heads": 0}, ConfigError),
    ({"head_dim": 3}, ConfigError),                      # odd rotary dimension
    ({"eos_token_id": 256}, ConfigError),                # outside the vocabulary
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, Unsupported),
    ({"rope_scaling": {"rope_type": "default", "factor": 2.0}}, Unsupported),
    ({"use_sliding_window": True}, Unsupported),
    ({"attention_bias": True}, Unsupported),
    ({"hidden_act": "gelu"}, Unsupported),
    ({"layer_types": ["full_attention", "linear_attention"]}, Unsupported),
    ({"layer_types": ["full_attention"]}, ConfigError),
    ({"hidden_size": None}, ConfigError),
    ({"max_position_embeddings": None}, ConfigError),
    ({"num_hidden_layers": 5000}, ConfigError),
    ({"rms_norm_eps": 0.0}, ConfigError),
    ({"partial_rotary_factor": 1.5}, ConfigError),
])
def test_rejections(patch, err):
    cfg = copy.deepcopy(TINY_A)
    for k, v in patch.items():
        if v is None:
            cfg.pop(k, None)
        else:
            cfg[k] = v
    with pytest.raises(err):
        spec_from_config(cfg)


def test_hidden_not_divisible_needs_head_dim():
    cfg = dict(TINY_B)
    cfg.pop("head_dim")
    cfg["hidden_size"] = 100
    with pytest.raises(ConfigError):
        spec_from_config(cfg)
