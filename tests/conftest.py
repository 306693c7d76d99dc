import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_terminal_summary(terminalreporter):
    """The largest engine-against-plain error of the run, per dtype: the tolerances in helpers.py are set
    from these figures."""
    try:
        from helpers import TOL, WORST
    except ImportError:
        return
    for dtype, (err, where) in sorted(WORST.items()):
        terminalreporter.write_line(f"worst error against the plain implementation, {dtype}: {err:.3e} of the "
                                    f"largest logit ({where}); tolerance {TOL[dtype]:.1e}")


# Two tiny Qwen3 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "eos_token_id": [7, 9],
}
# Two more with awkward sizes: C has a head size that is no multiple of 64 and as many KV heads as
# query heads; D has a width that is no multiple of 8 (no TMA, no 16-byte rows), 3 query heads per KV head.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 333, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 192,
}
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 80, "intermediate_size": 132, "vocab_size": 257, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 192,
}
# E and F: more than 16 query heads per KV head (32 and 20), where a decode step no longer fits the
# 16 rows of the keys-split attention kernels; head sizes 64 and 128.  G: half of every head rotated
# (partial_rotary_factor 0.5), head size 64, so decode steps leave the kernel that rotates whole heads.
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 32, "num_key_value_heads": 1,
    "head_dim": 64, "intermediate_size": 144, "vocab_size": 300, "rope_theta": 100000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 160,
}
TINY_F = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 1, "hidden_size": 72, "num_attention_heads": 40, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 96, "vocab_size": 200, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 160,
}
TINY_G = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 160, "vocab_size": 280, "rope_theta": 10000.0,
    "partial_rotary_factor": 0.5,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 160,
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4),
        "F": (TINY_F, 5), "G": (TINY_G, 6)}


def make_folder(tmp_path_factory_or_dir, config, seed, name="model", store="BF16"):
    from safetyraise_lmengine_b200.weights.random_init import write_model_folder
    base = tmp_path_factory_or_dir
    out = str(base.mktemp(name)) if hasattr(base, "mktemp") else os.path.join(str(base), name)
    return write_model_folder(config, seed, out, store=store)


@pytest.fixture(scope="session")
def folder_a(tmp_path_factory):
    return make_folder(tmp_path_factory, TINY_A, 0, "tiny_a")


@pytest.fixture(scope="session")
def folder_b(tmp_path_factory):
    return make_folder(tmp_path_factory, TINY_B, 1, "tiny_b")


@pytest.fixture(scope="session", params=["A", "B", "C", "D", "E", "F", "G"])
def tiny_folder(request, tmp_path_factory):
    cfg, seed = TINY[request.param]
    return request.param, make_folder(tmp_path_factory, cfg, seed, "tiny_" + request.param.lower())


# Folders whose matrices are stored in other types than bfloat16 (values not representable in it):
# config B (untied head) as F32 and config A (tied) as F16.
@pytest.fixture(scope="session", params=["B-F32", "A-F16"])
def stored_folder(request, tmp_path_factory):
    name, store = request.param.split("-")
    cfg, seed = TINY[name]
    return name, store, make_folder(tmp_path_factory, cfg, seed + 20, "stored_" + request.param.lower(), store=store)
