"""Generality of the part system: a toy mixer with state of its own, and a toy architecture that
mixes it with attention and runs one layer twice, are defined HERE, registered, built and stepped
without touching the package."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu


def define_toy():
    from safetyraise_lmengine_b200 import ARCHITECTURES, register_architecture
    from safetyraise_lmengine_b200.cache.manager import FIXED_STATE
    from safetyraise_lmengine_b200.config import qwen3
    from safetyraise_lmengine_b200.config.spec import LayerSpec, MixerSpec, ModelSpec, RunStep
    from safetyraise_lmengine_b200.parts import CacheNeed, Part, register_mixer
    from safetyraise_lmengine_b200.parts.linear import Linear
    from safetyraise_lmengine_b200.parts.model import DecoderModel
    from safetyraise_lmengine_b200.weights.loader import MATRIX, TensorDecl
    if "ToyEmaForCausalLM" in ARCHITECTURES:
        return

    @dataclass(frozen=True)
    class EmaSpec(MixerSpec):
        hidden_size: int = 0
        decay: float = 0.5

    @register_mixer("toy_ema")
    class EmaMixer(Part):
        """state <- decay * state + x_t, token by token; output = W . state.  One vector per request."""

        def __init__(self, spec, prefix, tensors, mctx):
            self.spec = spec
            self.proj = Linear(tensors[prefix + "ema.weight"])

        @classmethod
        def tensor_decls(cls, spec, prefix):
            return [TensorDecl(prefix + "ema.weight", (spec.hidden_size, spec.hidden_size), MATRIX)]

        def cache_need(self):
            return CacheNeed(FIXED_STATE, state_shape=(self.spec.hidden_size,), state_dtype=torch.float32)

        def forward(self, ctx, x, run_step):
            state = ctx.cache.state_of_entry(run_step.cache)        # [max_requests, hidden]
            seq = torch.empty_like(x, dtype=torch.float32)
            t0 = 0
            for slot, q in zip(ctx.host["slots"], ctx.host["q_lens"]):   # tokens of a request, in order
                s = state[slot]
                for t in range(t0, t0 + q):
                    s = self.spec.decay * s + x[t].float()
                    seq[t] = s
                state[slot] = s
                t0 += q
            return self.proj(ctx, seq.to(x.dtype), "toy.out")

    def read_spec(cfg):
        base = qwen3.read_spec(dict(cfg, architectures=["Qwen3ForCausalLM"], model_type="qwen3"))
        layers = list(base.layers)
        ema = EmaSpec(kind="toy_ema", hidden_size=base.hidden_size, decay=cfg["toy_decay"])
        layers[1] = LayerSpec(block="pre_norm", mixer=ema, feed_forward=layers[1].feed_forward,
                              mixer_norm=layers[1].mixer_norm, feed_forward_norm=layers[1].feed_forward_norm,
                              weight_prefix=layers[1].weight_prefix)
        # layer 0 (attention) runs twice, each time with a cache entry of its own
        order = (RunStep(0, 0), RunStep(1, 1), RunStep(0, 2))
        return ModelSpec(architecture="ToyEmaForCausalLM", hidden_size=base.hidden_size,
                         vocab_size=base.vocab_size, max_position_embeddings=base.max_position_embeddings,
                         layers=tuple(layers), run_order=order, final_norm=base.final_norm,
                         tie_word_embeddings=base.tie_word_embeddings)

    register_architecture("ToyEmaForCausalLM", read_spec, lambda spec, mctx, src: DecoderModel(spec, mctx, src))


TOY_CONFIG = {
    "architectures": ["ToyEmaForCausalLM"], "model_type": "toy", "toy_decay": 0.75,
    "num_hidden_layers": 2, "hidden_size": 48, "num_attention_heads": 3, "num_key_value_heads": 3,
    "head_dim": 16, "intermediate_size": 80, "vocab_size": 100, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
}


def plain_toy_logits(w, tokens):
    cfg = TOY_CONFIG
    w = {k: v.float().numpy().astype(np.float64) for k, v in w.items()}
    x = P.embedding(w["model.embed_tokens.weight"], tokens)
    pos = np.arange(len(tokens))

    def ema_block(x):
        p = "model.layers.1."
        n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
        s, seq = np.zeros(x.shape[1]), []
        for t in range(len(tokens)):
            s = cfg["toy_decay"] * s + n1[t]
            seq.append(s)
        r = x + P.linear(np.stack(seq), w[p + "ema.weight"])
        n2 = P.rms_norm(r, w[p + "post_attention_layernorm.weight"], 1e-6)
        return r + P.feed_forward_part(n2, w, p + "mlp.")

    x = P.block(x, pos, w, 0, cfg)
    x = ema_block(x)
    x = P.block(x, pos, w, 0, cfg)
    hn = P.rms_norm(x, w["model.norm.weight"], 1e-6)
    return P.linear(hn, w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from helpers import TOL, cut_bulk_tail, cut_portions, cut_whole, replay
    from safetyraise_lmengine_b200 import Engine, spec_from_config
    from safetyraise_lmengine_b200.cache.manager import FIXED_STATE
    from safetyraise_lmengine_b200.parts.model import tensor_decls
    from safetyraise_lmengine_b200.weights.random_init import RandomWeights
    define_toy()
    spec = spec_from_config(TOY_CONFIG)
    src = RandomWeights(tensor_decls(spec), seed=3)
    assert "model.layers.1.ema.weight" in set(src.names())
    assert "model.layers.1.self_attn.q_proj.weight" not in set(src.names())
    eng = Engine.from_source(TOY_CONFIG, src, dtype=dtype, page_size=4, num_pages=64, max_requests=3,
                             max_batch_tokens=128)
    kinds = sorted(g.kind for g in eng.cache.groups)
    assert kinds == [FIXED_STATE, "paged_all"]
    paged = [g for g in eng.cache.groups if g.kind == "paged_all"][0]
    assert paged.entries == (0, 2)                       # the layer that runs twice has two cache entries
    rng = np.random.default_rng(0)
    toks = [int(t) for t in rng.integers(0, 100, size=60)]
    ref = plain_toy_logits({n: src.get(n) for n in src.names()}, toks)
    other = [int(t) for t in rng.integers(0, 100, size=20)]
    for steps in (cut_whole("x", toks), cut_bulk_tail("x", toks, 32), cut_portions("x", toks)):
        # another request is fed first so that the slot's state must be cleared for the new one
        got = replay(eng, [{"entries": [("o", other, [])], "end": ["o"]}] + steps)
        rows = np.stack([got[("x", p)] for p in range(len(toks))])
        assert np.abs(rows - ref).max() <= TOL[dtype] * np.abs(ref).max()
    assert eng.cache.audit() == 0
