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
        replayable = False          # loops over the step's host lists: never recorded into a CUDA graph

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
    assert not eng.use_graphs and eng.graph_replays == 0      # a part that plans on the host runs eagerly



# ---------------------------------------------------------------------------
# A second toy architecture: the framework's own attention with a position encoding defined here
# (rotary angles of positions divided by a factor), and a feed-forward with routing defined here
# (a float32 router picks one of several small experts per token).  Both are replayable, so the
# decode steps run from CUDA graphs like those of the real architecture.
# ---------------------------------------------------------------------------
def define_routed_toy():
    import dataclasses

    from safetyraise_lmengine_b200 import ARCHITECTURES, register_architecture
    from safetyraise_lmengine_b200.config import qwen3
    from safetyraise_lmengine_b200.config.spec import FeedForwardSpec, LayerSpec, ModelSpec, PositionSpec
    from safetyraise_lmengine_b200.parts import Part, register_feed_forward, register_position_encoding
    from safetyraise_lmengine_b200.parts.linear import Linear
    from safetyraise_lmengine_b200.parts.model import DecoderModel
    from safetyraise_lmengine_b200.weights.loader import MATRIX, TensorDecl
    if "ToyRoutedForCausalLM" in ARCHITECTURES:
        return

    @dataclass(frozen=True)
    class ScaledPositionSpec(PositionSpec):
        factor: float = 1.0

    @register_position_encoding("toy_rotary_scaled")
    class ScaledRotary(Part):
        """cos/sin of (pos / factor) / theta^(2i/rotary_dim): the interface the attention part asks for."""

        def __init__(self, spec, mctx):
            self.spec, self.half = spec, spec.rotary_dim // 2
            self.key = ("toy_rotary_scaled", spec.theta, spec.rotary_dim, spec.factor)

        def tables(self, ctx):
            got = ctx.tables.get(self.key)
            if got is None:
                i = torch.arange(self.half, device=ctx.positions.device, dtype=torch.float64)
                inv = self.spec.theta ** (-2.0 * i / self.spec.rotary_dim)
                ang = (ctx.positions.double() / self.spec.factor)[:, None] * inv[None, :]
                got = ctx.tables[self.key] = (ang.cos().float().contiguous(), ang.sin().float().contiguous())
            return got

    @dataclass(frozen=True)
    class RoutedSpec(FeedForwardSpec):
        experts: int = 1

    @register_feed_forward("toy_top1")
    class Top1Experts(Part):
        """out[t] = down_e(silu(up_e(x[t]))) for e = argmax of the float32 router logits of token t."""

        def __init__(self, spec, prefix, tensors, mctx):
            self.spec, p = spec, prefix + "moe."
            self.router = tensors[p + "router.weight"]
            self.up = [Linear(tensors[p + f"experts.{e}.up.weight"]) for e in range(spec.experts)]
            self.down = [Linear(tensors[p + f"experts.{e}.down.weight"]) for e in range(spec.experts)]

        @classmethod
        def tensor_decls(cls, spec, prefix):
            p = prefix + "moe."
            decls = [TensorDecl(p + "router.weight", (spec.experts, spec.hidden_size), MATRIX)]
            for e in range(spec.experts):
                decls.append(TensorDecl(p + f"experts.{e}.up.weight", (spec.intermediate_size, spec.hidden_size), MATRIX))
                decls.append(TensorDecl(p + f"experts.{e}.down.weight", (spec.hidden_size, spec.intermediate_size), MATRIX))
            return decls

        def forward(self, ctx, x):
            choice = (x.float() @ self.router.float().t()).argmax(-1)          # router logits in float32
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.spec.experts):                                  # every expert on every token,
                h = self.up[e](ctx, x, "toy.moe.h")                             # the choice applied as a mask
                act = torch.nn.functional.silu(h.float()).to(x.dtype)
                y = self.down[e](ctx, act, "toy.moe.y")
                out += y.float() * (choice == e).unsqueeze(1)
            return out.to(x.dtype)

    def read_spec(cfg):
        base = qwen3.read_spec(dict(cfg, architectures=["Qwen3ForCausalLM"], model_type="qwen3"))
        layers = []
        for layer in base.layers:
            pos = layer.mixer.position
            scaled = ScaledPositionSpec(kind="toy_rotary_scaled", theta=pos.theta, rotary_dim=pos.rotary_dim,
                                        head_dim=pos.head_dim, factor=cfg["toy_position_factor"])
            ff = RoutedSpec(kind="toy_top1", hidden_size=base.hidden_size,
                            intermediate_size=cfg["intermediate_size"], experts=cfg["toy_experts"])
            layers.append(LayerSpec(block=layer.block, mixer=dataclasses.replace(layer.mixer, position=scaled),
                                    feed_forward=ff, mixer_norm=layer.mixer_norm,
                                    feed_forward_norm=layer.feed_forward_norm, weight_prefix=layer.weight_prefix))
        return ModelSpec(architecture="ToyRoutedForCausalLM", hidden_size=base.hidden_size,
                         vocab_size=base.vocab_size, max_position_embeddings=base.max_position_embeddings,
                         layers=tuple(layers), run_order=base.run_order, final_norm=base.final_norm,
                         tie_word_embeddings=base.tie_word_embeddings)

    register_architecture("ToyRoutedForCausalLM", read_spec, lambda spec, mctx, src: DecoderModel(spec, mctx, src))


ROUTED_CONFIG = {
    "architectures": ["ToyRoutedForCausalLM"], "model_type": "toy", "toy_experts": 3, "toy_position_factor": 2.5,
    "num_hidden_layers": 2, "hidden_size": 56, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 40, "vocab_size": 90, "rope_theta": 5000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 160,
}


def plain_routed_logits(w, tokens):
    """Whole sequence, no cache; returns the logits and the smallest margin of any routing decision."""
    cfg = ROUTED_CONFIG
    w = {k: v.float().numpy().astype(np.float64) for k, v in w.items()}
    x = P.embedding(w["model.embed_tokens.weight"], tokens)
    pos = np.arange(len(tokens)) / cfg["toy_position_factor"]
    margin = np.inf
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        r = x + P.attention_part(n1, pos, w, p + "self_attn.", cfg)
        n2 = P.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        logits = P.linear(n2, w[p + "moe.router.weight"])
        top = np.sort(logits, axis=-1)
        margin = min(margin, float((top[:, -1] - top[:, -2]).min() / np.abs(logits).max()))
        choice = logits.argmax(-1)
        out = np.zeros_like(r)
        for t, e in enumerate(choice):
            h = P.silu(P.linear(n2[t:t + 1], w[p + f"moe.experts.{e}.up.weight"]))
            out[t] = P.linear(h, w[p + f"moe.experts.{e}.down.weight"])[0]
        x = r + out
    hn = P.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    return P.linear(hn, w["lm_head.weight"]), margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_position_encoding(dtype):
    from helpers import TOL, cut_bulk_tail, cut_portions, cut_whole, replay
    from safetyraise_lmengine_b200 import Engine, spec_from_config
    from safetyraise_lmengine_b200.parts.model import tensor_decls
    from safetyraise_lmengine_b200.weights.random_init import RandomWeights
    define_routed_toy()
    spec = spec_from_config(ROUTED_CONFIG)
    rng = np.random.default_rng(1)
    toks = [int(t) for t in rng.integers(0, 90, size=70)]
    # random weights whose routing decisions are all clear-cut, so that bfloat16 rounding cannot flip one
    for seed in range(64):
        src = RandomWeights(tensor_decls(spec), seed=seed)
        ref, margin = plain_routed_logits({n: src.get(n) for n in src.names()}, toks)
        if margin > 0.012:
            break
    else:
        pytest.fail("no seed with clear routing decisions")
    assert "model.layers.1.moe.experts.2.down.weight" in set(src.names())
    assert "model.layers.0.mlp.gate_proj.weight" not in set(src.names())
    eng = Engine.from_source(ROUTED_CONFIG, src, dtype=dtype, page_size=8, num_pages=40, max_requests=2,
                             max_batch_tokens=128)
    assert eng.use_graphs
    for steps in (cut_whole("x", toks), cut_bulk_tail("x", toks, 32), cut_portions("x", toks)):
        got = replay(eng, steps)
        rows = np.stack([got[("x", p)] for p in range(len(toks))])
        assert np.abs(rows - ref).max() <= TOL[dtype] * np.abs(ref).max()
    assert eng.graph_replays > 0                           # the decoded tail ran from recorded graphs
    assert eng.cache.audit() == 0
    # the position factor matters: without it the logits differ
    plain = dict(ROUTED_CONFIG, toy_position_factor=1.0)
    assert spec_from_config(plain).layers[0].mixer.position.factor == 1.0
