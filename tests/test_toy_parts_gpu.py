"""Generality of the part system.  Three toy architectures are defined HERE, registered, built and
stepped without touching the package: (1) a mixer with state of its own beside attention, a layer
that runs twice, and a learned position table added to the embedding; (2) the framework's attention
under a rotary encoding with interleaved pairs and scaled positions, with a routed feed-forward;
(3) the framework's attention with a window, whose pages are given back as the window passes them."""
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
    from safetyraise_lmengine_b200.config.spec import LayerSpec, MixerSpec, ModelSpec, PositionSpec, RunStep
    from safetyraise_lmengine_b200.parts import EMBEDDING, CacheNeed, Part, register_mixer, register_position_encoding
    from safetyraise_lmengine_b200.parts.linear import Linear
    from safetyraise_lmengine_b200.parts.model import DecoderModel
    from safetyraise_lmengine_b200.weights.loader import MATRIX, TABLE, TensorDecl
    if "ToyEmaForCausalLM" in ARCHITECTURES:
        return

    @dataclass(frozen=True)
    class LearnedSpec(PositionSpec):
        positions: int = 0
        hidden_size: int = 0

    @register_position_encoding("toy_learned")
    class LearnedPositions(Part):
        """x[t] += table[position of t]: an encoding that acts on the embedding, not on q and k."""
        applies = EMBEDDING

        def __init__(self, spec, mctx, tensors, name):
            self.table = tensors[name]

        @classmethod
        def tensor_decls(cls, spec, name):
            return [TensorDecl(name, (spec.positions, spec.hidden_size), TABLE)]

        def add_to_embedding(self, ctx, residual):
            residual += self.table.float().index_select(0, ctx.positions.long())

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

        @classmethod
        def cache_need_of(cls, spec):
            return CacheNeed(FIXED_STATE, state_shape=(spec.hidden_size,), state_dtype=torch.float32)

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
                         tie_word_embeddings=base.tie_word_embeddings,
                         embed_position=LearnedSpec(kind="toy_learned", positions=base.max_position_embeddings,
                                                    hidden_size=base.hidden_size))

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
    pos = np.arange(len(tokens))
    x = P.embedding(w["model.embed_tokens.weight"], tokens) + w["model.embed_positions.weight"][pos]

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
    from safetyraise_lmengine_b200.parts import (ROTATION, Part, Rotation, register_feed_forward,
                                                 register_position_encoding)
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
        """Angles (pos / factor) / theta^(2i/rotary_dim) on INTERLEAVED pairs (2i, 2i+1) of the first
        rotary_dim elements of a head: the encoding says so in the Rotation it hands to the mixer."""
        applies = ROTATION

        def __init__(self, spec, mctx):
            self.spec, self.half = spec, spec.rotary_dim // 2
            self.key = ("toy_rotary_scaled", spec.theta, spec.rotary_dim, spec.factor)

        def rotation(self, ctx):
            got = ctx.tables.get(self.key)
            if got is None:
                i = torch.arange(self.half, device=ctx.positions.device, dtype=torch.float64)
                inv = self.spec.theta ** (-2.0 * i / self.spec.rotary_dim)
                ang = (ctx.positions.double() / self.spec.factor)[:, None] * inv[None, :]
                got = ctx.tables[self.key] = Rotation(ang.cos().float().contiguous(), ang.sin().float().contiguous(),
                                                      self.half, interleaved=True)
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
            scaled = ScaledPositionSpec(kind="toy_rotary_scaled", theta=pos.theta,
                                        rotary_dim=cfg["toy_rotary_dim"], head_dim=pos.head_dim,
                                        factor=cfg["toy_position_factor"])
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
    "toy_rotary_dim": 12,
    "num_hidden_layers": 2, "hidden_size": 56, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 40, "vocab_size": 90, "rope_theta": 5000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 160,
}


def rope_interleaved(x, positions, theta, rotary_dim):
    """Pairs (2i, 2i+1) of the first rotary_dim elements of x[T, heads, head_dim]; angles as P.rope."""
    half = rotary_dim // 2
    ang = positions[:, None] / np.power(theta, 2.0 * np.arange(half) / rotary_dim)[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    even, odd = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
    out[..., 0:rotary_dim:2] = even * cos - odd * sin
    out[..., 1:rotary_dim:2] = odd * cos + even * sin
    return out


def attention_interleaved(n1, positions, w, prefix, cfg, window=None):
    """The attention part of plain_qwen3 with the rotation above and, optionally, a window of keys."""
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = n1.shape[0]
    q = P.rms_norm(P.linear(n1, w[prefix + "q_proj.weight"]).reshape(T, nq, hd), w[prefix + "q_norm.weight"],
                   cfg["rms_norm_eps"])
    k = P.rms_norm(P.linear(n1, w[prefix + "k_proj.weight"]).reshape(T, nkv, hd), w[prefix + "k_norm.weight"],
                   cfg["rms_norm_eps"])
    v = P.linear(n1, w[prefix + "v_proj.weight"]).reshape(T, nkv, hd)
    if cfg.get("toy_rotary_dim"):
        q = rope_interleaved(q, positions, cfg["rope_theta"], cfg["toy_rotary_dim"])
        k = rope_interleaved(k, positions, cfg["rope_theta"], cfg["toy_rotary_dim"])
    else:
        q, k = P.rope(q, positions, cfg["rope_theta"], hd), P.rope(k, positions, cfg["rope_theta"], hd)
    out = np.zeros_like(q)
    for h in range(nq):
        s = (q[:, h] @ k[:, h // (nq // nkv)].T) / math.sqrt(hd)
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        seen = (j <= i) if window is None else (j <= i) & (j > i - window)     # a query sees itself and window-1 before
        s = np.where(seen, s, -np.inf)
        pr = np.exp(s - s.max(-1, keepdims=True))
        out[:, h] = (pr / pr.sum(-1, keepdims=True)) @ v[:, h // (nq // nkv)]
    return P.linear(out.reshape(T, nq * hd), w[prefix + "o_proj.weight"])


def plain_routed_logits(w, tokens, factor=None):
    """Whole sequence, no cache; returns the logits and the smallest margin of any routing decision."""
    cfg = ROUTED_CONFIG
    w = {k: v.float().numpy().astype(np.float64) for k, v in w.items()}
    x = P.embedding(w["model.embed_tokens.weight"], tokens)
    pos = np.arange(len(tokens)) / (factor or cfg["toy_position_factor"])
    margin = np.inf
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        r = x + attention_interleaved(n1, pos, w, p + "self_attn.", cfg)
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
    for seed in (163, *range(256)):      # 163: found by this same search
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
    # the encoding's constants and its pairing matter: the engine's logits are far from those of a plain
    # model with unscaled positions, and from those of plain_qwen3's half-split rotation
    unscaled, _ = plain_routed_logits({n: src.get(n) for n in src.names()}, toks, factor=1.0)
    assert np.abs(rows - unscaled).max() > 0.2 * np.abs(ref).max()


# ---------------------------------------------------------------------------
# Fixed-size state under failure, and under the generation loop
# ---------------------------------------------------------------------------
def ema_engine(dtype="float32", **kw):
    from safetyraise_lmengine_b200 import Engine, spec_from_config
    from safetyraise_lmengine_b200.parts.model import tensor_decls
    from safetyraise_lmengine_b200.weights.random_init import RandomWeights
    define_toy()
    src = RandomWeights(tensor_decls(spec_from_config(TOY_CONFIG)), seed=3)
    kw.setdefault("num_pages", 64)
    eng = Engine.from_source(TOY_CONFIG, src, dtype=dtype, page_size=4, max_requests=3, max_batch_tokens=128, **kw)
    return eng, {n: src.get(n) for n in src.names()}


def test_a_failed_step_leaves_fixed_size_state_as_it_was():
    """State of fixed size cannot be truncated: the engine keeps what the step's slots held and puts it
    back when the step fails (the failure is a fault word raised from the host)."""
    from helpers import TOL
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import StepFailed
    eng, w = ema_engine()
    rng = np.random.default_rng(5)
    toks = [int(t) for t in rng.integers(0, 100, size=30)]
    ref = plain_toy_logits(w, toks)
    s = eng.open_request()
    eng.step([StepEntry(s, toks[:11], [])])
    state = eng.cache.state_of_entry(1)[s].clone()
    assert float(state.abs().max()) > 0
    eng.status[2] = 1
    with pytest.raises(StepFailed):
        eng.step([StepEntry(s, toks[11:19], [7])])                   # ran, and overwrote the slot's state
    assert torch.equal(eng.cache.state_of_entry(1)[s], state) and eng.cache.length(s) == 11
    got = eng.step([StepEntry(s, toks[11:], list(range(19)))]).cpu().numpy()
    assert np.abs(got - ref[11:]).max() <= TOL["float32"] * np.abs(ref).max()
    assert eng.cache.audit() == 0


def test_generation_loop_starts_every_occupant_of_a_slot_from_zero_state():
    """Requests one after the other on the same slot, and a request that is thrown out and computed
    again, all through the scheduler, which opens slots itself: each must start from a zero state."""
    from safetyraise_lmengine_b200 import LLM, EngineConfig, SamplingParams

    def greedy(w, prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(plain_toy_logits(w, toks)[-1].argmax()))
        return toks[len(prompt):]

    rng = np.random.default_rng(8)
    prompts = [[int(t) for t in rng.integers(0, 100, size=n)] for n in (14, 9, 17)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=6)
    # one slot: the three requests follow each other on it
    eng, w = ema_engine()
    want = [greedy(w, p, 6) for p in prompts]
    llm = LLM(eng, EngineConfig(max_active=1, queue_capacity=4, page_size=4, max_batch_tokens=128,
                                prefill_chunk=8, max_context=128, dtype="float32"))
    assert [r.tokens for r in llm.generate(prompts, sp)] == want
    # three slots and few pages: the youngest is preempted and recomputed from its first token
    eng, _ = ema_engine(num_pages=14)
    llm = LLM(eng, EngineConfig(max_active=3, queue_capacity=4, page_size=4, max_batch_tokens=128,
                                prefill_chunk=8, max_context=128, dtype="float32"))
    got = llm.generate(prompts, sp)
    assert [r.tokens for r in got] == want
    assert llm.metrics()["preempted"] > 0 and eng.cache.audit() == 0 and eng.cache.free_pages() == 14


# ---------------------------------------------------------------------------
# A third toy architecture: the framework's attention with a window of 10 keys (a `paged_window`
# cache group: pages that the window has passed are given back at commit and used again).
# ---------------------------------------------------------------------------
WINDOW = 10
WINDOW_CONFIG = {
    "architectures": ["ToyWindowForCausalLM"], "model_type": "toy", "toy_window": WINDOW,
    "num_hidden_layers": 2, "hidden_size": 40, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 56, "vocab_size": 70, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 160,
}


def define_window_toy():
    import dataclasses

    from safetyraise_lmengine_b200 import ARCHITECTURES, register_architecture
    from safetyraise_lmengine_b200.config import qwen3
    from safetyraise_lmengine_b200.parts.model import DecoderModel
    if "ToyWindowForCausalLM" in ARCHITECTURES:
        return

    def read_spec(cfg):
        base = qwen3.read_spec(dict(cfg, architectures=["Qwen3ForCausalLM"], model_type="qwen3"))
        layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, window=cfg["toy_window"]))
                       for l in base.layers)
        return dataclasses.replace(base, architecture="ToyWindowForCausalLM", layers=layers)

    register_architecture("ToyWindowForCausalLM", read_spec, lambda spec, mctx, src: DecoderModel(spec, mctx, src))


def plain_window_logits(w, tokens):
    cfg = WINDOW_CONFIG
    w = {k: v.float().numpy().astype(np.float64) for k, v in w.items()}
    x = P.embedding(w["model.embed_tokens.weight"], tokens)
    pos = np.arange(len(tokens), dtype=np.float64)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        r = x + attention_interleaved(n1, pos, w, p + "self_attn.", cfg, window=WINDOW)
        n2 = P.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = r + P.feed_forward_part(n2, w, p + "mlp.")
    return P.linear(P.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_window_attention_gives_pages_back_and_matches_plain(dtype):
    """A window's edge inside a prompt portion, decoding far past the window after its pages were given
    back, and so few pages that the ones given back are the ones used next.  With a window of 10 every
    visible key carries about a tenth of the weight, so a window off by one key moves the logits far
    beyond the tolerance."""
    from helpers import TOL, cut_bulk_tail, cut_portions, replay
    from safetyraise_lmengine_b200 import Engine, spec_from_config
    from safetyraise_lmengine_b200.parts.model import tensor_decls
    from safetyraise_lmengine_b200.weights.random_init import RandomWeights
    define_window_toy()
    spec = spec_from_config(WINDOW_CONFIG)
    src = RandomWeights(tensor_decls(spec), seed=11)
    w = {n: src.get(n) for n in src.names()}
    rng = np.random.default_rng(2)
    toks = [int(t) for t in rng.integers(0, 70, size=75)]
    ref = plain_window_logits(w, toks)
    # the window's edge is there: the same weights with one key more or less give other logits
    global WINDOW
    for other in (WINDOW - 1, WINDOW + 1):
        keep, WINDOW = WINDOW, other
        try:
            assert np.abs(plain_window_logits(w, toks) - ref).max() > 0.05 * np.abs(ref).max()
        finally:
            WINDOW = keep
    # a step of 64 tokens holds its own keys and the window before it: 19 pages of 4 at most; 20 exist
    eng = Engine.from_source(WINDOW_CONFIG, src, dtype=dtype, page_size=4, num_pages=20, max_requests=2,
                             max_batch_tokens=128)
    assert [g.kind for g in eng.cache.groups] == ["paged_window"]
    for pool in eng.cache.kv_pools.values():
        pool.fill_(float("nan"))                      # a page read after it was given back would show
    decode_all = [{"entries": [("x", toks[i:i + 1], [0])]} for i in range(len(toks))]     # 7 windows deep
    for steps in (cut_portions("x", toks), cut_bulk_tail("x", toks, 32), decode_all):
        got = replay(eng, steps)
        rows = np.stack([got[("x", p)] for p in range(len(toks))])
        err = np.abs(rows - ref).max(axis=1) / np.abs(ref).max()
        assert err.max() <= TOL[dtype], f"first wrong position {int(np.argmax(err > TOL[dtype]))}"
        assert eng.cache.audit() == 0 and eng.cache.free_pages() == 20
    taken, reused = eng.cache.reuse_counts()
    assert reused > 0 and taken > 20


# ---------------------------------------------------------------------------
# A fourth toy architecture, data only: the framework's own parts in a run order whose last step runs
# layer 0's weights again and reads the keys and values that the first step wrote (it appends nothing).
# ---------------------------------------------------------------------------
SHARED_CONFIG = {
    "architectures": ["ToySharedForCausalLM"], "model_type": "toy",
    "num_hidden_layers": 2, "hidden_size": 72, "num_attention_heads": 2, "num_key_value_heads": 1,
    "head_dim": 64, "intermediate_size": 104, "vocab_size": 110, "rope_theta": 8000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256,
}


def define_shared_toy():
    import dataclasses

    from safetyraise_lmengine_b200 import ARCHITECTURES, register_architecture
    from safetyraise_lmengine_b200.config import qwen3
    from safetyraise_lmengine_b200.config.spec import RunStep
    from safetyraise_lmengine_b200.parts.model import DecoderModel
    if "ToySharedForCausalLM" in ARCHITECTURES:
        return

    def read_spec(cfg):
        base = qwen3.read_spec(dict(cfg, architectures=["Qwen3ForCausalLM"], model_type="qwen3"))
        order = (RunStep(0, 0), RunStep(1, 1), RunStep(0, 0, writes_cache=False))
        return dataclasses.replace(base, architecture="ToySharedForCausalLM", run_order=order)

    register_architecture("ToySharedForCausalLM", read_spec, lambda spec, mctx, src: DecoderModel(spec, mctx, src))


def plain_shared_logits(w, tokens):
    cfg = SHARED_CONFIG
    w = {k: v.float().numpy().astype(np.float64) for k, v in w.items()}
    nq, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    T = len(tokens)
    pos = np.arange(T)
    x = P.embedding(w["model.embed_tokens.weight"], tokens)
    p = "model.layers.0."
    # the first step's keys and values, as it leaves them in the cache
    n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], eps)
    k = P.rope(P.rms_norm(P.linear(n1, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd),
                          w[p + "self_attn.k_norm.weight"], eps), pos, cfg["rope_theta"], hd)
    v = P.linear(n1, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
    x = P.block(x, pos, w, 0, cfg)
    x = P.block(x, pos, w, 1, cfg)
    # the last step: layer 0's weights on the new hidden state, queries only
    n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = P.rope(P.rms_norm(P.linear(n1, w[p + "self_attn.q_proj.weight"]).reshape(T, nq, hd),
                          w[p + "self_attn.q_norm.weight"], eps), pos, cfg["rope_theta"], hd)
    r = x + P.linear(P.causal_attention(q, k, v).reshape(T, nq * hd), w[p + "self_attn.o_proj.weight"])
    n2 = P.rms_norm(r, w[p + "post_attention_layernorm.weight"], eps)
    x = r + P.feed_forward_part(n2, w, p + "mlp.")
    return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_run_step_reads_the_cache_that_another_step_wrote(dtype):
    """Three steps over two layers; the third attends over the first one's keys, this step's among them
    (written a few kernels earlier in the same forward pass), in prompts, portions and decode steps that are
    replayed from CUDA graphs."""
    from helpers import TOL, cut_bulk_tail, cut_portions, cut_whole, replay
    from safetyraise_lmengine_b200 import Engine, spec_from_config
    from safetyraise_lmengine_b200.parts.model import tensor_decls
    from safetyraise_lmengine_b200.weights.random_init import RandomWeights
    define_shared_toy()
    spec = spec_from_config(SHARED_CONFIG)
    src = RandomWeights(tensor_decls(spec), seed=5)
    w = {n: src.get(n) for n in src.names()}
    rng = np.random.default_rng(4)
    toks = [int(t) for t in rng.integers(0, 110, size=90)]
    ref = plain_shared_logits(w, toks)
    # the shared keys matter: with the last step attending over keys of its own the logits are others
    w64 = {k: v.float().numpy().astype(np.float64) for k, v in w.items()}
    x, pos = P.embedding(w64["model.embed_tokens.weight"], toks), np.arange(len(toks))
    for layer in (0, 1, 0):
        x = P.block(x, pos, w64, layer, SHARED_CONFIG)
    own = P.linear(P.rms_norm(x, w64["model.norm.weight"], 1e-6), w64["model.embed_tokens.weight"])
    assert np.abs(own - ref).max() > 0.05 * np.abs(ref).max()
    eng = Engine.from_source(SHARED_CONFIG, src, dtype=dtype, page_size=16, num_pages=24, max_requests=2,
                             max_batch_tokens=128)
    paged = [g for g in eng.cache.groups if g.kind == "paged_all"][0]
    assert paged.entries == (0, 1)                       # two cache entries for three steps
    for steps in (cut_whole("x", toks), cut_bulk_tail("x", toks, 32), cut_portions("x", toks)):
        got = replay(eng, steps)
        rows = np.stack([got[("x", p)] for p in range(len(toks))])
        err = np.abs(rows - ref).max(axis=1) / np.abs(ref).max()
        assert err.max() <= TOL[dtype], f"first wrong position {int(np.argmax(err > TOL[dtype]))}"
    assert eng.cache.audit() == 0
    if dtype == "bfloat16":
        assert eng.graph_replays >= 20
