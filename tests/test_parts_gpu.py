"""Each part alone (norm, position encoding, attention mixer, feed-forward, block), built from its own
specification and random tensors, against the plain function of the same part."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def close(got: torch.Tensor, ref: np.ndarray, dt):
    got = got.float().cpu().numpy().astype(np.float64)
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() <= TOL[dt] * max(1.0, np.abs(ref).max()), np.abs(got - ref).max()


def make_ctx(dt, T, kv_heads=0, head_dim=0, page_size=4, entries=((0, None),), cache_entries=(0,)):
    """A StepContext for one or more whole sequences that start at position 0.
    entries: ((slot, length or None = T), ...)."""
    from safetyraise_lmengine_b200.cache.manager import PAGED_ALL, CacheGroupSpec, CacheManager
    from safetyraise_lmengine_b200.parts.base import StepContext, Workspace
    groups = [CacheGroupSpec("kv", PAGED_ALL, tuple(cache_entries), kv_heads, head_dim)] if kv_heads else []
    cache = CacheManager(groups, page_size, 64, 4, dt, DEV)
    lens = [T if n is None else n for _, n in entries]
    assert sum(lens) == T
    slots = []
    for _ in entries:
        slots.append(cache.open_request())
    for s, n in zip(slots, lens):
        assert cache.reserve(s, n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    pos = [p for n in lens for p in range(n)]
    eot = [e for e, n in enumerate(lens) for _ in range(n)]
    tables, kv_slot = {}, {}
    if kv_heads:
        width = max((n + page_size - 1) // page_size for n in lens)
        bt = torch.zeros(len(lens), width, dtype=torch.int32)
        ks = []
        for e, (s, n) in enumerate(zip(slots, lens)):
            tab = cache.table("kv", s)
            bt[e, :len(tab)] = torch.tensor(tab, dtype=torch.int32)
            ks += [tab[p // page_size] * page_size + p % page_size for p in range(n)]
        tables["kv"], kv_slot["kv"] = bt.to(DEV), i32(ks)
    return StepContext(
        T=T, n_entries=len(lens), token_ids=i32([0] * T), positions=i32(pos), entry_of_token=i32(eot),
        slots=i32(slots), cu_q=i32([0] + list(np.cumsum(lens))), kv_lens=i32(lens), logit_rows=i32([T - 1]),
        block_tables=tables, kv_slot=kv_slot,
        host={"q_lens": lens, "starts": [0] * len(lens), "kv_lens": lens, "slots": slots},
        cache=cache, workspace=Workspace(DEV, T), dtype=dt, max_q_len=max(lens), max_kv_len=max(lens),
        kv_bound=max(lens))


def mctx(dt, **options):
    from safetyraise_lmengine_b200.parts.base import ModelContext
    return ModelContext(DEV, dt, 256, dict(options))


def rand(shape, g, scale=1.0):
    return torch.randn(shape, generator=g) * scale


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H, eps", [(96, 1e-5), (257, 1e-6)])
def test_rmsnorm_part(dt, H, eps):
    from safetyraise_lmengine_b200.config.spec import NormSpec
    from safetyraise_lmengine_b200.parts.norm import RMSNorm
    g = torch.Generator().manual_seed(1)
    w = 1 + 0.1 * rand((H,), g)
    part = RMSNorm(NormSpec("rmsnorm", H, eps), "n.weight", {"n.weight": w.to(DEV)}, mctx(dt))
    res, delta = rand((9, H), g, 3.0), rand((9, H), g).to(dt)
    r = res.to(DEV).clone()
    out = torch.empty(9, H, device=DEV, dtype=dt)
    part.apply(r, delta.to(DEV), out)
    x = res.double().numpy() + delta.double().numpy()
    close(r, x, torch.float32)
    close(out, P.rms_norm(x, w.double().numpy(), eps), dt)


@pytest.mark.parametrize("theta, hd", [(1e4, 16), (1e6, 128)])
def test_rotary_part(theta, hd):
    from safetyraise_lmengine_b200.config.spec import PositionSpec
    from safetyraise_lmengine_b200.parts.position import RotaryHalf
    part = RotaryHalf(PositionSpec("rotary_half", theta, hd, hd), mctx(torch.float32))
    ctx = make_ctx(torch.float32, 50)
    rot = part.rotation(ctx)
    cos, sin = rot.cos, rot.sin
    assert part.rotation(ctx) is rot and part.applies == "rotation"       # made once per step
    assert rot.pairs == hd // 2 and not rot.interleaved
    x = np.random.default_rng(0).normal(size=(50, 3, hd))
    got = x.copy()
    c, s = cos.cpu().double().numpy()[:, None, :], sin.cpu().double().numpy()[:, None, :]
    half = hd // 2
    got[..., :half] = x[..., :half] * c - x[..., half:] * s
    got[..., half:] = x[..., half:] * c + x[..., :half] * s
    assert np.abs(got - P.rope(x, np.arange(50), theta, hd)).max() < 1e-6


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H, I, T", [(64, 128, 5), (96, 256, 40), (120, 200, 9), (100, 132, 7)])
def test_gated_dense_part(dt, H, I, T):
    from safetyraise_lmengine_b200.config.spec import FeedForwardSpec
    from safetyraise_lmengine_b200.parts.feedforward import GatedDense
    g = torch.Generator().manual_seed(2)
    w = {"L.mlp.gate_proj.weight": rand((I, H), g, 0.1), "L.mlp.up_proj.weight": rand((I, H), g, 0.1),
         "L.mlp.down_proj.weight": rand((H, I), g, 0.1)}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    x = rand((T, H), g).to(dt)
    ref = P.feed_forward_part(x.double().numpy(), {k: v.double().numpy() for k, v in w.items()}, "L.mlp.")
    for unfused in (False, True):
        part = GatedDense(FeedForwardSpec("gated_dense", H, I), "L.", {k: v.to(DEV).to(dt) for k, v in w.items()},
                          mctx(dt, unfused_swiglu=unfused))
        assert part.fused == (dt == torch.bfloat16 and not unfused and H % 8 == 0 and I % 8 == 0)
        out = part.forward(make_ctx(dt, T), x.to(DEV))
        close(out, ref, dt)


def attention_case(dt, hidden, nq, nkv, hd, T, theta=1e4, eps=1e-6):
    from safetyraise_lmengine_b200.config.spec import AttentionSpec, NormSpec, PositionSpec
    g = torch.Generator().manual_seed(3)
    p = "L.self_attn."
    w = {p + "q_proj.weight": rand((nq * hd, hidden), g, 0.08), p + "k_proj.weight": rand((nkv * hd, hidden), g, 0.08),
         p + "v_proj.weight": rand((nkv * hd, hidden), g, 0.08), p + "o_proj.weight": rand((hidden, nq * hd), g, 0.08)}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    w[p + "q_norm.weight"] = 1 + 0.1 * rand((hd,), g)
    w[p + "k_norm.weight"] = 1 + 0.1 * rand((hd,), g)
    spec = AttentionSpec(kind="paged_attention", hidden_size=hidden, heads=nq, kv_heads=nkv, head_dim=hd,
                         qk_norm=NormSpec("rmsnorm", hd, eps), position=PositionSpec("rotary_half", theta, hd, hd),
                         softmax_scale=1 / math.sqrt(hd))
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": hidden,
           "rms_norm_eps": eps, "rope_theta": theta}
    dev_w = {k: (v.to(DEV) if "norm" in k else v.to(DEV).to(dt)) for k, v in w.items()}
    return spec, cfg, w, dev_w, rand((T, hidden), g).to(dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("hidden, nq, nkv, hd, T", [(64, 4, 2, 16, 23), (96, 6, 1, 32, 50), (128, 4, 4, 64, 70),
                                                   (120, 5, 5, 48, 19)])
def test_attention_part(dt, hidden, nq, nkv, hd, T):
    from safetyraise_lmengine_b200.config.spec import RunStep
    from safetyraise_lmengine_b200.parts.attention import PagedAttention
    spec, cfg, w, dev_w, x = attention_case(dt, hidden, nq, nkv, hd, T)
    part = PagedAttention(spec, "L.", dev_w, mctx(dt))
    need = part.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim) == ("paged_all", nkv, hd)
    # two sequences in one batch: each attends to itself only
    split = T // 3
    ctx = make_ctx(dt, T, nkv, hd, entries=((0, split), (1, T - split)))
    out = part.forward(ctx, x.to(DEV), RunStep(0, 0, True))
    wn = {k: v.double().numpy() for k, v in w.items()}
    xs = x.double().numpy()
    ref = np.concatenate([P.attention_part(xs[:split], np.arange(split), wn, "L.self_attn.", cfg),
                          P.attention_part(xs[split:], np.arange(T - split), wn, "L.self_attn.", cfg)])
    close(out, ref, dt)


@pytest.mark.parametrize("dt", DTYPES)
def test_block_part(dt):
    from safetyraise_lmengine_b200.config.spec import FeedForwardSpec, LayerSpec, NormSpec, RunStep
    from safetyraise_lmengine_b200.parts.block import PreNormBlock
    hidden, nq, nkv, hd, I, T = 96, 6, 2, 32, 160, 31
    spec_a, cfg, w, dev_w, x = attention_case(dt, hidden, nq, nkv, hd, T, eps=1e-5)
    g = torch.Generator().manual_seed(4)
    extra = {"L.mlp.gate_proj.weight": rand((I, hidden), g, 0.1).to(torch.bfloat16),
             "L.mlp.up_proj.weight": rand((I, hidden), g, 0.1).to(torch.bfloat16),
             "L.mlp.down_proj.weight": rand((hidden, I), g, 0.1).to(torch.bfloat16),
             "L.input_layernorm.weight": 1 + 0.1 * rand((hidden,), g),
             "L.post_attention_layernorm.weight": 1 + 0.1 * rand((hidden,), g)}
    w.update(extra)
    dev_w.update({k: (v.to(DEV) if "norm" in k else v.to(DEV).to(dt)) for k, v in extra.items()})
    layer = LayerSpec("pre_norm", spec_a, FeedForwardSpec("gated_dense", hidden, I), NormSpec("rmsnorm", hidden, 1e-5),
                      NormSpec("rmsnorm", hidden, 1e-5), "L.")
    names = {d.name for d in PreNormBlock.tensor_decls(layer)}
    assert names == set(w)
    block = PreNormBlock(layer, dev_w, mctx(dt))
    ctx = make_ctx(dt, T, nkv, hd)
    residual = x.float().to(DEV).clone()
    pending = block.forward(ctx, residual, None, RunStep(0, 0, True))
    got = residual + pending.float() if pending is not None else residual
    wn = {("model.layers.0." + k[2:]): v.double().numpy() for k, v in w.items()}
    cfg.update(intermediate_size=I)
    ref = P.block(x.double().numpy(), np.arange(T), wn, 0, cfg)
    close(got, ref, dt)
