"""The engine against the plain implementation, under every way of cutting the work."""
import numpy as np
import pytest
import torch
from conftest import TINY
from helpers import (TOL, check_against_plain, cut_bulk_tail, cut_portions, cut_whole, note_error, plain_logits,
                     random_tokens, rel_err, replay)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def build(folder, dtype, num_pages=64, page_size=16, **kw):
    from safetyraise_lmengine_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages,
                              max_requests=4, max_batch_tokens=512, **kw)


def requests_for(name, seed=0):
    cfg, _ = TINY[name]
    rng = np.random.default_rng(100 + seed)
    lens = [5, 11, 17, 70] if name in ("A", "C") else [1, 7, 33, 64, 100]
    return {f"r{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate(lens)}


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_requests_alone(tiny_folder, dtype):
    name, folder = tiny_folder
    eng = build(folder, dtype)
    reqs = requests_for(name)
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_whole(rid, toks)))
    check_against_plain(got, folder, reqs, dtype)
    assert eng.cache.audit() == 0 and eng.cache.free_pages() == 64


@pytest.mark.parametrize("dtype", DTYPES)
def test_bulk_then_last_32_one_by_one(tiny_folder, dtype):
    name, folder = tiny_folder
    eng = build(folder, dtype)
    reqs = {k: v for k, v in requests_for(name).items() if len(v) >= 33}
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_bulk_tail(rid, toks, 32)))
    check_against_plain(got, folder, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [4, 16])
def test_portions_of_changing_size(tiny_folder, dtype, page_size):
    name, folder = tiny_folder
    eng = build(folder, dtype, num_pages=40, page_size=page_size)
    reqs = requests_for(name)
    got = {}
    for rid, toks in reqs.items():
        if len(toks) < 2:
            continue
        got.update(replay(eng, cut_portions(rid, toks)))
    check_against_plain(got, folder, {k: v for k, v in reqs.items() if len(v) >= 2}, dtype)


def mixed_schedule(reqs, chunk=8):
    """Up to four live requests; portions of prompts beside single tokens of requests whose last 6
    tokens are fed one at a time; a finished request's pages go to the next one."""
    order = list(reqs)
    live, waiting, steps = [], list(order), []
    fed = {r: 0 for r in order}
    while live or waiting:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, ended = [], []
        for r in live:
            toks = reqs[r]
            left = len(toks) - fed[r]
            n = 1 if left <= 6 else min(chunk + (len(steps) % 3), left - 6)
            entries.append((r, toks[fed[r]:fed[r] + n], list(range(n))))
            fed[r] += n
            if fed[r] == len(toks):
                ended.append(r)
        steps.append({"entries": entries, "end": ended})
        live = [r for r in live if r not in ended]
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page", [4, 16])
def test_mixed_batches_with_page_reuse(tiny_folder, dtype, page):
    name, folder = tiny_folder
    cfg, _ = TINY[name]
    rng = np.random.default_rng(7)
    lens = [23, 9, 41, 30, 17, 55, 12, 38]
    reqs = {f"m{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate(lens)}
    # room for the four largest at once, far less than all eight: pages must be used again
    num_pages = sum(sorted((n + page - 1) // page for n in lens)[-4:])
    eng = build(folder, dtype, num_pages=num_pages, page_size=page)
    # poison the pools so that a stale or unwritten page shows
    for pool in eng.cache.kv_pools.values():
        pool.fill_(float("nan"))
    got = replay(eng, mixed_schedule(reqs))
    check_against_plain(got, folder, reqs, dtype)
    taken, reused = eng.cache.reuse_counts()
    assert reused > 0 and taken > num_pages
    assert eng.cache.audit() == 0 and eng.cache.free_pages() == num_pages


@pytest.mark.parametrize("dtype", DTYPES)
def test_folders_stored_as_f32_and_f16_through_the_cuttings(stored_folder, dtype):
    """Matrices stored in 32 bits stay in 32 bits (in a bfloat16 engine they run the float32 product
    between bfloat16 activations); matrices stored as F16 are widened for the float32 engine and
    rounded to bfloat16 for the other.  Their values are not representable in bfloat16, so the float32
    engine is shown weights that bfloat16 cannot hold."""
    name, store, folder = stored_folder
    eng = build(folder, dtype, num_pages=40, page_size=4)
    w = eng.model.blocks[0].mixer.qkv.weight
    assert w.dtype == (torch.float32 if store == "F32" or dtype == "float32" else torch.bfloat16)
    if dtype == "float32":
        assert not torch.equal(w, w.to(torch.bfloat16).float())            # more bits than bfloat16 holds
    reqs = requests_for(name, seed=3)
    long = {k: v for k, v in reqs.items() if len(v) >= 33}
    for cut, which in ((cut_whole, reqs), (cut_bulk_tail, long), (cut_portions, {k: v for k, v in reqs.items() if len(v) >= 2})):
        got = {}
        for rid, toks in which.items():
            got.update(replay(eng, cut(rid, toks)))
        check_against_plain(got, folder, which, dtype)
    cfg, _ = TINY[name]
    rng = np.random.default_rng(17)
    mixed = {f"m{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate([23, 9, 41, 30, 17, 38])}
    tight = build(folder, dtype, num_pages=sum(sorted((n + 3) // 4 for n in (23, 9, 41, 30, 17, 38))[-4:]), page_size=4)
    check_against_plain(replay(tight, mixed_schedule(mixed)), folder, mixed, dtype)
    assert tight.cache.reuse_counts()[1] > 0 and tight.cache.audit() == 0


@pytest.mark.parametrize("name", ["E", "F"])
def test_decode_steps_with_large_head_groups_replay_graphs(name, tmp_path_factory):
    """More than 16 query heads per KV head: a decode step runs the rows-split attention kernel, whose
    work list must be on the device before a CUDA graph of the step is recorded.  The decoded tail of
    32 tokens runs from the recorded graph and must agree with the plain implementation."""
    from conftest import make_folder
    cfg, seed = TINY[name]
    folder = make_folder(tmp_path_factory, cfg, seed, "groups_" + name.lower())
    eng = build(folder, "bfloat16")
    assert eng.use_graphs
    reqs = {k: v for k, v in requests_for(name).items() if len(v) >= 64}
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_bulk_tail(rid, toks, 32)))
    check_against_plain(got, folder, reqs, "bfloat16")
    assert eng.graph_replays >= 30 * len(reqs) - 4
    # two requests decoding side by side, one graph for both
    two = dict(list(requests_for(name, seed=1).items())[-2:])
    steps = [{"entries": [(r, t[:40], list(range(40))) for r, t in two.items()]}]
    steps += [{"entries": [(r, t[40 + i:41 + i], [0]) for r, t in two.items()]} for i in range(24)]
    two = {r: t[:64] for r, t in two.items()}
    before = eng.graph_replays
    check_against_plain(replay(eng, steps), folder, two, "bfloat16")
    assert eng.graph_replays >= before + 20


@pytest.mark.parametrize("which", ["B", "G", "long"])
def test_mixed_steps_send_their_decoding_requests_to_the_keys_split_kernel(which, tmp_path_factory, long_prompt_folder):
    """With many decoding requests of similar length beside a portion, a mixed step runs two attention
    launches: the decoding requests at the head and at the tail of the batch on the keys-split kernel, the
    rest on the rows-split one.  The threshold is lowered so that four requests reach it."""
    from conftest import make_folder
    from safetyraise_lmengine_b200.kernels import ops
    if which == "long":
        folder, vocab = long_prompt_folder, 512
    else:
        cfg, seed = TINY[which]
        folder, vocab = make_folder(tmp_path_factory, cfg, seed, "split_" + which.lower()), cfg["vocab_size"]
    rng = np.random.default_rng(31)
    reqs = {r: random_tokens(rng, n, vocab) for r, n in (("a", 70), ("b", 66), ("p", 90), ("c", 72))}
    # a, b and c are fed whole but for their last 12 tokens, which then come one by one beside portions of p;
    # the order a, b, p, c puts decoding requests at the head and at the tail of the batch
    steps = [{"entries": [(r, reqs[r][:-12], []) for r in ("a", "b", "c")]}]
    for i in range(12):
        entries = [(r, reqs[r][len(reqs[r]) - 12 + i:len(reqs[r]) - 11 + i], [0]) for r in ("a", "b")]
        lo, hi = (0, 35) if i == 0 else (35 + 5 * (i - 1), 35 + 5 * i)
        entries.append(("p", reqs["p"][lo:hi], list(range(hi - lo))))
        entries.append(("c", reqs["c"][len(reqs["c"]) - 12 + i:len(reqs["c"]) - 11 + i], [0]))
        steps.append({"entries": entries})
    keep = ops.split_mixed_min_blocks
    ops.split_mixed_min_blocks = 1
    try:
        eng = Engine_for(folder)
        ops.begin_timing()
        got = replay(eng, steps)
        names = set(k.split("[")[0] for k in ops.end_timing())
    finally:
        ops.split_mixed_min_blocks = keep
    assert names & {"paged_attention_decode_tma", "paged_attention_keys"}, names
    assert names & {"paged_attention_rows", "paged_attention_rows_tma", "paged_attention_prefill_tcgen05"}, names
    ref = {r: plain_logits(folder, t) for r, t in reqs.items()}
    worst = 0.0
    for (r, pos), row in got.items():
        worst = max(worst, np.abs(row - ref[r][pos]).max() / np.abs(ref[r]).max())
    assert len(got) == 3 * 12 + 90 and worst <= TOL["bfloat16"], worst


def Engine_for(folder):
    from safetyraise_lmengine_b200 import Engine
    return Engine.from_folder(folder, dtype="bfloat16", page_size=16, num_pages=64, max_requests=4,
                              max_batch_tokens=512, options={"cuda_graphs": False})


@pytest.mark.parametrize("dtype", DTYPES)
def test_cuttings_agree_with_each_other(folder_b, dtype):
    """Beyond agreeing with the oracle: the float32 path gives the same bits however the work is cut."""
    eng = build(folder_b, dtype)
    toks = requests_for("B")["r4"]
    a = replay(eng, cut_whole("x", toks))
    b = replay(eng, cut_bulk_tail("x", toks, 32))
    c = replay(eng, cut_portions("x", toks))
    for p in range(len(toks)):
        if dtype == "float32":
            assert np.array_equal(a[("x", p)], b[("x", p)]) and np.array_equal(a[("x", p)], c[("x", p)]), p
        else:
            scale = np.abs(a[("x", p)]).max()
            assert np.abs(a[("x", p)] - b[("x", p)]).max() <= TOL[dtype] * scale
            assert np.abs(a[("x", p)] - c[("x", p)]).max() <= TOL[dtype] * scale


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decoding(folder_b, dtype):
    cfg, _ = TINY["B"]
    rng = np.random.default_rng(3)
    toks = random_tokens(rng, 200, cfg["vocab_size"])
    eng = build(folder_b, dtype)
    steps = [{"entries": [("d", toks[i:i + 1], [0])]} for i in range(len(toks))]
    got = replay(eng, steps)
    check_against_plain(got, folder_b, {"d": toks}, dtype)


def test_refused_step_changes_nothing(folder_a):
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import ResourceExhausted, ShapeError
    eng = build(folder_a, "float32", num_pages=3, page_size=4)
    s = eng.open_request()
    ref = eng.step([StepEntry(s, [1, 2, 3, 4, 5], [4])]).cpu().numpy().copy()
    free = eng.cache.free_pages()
    with pytest.raises(ShapeError):
        eng.step([StepEntry(s, [1, 999], [0])])                  # id outside the vocabulary
    with pytest.raises(ResourceExhausted):
        eng.step([StepEntry(s, list(range(20)), [0])])            # more pages than exist
    with pytest.raises(ShapeError):
        eng.step([StepEntry(s, [], [])])
    assert eng.cache.length(s) == 5 and eng.cache.free_pages() == free and eng.cache.audit() == 0
    eng.close_request(s)
    s2 = eng.open_request()
    again = eng.step([StepEntry(s2, [1, 2, 3, 4, 5], [4])]).cpu().numpy()
    assert np.array_equal(ref, again)


def test_recorded_decode_steps_equal_eager_ones(folder_b):
    """Decode-only steps replay a CUDA graph from their third occurrence on: same logits as eager."""
    cfg, _ = TINY["B"]
    rng = np.random.default_rng(9)
    prompts = {r: random_tokens(rng, n, cfg["vocab_size"]) for r, n in (("p", 20), ("q", 33))}
    tails = {r: random_tokens(rng, 40, cfg["vocab_size"]) for r in prompts}
    results = []
    for graphs in (False, True):
        eng = build(folder_b, "bfloat16", options={"cuda_graphs": graphs})
        steps = [{"entries": [(r, prompts[r], []) for r in prompts]}]
        steps += [{"entries": [(r, [tails[r][i]], [0]) for r in prompts]} for i in range(40)]
        results.append(replay(eng, steps))
        assert (eng.graph_replays > 30) == graphs
    eager, recorded = results
    assert eager.keys() == recorded.keys()
    for k in eager:
        assert np.array_equal(eager[k], recorded[k]), k
    both = {r: prompts[r] + tails[r] for r in prompts}
    for r, toks in both.items():
        ref = plain_logits(folder_b, toks)
        for p in range(len(prompts[r]), len(toks)):
            assert np.abs(recorded[(r, p)] - ref[p]).max() <= TOL["bfloat16"] * np.abs(ref).max()


LAYER_SIZES = {   # one block at the layer sizes of the large configurations, small vocabulary
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288),
    "14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=17408),
    "32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=25600),
}


@pytest.mark.parametrize("size", ["8b", "14b", "32b"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_one_block_at_large_layer_sizes(size, dtype, tmp_path_factory):
    """Logits of a one-layer model with the real layer sizes: whole prompt, then decoded tokens, then a
    second request beside it, against the plain implementation."""
    from conftest import make_folder
    cfg = dict(TINY["B"][0], num_hidden_layers=1, vocab_size=512, max_position_embeddings=512, **LAYER_SIZES[size])
    folder = make_folder(tmp_path_factory, cfg, 5, f"block_{size}")
    eng = build(folder, dtype, num_pages=32, page_size=16)
    rng = np.random.default_rng(1)
    a, b = random_tokens(rng, 90, 512), random_tokens(rng, 21, 512)
    steps = [{"entries": [("a", a[:70], list(range(70)))]},
             {"entries": [("a", a[70:71], [0]), ("b", b[:20], list(range(20)))]}]
    steps += [{"entries": [("a", a[71 + i:72 + i], [0])] + ([("b", b[20:], [0])] if i == 0 else [])} for i in range(19)]
    got = replay(eng, steps)
    check_against_plain(got, folder, {"a": a, "b": b}, dtype)


@pytest.fixture(scope="module")
def long_prompt_folder(tmp_path_factory):
    from conftest import make_folder
    cfg = dict(TINY["B"][0], num_hidden_layers=2, hidden_size=256, num_attention_heads=8, num_key_value_heads=2,
               head_dim=128, intermediate_size=384, vocab_size=512, max_position_embeddings=4096)
    return make_folder(tmp_path_factory, cfg, 9, "long_prompt")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions_then_decoding(dtype, long_prompt_folder):
    """3,000 tokens with heads of 128 (the tensor-memory attention kernel in bfloat16): portions of 1,024
    whose keys span dozens of tiles and hundreds of pages, logits at the portions' ends, then decoding
    beside the portion of another request."""
    from safetyraise_lmengine_b200 import Engine
    folder = long_prompt_folder
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, num_pages=220, max_requests=2,
                             max_batch_tokens=1100, max_context=4096)
    rng = np.random.default_rng(3)
    a, b = random_tokens(rng, 3000, 512), random_tokens(rng, 40, 512)
    steps, at = [], 0
    for n in (1024, 1024, 940):                      # the last 8 places of every portion
        steps.append({"entries": [("a", a[at:at + n], list(range(n - 8, n)))]})
        at += n
    steps.append({"entries": [("a", a[at:at + 1], [0]), ("b", b[:30], [28, 29])]})
    at += 1
    for i in range(10):
        steps.append({"entries": [("a", a[at + i:at + i + 1], [0]), ("b", b[30 + i:31 + i], [0])]})
    steps.append({"entries": [("a", a[at + 10:], [0])]})
    got = replay(eng, steps)
    assert len(got) == 3 * 8 + 1 + 2 + 20 + 1
    ref_a, ref_b = plain_logits(folder, a), plain_logits(folder, b)
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = (ref_a if rid == "a" else ref_b)[pos]
        worst = max(worst, np.abs(row - ref).max() / np.abs(ref).max())
    assert worst <= TOL[dtype], worst
    assert eng.cache.audit() == 0


@pytest.mark.parametrize("streaming_tokens", [0, 8])
def test_norms_fused_into_products_agree_with_the_separate_kernels(folder_b, streaming_tokens):
    """Decode steps of up to 8 tokens run their RMSNorms inside the products around them; the same
    steps with the fusion switched off must give the same logits within rounding.  Once on the
    tensor-core kernel (the default), once on the weight-streaming kernel that may stand in for it."""
    from safetyraise_lmengine_b200.kernels import ops
    cfg, _ = TINY["B"]
    rng = np.random.default_rng(13)
    reqs = {r: random_tokens(rng, n, cfg["vocab_size"]) for r, n in (("a", 30), ("b", 47), ("c", 12))}
    steps = [{"entries": [(r, t[:-8], []) for r, t in reqs.items()]}]
    steps += [{"entries": [(r, t[len(t) - 8 + i:len(t) - 7 + i], [0]) for r, t in reqs.items()]} for i in range(8)]
    steps[-1]["end"] = list(reqs)
    steps += [{"entries": [("d", reqs["a"][:5], [0, 4]), ("e", reqs["b"][:3], [2])]}]      # 8 prompt tokens
    out = {}
    keep, ops.skinny_max_tokens = ops.skinny_max_tokens, streaming_tokens
    try:
        for fused in (True, False):
            eng = build(folder_b, "bfloat16", options={"unfused_norms": not fused, "cuda_graphs": False})
            ops.begin_timing()
            out[fused] = replay(eng, steps)
            names = set(k.split("[")[0] for k in ops.end_timing())
            assert (("gemm_tn_skinny_fused" if streaming_tokens else "gemm_tn_tcgen05_fused") in names) == fused, names
            assert ("gemm_tn_skinny" in names or "gemm_tn_skinny_fused" in names) == bool(streaming_tokens), names
    finally:
        ops.skinny_max_tokens = keep
    assert out[True].keys() == out[False].keys() and len(out[True]) == 3 * 8 + 3
    for k in out[True]:
        scale = np.abs(out[False][k]).max()
        assert np.abs(out[True][k] - out[False][k]).max() <= 2e-2 * scale, k
    full = {r: t for r, t in reqs.items()}
    for r, t in full.items():
        ref = plain_logits(folder_b, t)
        for p in range(len(t) - 8, len(t)):
            assert np.abs(out[True][(r, p)] - ref[p]).max() <= TOL["bfloat16"] * np.abs(ref).max()


@pytest.mark.parametrize("name", ["B", "G"])
def test_norms_fused_into_products_of_up_to_128_tokens(name, tmp_path_factory):
    """Steps of 9 to 128 tokens run their RMSNorms inside the tensor-core products: decode batches of a
    dozen requests and short portions beside them, against the separate kernels and the plain logits."""
    from conftest import make_folder
    from safetyraise_lmengine_b200 import Engine
    from safetyraise_lmengine_b200.kernels import ops
    cfg, seed = TINY[name]
    folder = make_folder(tmp_path_factory, cfg, seed, "fused64_" + name.lower())
    rng = np.random.default_rng(23)
    reqs = {f"r{i}": random_tokens(rng, 35 + 3 * i, cfg["vocab_size"]) for i in range(12)}
    steps = [{"entries": [(r, t[:15], []) for r, t in reqs.items()]}]                      # 180 tokens: unfused
    steps += [{"entries": [(r, t[15:23], [7]) for r, t in reqs.items()]}]                  # 96 tokens: fused
    steps += [{"entries": [(r, t[23:27], [3]) for r, t in reqs.items()]}]                  # 48 tokens: fused
    steps += [{"entries": [(r, t[27 + i:28 + i], [0]) for r, t in reqs.items()]} for i in range(8)]   # 12 tokens
    out = {}
    for fused in (True, False):
        ops.fuse_norms_into_products = fused
        try:
            eng = Engine.from_folder(folder, dtype="bfloat16", page_size=16, num_pages=64, max_requests=12,
                                     max_batch_tokens=512, options={"cuda_graphs": False})
            ops.begin_timing()                       # (events between launches: not while a graph is recorded)
            out[fused] = replay(eng, steps)
            names = set(k.split("[")[0] for k in ops.end_timing())
        finally:
            ops.fuse_norms_into_products = True
        assert ("gemm_tn_tcgen05_fused" in names) == fused, names
    # the same steps with the decode steps replayed from CUDA graphs: the same bits
    eng = Engine.from_folder(folder, dtype="bfloat16", page_size=16, num_pages=64, max_requests=12,
                             max_batch_tokens=512)
    recorded = replay(eng, steps)
    assert eng.graph_replays >= 5
    for k in recorded:
        assert np.array_equal(recorded[k], out[True][k]), k
    assert out[True].keys() == out[False].keys() and len(out[True]) == 12 * 10
    for k in out[True]:
        scale = np.abs(out[False][k]).max()
        assert np.abs(out[True][k] - out[False][k]).max() <= 2e-2 * scale, k
    for r, t in reqs.items():
        ref = plain_logits(folder, t[:35])
        for p in [22, 26] + list(range(27, 35)):
            assert np.abs(out[True][(r, p)] - ref[p]).max() <= TOL["bfloat16"] * np.abs(ref).max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["F", "G"])
def test_schedules_drawn_at_random_agree_with_plain(name, dtype, tmp_path_factory):
    """Up to four live requests fed in portions and single tokens of random sizes, some sitting a step out,
    with as few pages as the four longest need: every asked place against the plain logits (fixed seeds)."""
    from conftest import make_folder
    from safetyraise_lmengine_b200 import Engine
    cfg, wseed = TINY[name]
    folder = make_folder(tmp_path_factory, cfg, wseed, "sched_" + name.lower())
    for trial in range(4):
        rng = np.random.default_rng(100 + trial)
        ps = int(rng.choice([4, 16]))
        maxlen = min(cfg["max_position_embeddings"], 140)
        reqs = {f"r{i}": random_tokens(rng, int(rng.integers(2, maxlen)), cfg["vocab_size"])
                for i in range(int(rng.integers(3, 9)))}
        pages = sorted(((len(t) + ps - 1) // ps for t in reqs.values()), reverse=True)
        num_pages = sum(pages[:4]) + 1
        eng = Engine.from_folder(folder, dtype=dtype, page_size=ps, num_pages=num_pages, max_requests=4,
                                 max_batch_tokens=512)
        waiting, live, fed, steps = list(reqs), [], {}, []
        while waiting or live:
            while waiting and len(live) < 4 and rng.random() < 0.7:
                live.append(waiting.pop(0))
                fed[live[-1]] = 0
            entries, ends = [], []
            for r in list(live):
                if rng.random() < 0.25 and len(live) > 1:
                    continue                                  # sits this step out
                left = len(reqs[r]) - fed[r]
                n = 1 if rng.random() < 0.5 else int(rng.integers(1, min(left, 40) + 1))
                want = sorted(set(int(x) for x in rng.integers(0, n, size=int(rng.integers(0, min(n, 3) + 1)))))
                entries.append((r, reqs[r][fed[r]:fed[r] + n], want))
                fed[r] += n
                if fed[r] == len(reqs[r]):
                    ends.append(r)
                    live.remove(r)
            if entries:
                steps.append({"entries": entries, "end": ends})
        got = replay(eng, steps)
        assert got
        for (r, pos), row in got.items():
            ref = plain_logits(folder, reqs[r])
            err = float(np.abs(row - ref[pos]).max() / np.abs(ref).max())
            note_error(dtype, err, f"random schedule {name}")
            assert err <= TOL[dtype], (trial, r, pos, err)
        assert eng.cache.audit() == 0 and eng.cache.free_pages() == num_pages
