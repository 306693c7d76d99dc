"""Generation through the Python entry point, the scheduler on a GPU, sampling kernels, the CLI and
bin/trace_run as a user runs it."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
from conftest import ROOT, TINY
from helpers import TOL, plain_logits, random_tokens

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_llm(folder, dtype, **kw):
    from safetyraise_lmengine_b200 import LLM
    opts = dict(dtype=dtype, page_size=4, num_pages=64, max_active=4, max_batch_tokens=64, prefill_chunk=8,
                max_context=128, queue_capacity=8)
    opts.update(kw)
    return LLM.from_folder(folder, **opts)


def check_greedy_path(folder, prompt, generated, dtype):
    """Every generated token must be the plain argmax of its position (float32), or within the
    bfloat16 tolerance of it."""
    toks = list(prompt) + list(generated)
    ref = plain_logits(folder, toks[:-1]) if len(toks) > 1 else None
    for i, tok in enumerate(generated):
        row = ref[len(prompt) - 1 + i]
        if dtype == "float32":
            assert tok == int(np.argmax(row)), (i, tok, int(np.argmax(row)))
        else:
            assert row[tok] >= row.max() - 2 * TOL[dtype] * np.abs(row).max(), (i, tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(tiny_folder, dtype):
    from safetyraise_lmengine_b200 import SamplingParams
    name, folder = tiny_folder
    cfg, _ = TINY[name]
    rng = np.random.default_rng(11)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (5, 11, 17)]
    llm = make_llm(folder, dtype)
    llm.eos = set()                                   # compare all 8 tokens
    res = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    for prompt, r in zip(prompts, res):
        assert r.finish_reason == "length" and len(r.tokens) == 8 and r.usage.completion_tokens == 8
        check_greedy_path(folder, prompt, r.tokens, dtype)
    if dtype == "float32":
        cfgd, w = P.read_model_folder(folder)
        assert res[0].tokens == P.greedy_generate(cfgd, w, prompts[0], 8)
    m = llm.metrics()
    assert m["completed"] == 3 and m["generated_tokens"] == 24 and m["active"] == 0
    assert llm.engine.cache.audit() == 0 and llm.engine.cache.free_pages() == 64


def test_planning_ahead_changes_no_token_and_no_count(folder_b):
    """The host half of the next decode step runs while the device works (the default); with a stop
    token among the samples, with seeds, with more requests than slots and with few pages the tokens,
    finish reasons and counters are those of the plain order of work."""
    from safetyraise_lmengine_b200 import SamplingParams
    from safetyraise_lmengine_b200.engine.scheduler import GenerationRequest
    rng = np.random.default_rng(5)
    prompts = [random_tokens(rng, n, 100) for n in (9, 14, 3, 21, 6, 12)]

    def run(ahead, stop, penalty=1.2, **kw):
        llm = make_llm(folder_b, "float32", plan_ahead=ahead, **kw)
        llm.eos = set(stop)
        ids = []
        for i, pr in enumerate(prompts):
            sp = SamplingParams(temperature=0.0 if i % 2 == 0 else 0.9, top_k=20, top_p=0.9, seed=100 + i,
                                repetition_penalty=1.0 if i % 3 else penalty, max_new_tokens=10 + i)
            ids.append(llm.submit(GenerationRequest(pr, sp)))
        seen = []
        llm.run_until_idle(lambda rid, tok, n: seen.append((rid, tok, n)))
        out = [llm.take_result(i) for i in ids]
        m = llm.metrics()
        assert llm.engine.cache.audit() == 0 and llm.engine.cache.free_pages() == llm.engine.cache.num_pages
        return [(r.tokens, r.finish_reason, r.usage.completion_tokens) for r in out], seen, \
            {k: m[k] for k in ("completed", "generated_tokens", "active", "queued")}, llm

    plain, seen0, m0, _ = run(False, ())
    ahead, seen1, m1, llm = run(True, ())
    assert ahead == plain and seen1 == seen0 and m1 == m0
    assert all(reason == "length" for _, reason, _ in plain)
    # a token that the second and the fourth request generate midway becomes the stop token
    stop = {plain[1][0][4], plain[3][0][7]}
    plain_s, seen0, m0, _ = run(False, stop)
    ahead_s, seen1, m1, _ = run(True, stop)
    assert ahead_s == plain_s and seen1 == seen0 and m1 == m0
    assert any(reason == "stop" for _, reason, _ in plain_s)
    # few pages: requests are preempted and recomputed while steps are laid out ahead
    plain_p, _, m0, _ = run(False, stop, num_pages=14)
    ahead_p, _, m1, llm = run(True, stop, num_pages=14)
    assert ahead_p == plain_p and m1 == m0
    assert [t for t, _, _ in plain_p] == [t for t, _, _ in plain_s]
    # (a repetition penalty needs the token before it on the host: steps with one are not queued ahead; the
    # runs above queue steps ahead only once the requests with a penalty have ended)
    # without penalties the next step is queued on the device before this step's tokens are read; a stop
    # token among them takes the queued step back; the tokens, their order and the counters stay the same
    for kw in ({"max_active": 6}, {}, {"num_pages": 14}):
        plain_q, seen0, m0, _ = run(False, (), penalty=1.0, **kw)
        stop = {plain_q[1][0][4], plain_q[3][0][7]}
        for stops in ((), stop):
            plain_q, seen0, m0, _ = run(False, stops, penalty=1.0, **kw)
            ahead_q, seen1, m1, llm = run(True, stops, penalty=1.0, **kw)
            off_q, seen2, m2, off = run(True, stops, penalty=1.0, launch_ahead=False, **kw)
            assert ahead_q == plain_q == off_q and m1 == m0 == m2, (kw, stops)
            if "num_pages" not in kw:      # (with preemptions the order in which tokens are published may differ)
                assert seen1 == seen0 == seen2, (kw, stops)
            assert llm.steps_ahead > 3 and off.steps_ahead == 0
            if not stops:
                assert llm.steps_dropped == 0
            elif "max_active" in kw:                   # all six decode together when the stop tokens come
                assert llm.steps_dropped > 0


def test_a_cancelled_request_takes_the_step_queued_ahead_back(folder_b):
    """While three requests decode, each turn queues the next step on the device before it reads the
    current one.  A request cancelled between two turns is part of the step in flight: that step is waited
    for and taken back (lengths, pages), the request ends, the others go on from where they were and
    produce the tokens they would have produced alone."""
    from safetyraise_lmengine_b200 import SamplingParams
    from safetyraise_lmengine_b200.engine.scheduler import GenerationRequest
    cfg, _ = TINY["B"]
    rng = np.random.default_rng(21)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (7, 12, 5)]
    llm = make_llm(folder_b, "float32")
    llm.eos = set()
    ids = [llm.submit(GenerationRequest(p, SamplingParams(temperature=0.0, max_new_tokens=14))) for p in prompts]
    while llm.steps_ahead < 3:
        assert llm.step()
    assert llm._inflight is not None and llm.steps_dropped == 0
    llm.cancel(ids[1])
    llm.run_until_idle()
    assert llm.steps_dropped == 1
    res = [llm.take_result(i) for i in ids]
    assert [r.finish_reason for r in res] == ["length", "cancelled", "length"]
    for p, r in zip(prompts, res):
        check_greedy_path(folder_b, p, r.tokens, "float32")
    assert len(res[0].tokens) == len(res[2].tokens) == 14 and 0 < len(res[1].tokens) < 14
    assert llm.engine.cache.audit() == 0 and llm.engine.cache.free_pages() == 64


def test_preemption_and_recompute_give_the_same_tokens(folder_b):
    from safetyraise_lmengine_b200 import SamplingParams
    cfg, _ = TINY["B"]
    rng = np.random.default_rng(12)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (40, 33, 64, 20)]
    sp = SamplingParams(temperature=0.8, top_p=0.9, top_k=50, seed=1234, max_new_tokens=6)
    roomy = make_llm(folder_b, "float32", page_size=16, num_pages=64)
    roomy.eos = set()
    want = [r.tokens for r in roomy.generate(prompts, sp)]
    assert roomy.metrics()["preempted"] == 0
    # 6 pages of 16 where the four requests need 3 + 3 + 5 + 2: the younger ones are thrown out and recomputed
    tight = make_llm(folder_b, "float32", page_size=16, num_pages=6)
    tight.eos = set()
    got = tight.generate(prompts, sp)
    assert [r.tokens for r in got] == want
    assert tight.metrics()["preempted"] > 0 and sum(r.usage.preemptions for r in got) > 0
    assert tight.engine.cache.audit() == 0 and tight.engine.cache.free_pages() == 6


def test_stop_token_cancel_deadline_and_queue(folder_b):
    from safetyraise_lmengine_b200 import SamplingParams
    from safetyraise_lmengine_b200.engine.scheduler import GenerationRequest
    from safetyraise_lmengine_b200.errors import ConfigError, ResourceExhausted
    cfg, _ = TINY["B"]
    llm = make_llm(folder_b, "float32", max_active=1, queue_capacity=2)
    prompt = random_tokens(np.random.default_rng(5), 9, cfg["vocab_size"])
    free = llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=12))[0].tokens
    # make the first token that differs from the ones before it an end-of-sequence id: it ends the
    # request and is not returned (a tiny random model may repeat itself, then the first token is it)
    k = next((i for i in range(1, len(free)) if free[i] not in free[:i]), 0)
    llm.eos = {free[k]}
    r = llm.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=12))[0]
    assert r.finish_reason == "stop" and r.tokens == free[:k] and r.usage.completion_tokens == k
    llm.eos = set()
    # cancelled between steps, mid-prefill; deadline passed while queued
    a = llm.submit(GenerationRequest(prompt * 6, SamplingParams(temperature=0.0, max_new_tokens=4)))
    b = llm.submit(GenerationRequest(prompt, SamplingParams(temperature=0.0, max_new_tokens=4), deadline_ms=1))
    with pytest.raises(ResourceExhausted):
        llm.submit(GenerationRequest(prompt, SamplingParams(max_new_tokens=4))), llm.submit(GenerationRequest(prompt, SamplingParams(max_new_tokens=4)))
    llm.step()
    llm.cancel(a)
    import time
    time.sleep(0.01)
    llm.run_until_idle()
    ra, rb = llm.take_result(a), llm.take_result(b)
    assert ra.finish_reason == "cancelled" and rb.finish_reason == "deadline" and rb.tokens == []
    llm.run_until_idle()
    for bad in (GenerationRequest([]), GenerationRequest([cfg["vocab_size"]]),
                GenerationRequest(prompt, SamplingParams(top_p=0.0)),
                GenerationRequest(prompt, SamplingParams(max_new_tokens=1000))):
        with pytest.raises(ConfigError):
            llm.submit(bad)
    while llm._live:
        llm.run_until_idle()
    assert llm.engine.cache.audit() == 0 and llm.engine.cache.free_pages() == 64


def consistent_with_plain(token, logits, history, temperature, top_k, top_p, penalty, u) -> bool:
    adj = P.apply_repetition_penalty(logits, history, penalty)
    if temperature == 0:
        return token == int(np.argmax(adj))
    ids, wts, kept = P.sample_distribution(adj, temperature, top_k, top_p)
    if token == P.sample(logits, history, temperature, top_k, top_p, penalty, u):
        return True
    where = np.nonzero(ids == token)[0]          # allowed only when the draw sits on a boundary
    if where.size == 0:
        return False
    cum = np.cumsum(wts.astype(np.float64))
    lo = cum[where[0]] - wts[where[0]]
    return lo - 1e-5 <= u * kept <= cum[where[0]] + 1e-5


@pytest.mark.parametrize("V", [5, 384, 151936])
def test_sampling_kernel_follows_the_plain_sampler(V):
    from safetyraise_lmengine_b200.sampling.params import SamplingParams
    from safetyraise_lmengine_b200.sampling.sampler import Sampler, uniform_for
    rng = np.random.default_rng(V)
    n = 24
    logits = (rng.normal(0, 2.5, size=(n, V))).astype(np.float32)
    logits[3, :] = 1.0                                 # all equal: ties by id everywhere
    logits[4, : min(V, 7)] = 9.0                       # a tie at the top
    params, seeds, idx, hist = [], [], [], []
    for i in range(n):
        params.append(SamplingParams(temperature=[0.0, 0.8, 1.0, 1.7][i % 4], top_p=[1.0, 0.95, 0.5, 0.05][(i // 4) % 4],
                                     top_k=[0, 1, 3, 50][(i // 2) % 4] if V > 50 else [0, 1, 3, 4][(i // 2) % 4],
                                     repetition_penalty=[1.0, 1.3, 0.7][i % 3]))
        seeds.append(1000 + i)
        idx.append(i % 5)
        hist.append([int(t) for t in rng.integers(0, V, size=10)] + [int(np.argmax(logits[i]))])
    s = Sampler(DEV, V, n)
    got = s.sample(torch.tensor(logits, device=DEV), params, seeds, idx, hist)
    assert s.bad.item() == 0
    for i in range(n):
        p = params[i]
        u = uniform_for(seeds[i], idx[i])
        assert 0.0 <= u < 1.0
        assert consistent_with_plain(got[i], logits[i], hist[i], p.temperature, p.top_k, p.top_p,
                                     p.repetition_penalty, u), (i, got[i], vars(p))
    again = s.sample(torch.tensor(logits, device=DEV), params, seeds, idx, hist)
    assert again == got                               # same seed and index: same tokens


def test_a_penalty_counts_the_token_that_is_still_on_the_device():
    """The last id of a row's history may be the token that the launch before this one sampled and that the
    host has not read yet: the sampler puts it in place on the device (``pending``)."""
    from safetyraise_lmengine_b200.sampling.sampler import Sampler
    V, n = 700, 4
    g = torch.Generator(device="cuda").manual_seed(4)
    rng = np.random.default_rng(8)
    last = [int(t) for t in rng.integers(0, V, size=n)]               # what the launch before "sampled"
    first = torch.full((n, V), -5.0, device="cuda")
    for i, t in enumerate(last):
        first[i, t] = 9.0
    logits = torch.randn(n, V, device="cuda", generator=g) * 3
    for i, t in enumerate(last):
        logits[i, t] = logits[i].max() + 0.5                          # the penalty on that id decides the row
    hist = [[int(t) for t in rng.integers(0, V, size=k)] for k in (5, 0, 17, 3)]
    params = [SamplingParamsOf(1.5, 0.0), SamplingParamsOf(1.3, 0.8), SamplingParamsOf(1.0, 0.7), SamplingParamsOf(2.0, 0.0)]
    seeds, idx = [11, 12, 13, 14], [3, 4, 5, 6]
    whole = Sampler("cuda", V, n).sample(logits, params, seeds, idx, [h + [t] for h, t in zip(hist, last)])
    s = Sampler("cuda", V, n)
    s.launch(first, [SamplingParamsOf(1.0, 0.0)] * n, seeds, idx, [[]] * n)          # leaves `last` in the rows
    got = s.collect(s.launch(logits, params, seeds, idx, hist, pending=[0, 1, 2, 3]))
    assert got == whole
    without = Sampler("cuda", V, n).sample(logits, params, seeds, idx, hist)
    assert without[0] == last[0] != whole[0] and without[3] == last[3] != whole[3]   # it was the penalty's doing
    # a row that waits for no token keeps its history as given
    got = s.collect(s.launch(logits, params, seeds, idx, [h + [t] for h, t in zip(hist, last)], pending=[None] * n))
    assert got == whole


def SamplingParamsOf(penalty, temperature):
    from safetyraise_lmengine_b200 import SamplingParams
    return SamplingParams(temperature=temperature, repetition_penalty=penalty, top_k=0, top_p=1.0, max_new_tokens=4)


@pytest.mark.parametrize("V, n", [(151936, 2), (40000, 30), (9000, 5), (8196, 70), (33000, 148)])
def test_sampling_rows_shared_by_clusters_of_blocks(V, n):
    """Long rows are shared by a cluster of 8, 4, 2 or 1 blocks, depending on their length and number:
    every choice gives the plain sampler's token, and the argmax kernel the plain argmax."""
    from safetyraise_lmengine_b200.kernels import ops
    from safetyraise_lmengine_b200.sampling.params import SamplingParams
    from safetyraise_lmengine_b200.sampling.sampler import Sampler, uniform_for
    rng = np.random.default_rng(V + n)
    rows = min(n, 12)                                   # rows checked against the plain sampler
    logits = (rng.normal(0, 3.0, size=(n, V))).astype(np.float32)
    logits[0, V - 3:] = 25.0                            # a tie at the top in the last block's slice
    logits[1 % n, ::2] = logits[1 % n, 1::2][: (V + 1) // 2]   # many exact pairs of equal values
    params, seeds, idx, hist = [], [], [], []
    for i in range(n):
        params.append(SamplingParams(temperature=[0.7, 1.0, 1.3][i % 3], top_p=[1.0, 0.9, 0.3][(i // 3) % 3],
                                     top_k=[0, 2, 40, 3000][i % 4], repetition_penalty=[1.0, 1.2][i % 2]))
        seeds.append(7 + i)
        idx.append(i % 3)
        hist.append([int(t) for t in rng.integers(0, V, size=20)] + [int(np.argmax(logits[i]))])
    dev_logits = torch.tensor(logits, device=DEV)
    s = Sampler(DEV, V, n)
    got = s.sample(dev_logits, params, seeds, idx, hist)
    assert s.bad.item() == 0 and len(got) == n
    for i in range(rows):
        p = params[i]
        assert consistent_with_plain(got[i], logits[i], hist[i], p.temperature, p.top_k, p.top_p,
                                     p.repetition_penalty, uniform_for(seeds[i], idx[i])), (i, got[i], vars(p))
    assert s.sample(dev_logits, params, seeds, idx, hist) == got
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.argmax(dev_logits, out, s.bad)
    assert out.tolist() == [int(np.argmax(r)) for r in logits]


def test_sampling_statistics():
    """Frequencies over many draws follow the truncated distribution."""
    from safetyraise_lmengine_b200.sampling.params import SamplingParams
    from safetyraise_lmengine_b200.sampling.sampler import Sampler
    V, n = 16, 4000
    base = np.linspace(2.0, -2.0, V).astype(np.float32)
    s = Sampler(DEV, V, n)
    sp = SamplingParams(temperature=1.0, top_p=0.9, top_k=8)
    got = s.sample(torch.tensor(np.tile(base, (n, 1)), device=DEV), [sp] * n, list(range(n)), [0] * n, [[]] * n)
    ids, wts, kept = P.sample_distribution(base, 1.0, 8, 0.9)
    freq = np.bincount(got, minlength=V) / n
    assert set(np.nonzero(freq)[0]) <= set(int(i) for i in ids)
    for i, w in zip(ids, wts):
        assert abs(freq[i] - w / kept) < 0.03


def run_cli(*args, stdin=None):
    env = dict(os.environ, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, "-m", "safetyraise_lmengine_b200", *args], input=stdin, env=env,
                          capture_output=True, text=True, timeout=600)


def test_cli_inspect_run_benchmark(folder_a, tmp_path):
    cfg = tmp_path / "svc.json"
    cfg.write_text(json.dumps({"model_path": folder_a, "model_name": "tiny-a",
                               "engine": {"max_context": 128, "max_active": 2, "prefill_chunk": 4,
                                          "page_size": 4, "num_pages": 40, "dtype": "float32",
                                          "max_batch_tokens": 32}}))
    req = tmp_path / "req.json"
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    req.write_text(json.dumps({"prompt_ids": prompt, "max_tokens": 5, "temperature": 0.0}))
    out = run_cli("inspect", "--model-path", folder_a, "--context", "64")
    assert out.returncode == 0, out.stderr
    info = json.loads(out.stdout)
    assert info["tensors"] == 24 and info["context"] == 64 and info["state_bytes_per_request"] == 2 * 2 * 2 * 16 * 2 * 64
    out = run_cli("run", "--config", str(cfg), "--request", str(req))
    assert out.returncode == 0, out.stderr
    res = json.loads(out.stdout)
    cfgd, w = P.read_model_folder(folder_a)
    assert res["tokens"] == P.greedy_generate(cfgd, w, prompt, 5) and res["finish_reason"] == "length"
    assert res["usage"]["prompt_tokens"] == 8 and res["usage"]["completion_tokens"] == 5
    out = run_cli("benchmark", "--config", str(cfg), "--request", str(req), "--iterations", "2")
    assert out.returncode == 0, out.stderr
    b = json.loads(out.stdout)
    assert len(b["runs"]) == 2 and b["runs"][0]["completion_tokens"] == 5
    groups = info["cache_groups"]
    assert len(groups) == 1 and groups[0]["kind"] == "paged_all" and groups[0]["entries"] == 2
    # the random-weights mode: config.json alone; the tensors are functions of (seed, name), so a folder
    # written from the same seed holds the same model
    from safetyraise_lmengine_b200.weights.random_init import write_model_folder
    cj = tmp_path / "model_config.json"
    cj.write_text(json.dumps(TINY["B"][0]))
    out = run_cli("inspect", "--random-weights", "77", "--config-json", str(cj), "--context", "32", "--dtype", "float32")
    assert out.returncode == 0, out.stderr
    assert json.loads(out.stdout)["tensors"] == 3 * 11 + 3
    eng_only = tmp_path / "engine_only.json"
    eng_only.write_text(json.dumps({"engine": {"max_context": 128, "max_active": 2, "page_size": 4, "num_pages": 40,
                                               "dtype": "float32", "max_batch_tokens": 32}}))
    out = run_cli("run", "--random-weights", "77", "--config-json", str(cj), "--config", str(eng_only),
                  "--request", str(req))
    assert out.returncode == 0, out.stderr
    cfgd, w = P.read_model_folder(write_model_folder(TINY["B"][0], 77, str(tmp_path / "same_seed")))
    assert json.loads(out.stdout)["tokens"] == P.greedy_generate(cfgd, w, prompt, 5)
    out = run_cli("run", "--random-weights", "77", "--request", str(req))
    assert out.returncode == 2 and "go together" in out.stderr
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"model_path": folder_a, "engine": {"no_such_option": 1}}))
    out = run_cli("run", "--config", str(bad), "--request", str(req))
    assert out.returncode == 2 and "no_such_option" in out.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folder_b, tmp_path, dtype):
    """bin/trace_run as a separate process: portions, decoded tokens beside them, ends, page reuse."""
    cfg, _ = TINY["B"]
    rng = np.random.default_rng(21)
    a, b, c = (random_tokens(rng, n, cfg["vocab_size"]) for n in (50, 40, 45))
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": [1]},
                                {"id": "b", "tokens": b[:38], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[38:39], "want": [0]}], "end": []},   # a is left out
        {"step": 3, "entries": [{"id": "a", "tokens": a[32:], "want": [17]},
                                {"id": "b", "tokens": b[39:], "want": [0]}], "end": ["a", "b"]},
        {"step": 4, "entries": [{"id": "c", "tokens": c, "want": list(range(45))}], "end": ["c"]},
    ]
    out_dir = tmp_path / "out"
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder_b, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "4"]
    V = cfg["vocab_size"]
    read = lambda i: np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, V)
    ra, rb, rc = plain_logits(folder_b, a), plain_logits(folder_b, b), plain_logits(folder_b, c)
    checks = [(read(0), ra[[0, 29]]), (read(1), ra[[31]]), (read(2), rb[[38]]),
              (read(3), np.stack([ra[49], rb[39]])), (read(4), rc)]
    for got, ref in checks:
        assert got.shape == ref.shape
        assert np.abs(got - ref).max() <= TOL[dtype] * np.abs(ref).max()
