"""Decode and prefill throughput of the engine at Qwen3 layer sizes, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 8b|14b|32b] [--workload decode|mixed]

A "step" is one decode step: every request of the batch gets its next token.
The default run has the sizes of the 8B configuration (36 layers, hidden 4096,
32/8 heads of 128, intermediate 12288, vocabulary 151936), random weights in
bfloat16, a batch of 8 and 2,048 tokens of context per request.  It prints one
JSON line:

* ``value``: decoded tokens a second of whole steps run back to back through the
  step function (host half -- checks, page reservation, batch layout -- and
  device half -- one upload, the forward), timed on the device with CUDA events
  around blocks of exactly ``--steps`` steps; the block is repeated until at
  least two seconds are timed and the median block is reported.
  ``device_half_ms`` is the device half alone (the host half done before the
  first event), ``eager_ms`` the same step launched kernel by kernel instead of
  replayed from its CUDA graph.
* ``e2e``: the same through the Python entry point (``LLM.step``), by the wall
  clock, host token ids in and sampled token ids out every step.
* ``prefill``: a 2,048-token prompt (median of runs back to back: the GPU is at
  its power cap by then); ``roofline``: the decode step's bytes over its time
  against the measured copy bandwidth; ``points``: decode at batch 1 and 64,
  device-timed and end to end; ``kernels``: a table of where an eager decode
  step's and a prefill's time goes, kernel by kernel.

``--shape 32b`` runs the 32B configuration's workload (decode at batch 1 and 64
with 4,096 tokens of context, one 2,048-token prefill), ``--shape 14b`` (whose
default workload is ``mixed``) 32 requests with prompts of 128 to 3,072 tokens
prefilled in portions of up to 512 tokens beside the decoding ones, through the
scheduler.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASE = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "head_dim": 128, "num_key_value_heads": 8,
        "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
        "max_position_embeddings": 8192}   # room for the tokens decoded on top of a 4,096-token context
SHAPES = {      # layer sizes of the benchmark configurations; context = tokens each request holds while decoding
    "8b": dict(BASE, num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, intermediate_size=12288),
    "14b": dict(BASE, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408),
    "32b": dict(BASE, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600),
}
CONTEXT = {"8b": 2048, "14b": 2048, "32b": 4096}
BATCH = {"8b": 8, "14b": 8, "32b": 64}
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
MIN_TIMED_SECONDS = 2.0
MAX_GROWTH = 640          # tokens a request's context may grow by over all timed blocks of one measurement


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    if os.path.isfile(path):
        try:
            with open(path) as f:
                got = json.load(f)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(got.get(k), (int, float)) and got[k] > 0:
                    out[k] = float(got[k])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(int(r[0]) for r in self.rows)),
                "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons, "samples": len(self.rows)}


def reference_arm():
    # The reference is a Rust crate; this machine has no cargo/rustc and no network, and pip cannot
    # install a crate.  Its only CUDA code (one naive linear kernel) was never wired to a model run.
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Rust crate (no Python package to pip-install; no cargo/rustc here)"}))
    return 0


def build_engine(config: dict, layers: int, max_requests: int, tokens_in_cache: int, max_batch_tokens: int,
                 graphs=True):
    import torch
    from safetyraise_lmengine_b200 import Engine, spec_from_config
    from safetyraise_lmengine_b200.parts.model import tensor_decls
    from safetyraise_lmengine_b200.weights.random_init import RandomWeights
    cfg = dict(config, num_hidden_layers=layers)
    spec = spec_from_config(cfg)
    src = RandomWeights(tensor_decls(spec), seed=0, device="cuda:0")
    num_pages = (tokens_in_cache + PAGE_SIZE - 1) // PAGE_SIZE + max_requests
    eng = Engine.from_source(cfg, src, dtype="bfloat16", page_size=PAGE_SIZE, num_pages=num_pages,
                             max_requests=max_requests, max_batch_tokens=max_batch_tokens, max_context=8192,
                             options={"cuda_graphs": graphs})
    torch.cuda.synchronize()
    return eng


def randomize_cache(eng):
    """Random cache contents, N(0, 1).  The work does not depend on the values, the power does: at its power cap
    the GPU runs a 32B decode step of batch 64 in 23.4 ms over such contents and in 22.2 ms over zeros."""
    for pool in eng.cache.kv_pools.values():
        flat = pool.view(-1)
        step = 1 << 26
        for lo in range(0, flat.numel(), step):
            flat[lo:lo + step].normal_(0.0, 1.0)


def fill_contexts(eng, batch: int, context: int):
    """Opens `batch` requests that each hold `context` tokens; the page accounting is the real one."""
    import torch
    slots = []
    for _ in range(batch):
        s = eng.open_request()
        assert eng.cache.reserve(s, context)
        eng.cache.commit(s, context)
        slots.append(s)
    torch.cuda.synchronize()
    return slots


def blocks_for(steps: int, warmup: int, ms_per_step: float, min_seconds: float) -> int:
    """How many blocks of `steps` steps: enough for `min_seconds`, within the growth a context is allowed."""
    want = math.ceil(min_seconds * 1000.0 / max(ms_per_step * steps, 1e-3))
    return max(1, min(want, (MAX_GROWTH - warmup - 8) // max(steps, 1)))


def time_decode(eng, slots, context: int, steps: int, warmup: int, min_seconds: float):
    """Whole decode steps back to back through the step function, CUDA events around blocks of exactly
    `steps` steps.  Returns a dict: ms_per_step (median block), device_half_ms (median step, host half
    outside the events), blocks, mean_context (of the timed steps), launches (of one block)."""
    import torch
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.kernels import ops
    gen = torch.Generator().manual_seed(0)
    vocab = eng.spec.vocab_size
    def entries():
        toks = torch.randint(0, vocab, (len(slots),), generator=gen).tolist()
        return [StepEntry(s, [t], [0]) for s, t in zip(slots, toks)]
    for _ in range(warmup):
        eng.run(eng.prepare(entries()))
    torch.cuda.synchronize()
    # the device half alone: host half before the first event
    half = []
    for _ in range(min(steps, 20)):
        prep = eng.prepare(entries())
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.run(prep)
        b.record()
        torch.cuda.synchronize()
        half.append(a.elapsed_time(b))
    for s in slots:
        eng.cache.truncate(s, context + warmup)
    nblocks = blocks_for(steps, warmup, statistics.median(half), min_seconds)
    block_ms, launches = [], 0
    for _ in range(nblocks):
        batches = [entries() for _ in range(steps)]
        before = ops.launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for e in batches:
            eng.run(eng.prepare(e))             # host half and device half of every step inside the events
        b.record()
        torch.cuda.synchronize()
        block_ms.append(a.elapsed_time(b))
        launches = ops.launches - before
    grown = warmup + nblocks * steps
    for s in slots:
        eng.cache.truncate(s, context)
    return {"ms_per_step": statistics.median(block_ms) / steps, "device_half_ms": statistics.median(half),
            "blocks": nblocks, "mean_context": context + warmup + (grown - warmup) // 2, "launches": launches,
            "timed_seconds": sum(block_ms) / 1000.0}


def decode_bytes(eng, batch: int, context: int) -> int:
    """Bytes a decode step has to read: every weight it uses once (the embedding table is only
    gathered) and the cache of the live requests."""
    spec = eng.spec
    total = eng.model.weight_bytes()
    if not spec.tie_word_embeddings:
        total -= spec.vocab_size * spec.hidden_size * 2      # embedding table: `batch` rows only
    total += batch * spec.hidden_size * 2
    total += batch * context * eng.cache.bytes_per_page() // eng.cache.page_size
    return total


def linear_flops_per_token(spec) -> float:
    total = 0.0
    for step in spec.run_order:
        layer = spec.layers[step.layer]
        m, ff, H = layer.mixer, layer.feed_forward, spec.hidden_size
        total += 2 * ((m.heads + 2 * m.kv_heads) * m.head_dim * H + m.heads * m.head_dim * H
                      + 3 * H * ff.intermediate_size)
    return total


def attention_flops(spec, q_len: int, start: int) -> float:
    """QK^T and PV of q_len queries that follow `start` cached tokens (causal)."""
    total = 0.0
    keys = q_len * start + q_len * (q_len + 1) / 2.0
    for step in spec.run_order:
        m = spec.layers[step.layer].mixer
        total += 2 * 2 * keys * m.heads * m.head_dim
    return total


def prefill_flops(spec, tokens: int) -> float:
    return tokens * linear_flops_per_token(spec) + attention_flops(spec, tokens, 0) \
        + 2 * spec.vocab_size * spec.hidden_size


def time_prefill(eng, tokens: int, repeats: int):
    import torch
    from safetyraise_lmengine_b200 import StepEntry
    gen = torch.Generator().manual_seed(1)
    times = []
    for i in range(repeats + 3):
        toks = torch.randint(0, eng.spec.vocab_size, (tokens,), generator=gen).tolist()
        s = eng.open_request()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([StepEntry(s, toks, [tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        eng.close_request(s)
        if i >= 3:                     # three runs warm up
            times.append(a.elapsed_time(b))
    return statistics.median(times)    # after the warm-ups the GPU sits at its power cap (sustained clocks)


def time_e2e(eng, batch: int, context: int, steps: int, warmup: int, ms_hint: float, min_seconds: float):
    """Decode through the Python entry point: requests are submitted as token ids, prefilled by the
    scheduler, and each timed step copies its token ids and batch layout from pinned host memory
    and reads the sampled tokens back to the host.  Blocks of `steps` steps by the wall clock with a
    synchronize on both sides; the median block."""
    import torch
    from safetyraise_lmengine_b200 import LLM, EngineConfig, SamplingParams
    from safetyraise_lmengine_b200.engine.scheduler import GenerationRequest
    cfg = EngineConfig(max_context=8192, max_active=batch, queue_capacity=batch, prefill_chunk=2048,
                       max_batch_tokens=eng.mctx.max_batch_tokens, page_size=PAGE_SIZE)
    llm = LLM(eng, cfg)
    llm.eos = set()
    nblocks = blocks_for(steps, warmup, ms_hint, min_seconds)
    gen = torch.Generator().manual_seed(2)
    for _ in range(batch):
        prompt = torch.randint(0, eng.spec.vocab_size, (context,), generator=gen).tolist()
        llm.submit(GenerationRequest(prompt, SamplingParams(temperature=0.0,
                                                            max_new_tokens=warmup + nblocks * steps + 8)))
    decoding = lambda: all(len(st.tokens) > st.usage.prompt_tokens for st in llm._live.values())
    while not decoding():
        llm.step()
    for _ in range(warmup):
        llm.step()
    seconds = []
    with ClockSampler() as clocks:
        for _ in range(nblocks):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                llm.step()
            torch.cuda.synchronize()
            seconds.append(time.perf_counter() - t0)
    time_e2e.clocks = clocks.summary()       # (of the last call: under a power cap the two arms may see other clocks)
    h2d = eng.last_h2d_bytes
    d2h = (8 + batch) * 4                                # the fault words and one token id per request
    for rid in list(llm._live):
        llm.cancel(rid)
    llm.step()
    assert eng.steps_failed == 0
    return batch * steps / statistics.median(seconds), h2d, d2h, nblocks


def kernel_table(eng, slots, context: int, top: int = 8):
    """Where the time of one eager decode step goes, kernel by kernel (events between the launches)."""
    import torch
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.kernels import ops
    graphs, eng.use_graphs = eng.use_graphs, False
    try:
        for i in range(3):
            if i == 2:
                ops.begin_timing()
            eng.run(eng.prepare([StepEntry(s, [1 + i], [0]) for s in slots]))
        table = ops.end_timing()
    finally:
        eng.use_graphs = graphs
        for s in slots:
            eng.cache.truncate(s, context)
    total = sum(ms for _, ms in table.values()) or 1.0
    rows = sorted(table.items(), key=lambda kv: -kv[1][1])[:top]
    return {name: {"launches": n, "ms": round(ms, 3), "share": round(ms / total, 3)} for name, (n, ms) in rows}


def prefill_kernel_table(eng, tokens: int, top: int = 8):
    import torch
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.kernels import ops
    s = eng.open_request()
    ops.begin_timing()
    eng.step([StepEntry(s, [7] * tokens, [tokens - 1])])
    table = ops.end_timing()
    eng.close_request(s)
    total = sum(ms for _, ms in table.values()) or 1.0
    rows = sorted(table.items(), key=lambda kv: -kv[1][1])[:top]
    return {name: {"launches": n, "ms": round(ms, 3), "share": round(ms / total, 3)} for name, (n, ms) in rows}


def config_record(shape: str, cfg: dict, layers: int, batch: int, context: int, workload: str) -> dict:
    return {"model": f"Qwen3-{shape.upper()} layer sizes", "layers": layers, "layers_of_config": cfg["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": batch, "seq_len": context, "benchmark_context": 4096, "page_size": PAGE_SIZE,
            "workload": workload, "parallelism": "single GPU",
            "l2": "not flushed: each step reads far more weight bytes than the 126 MB L2 holds"}


def run_decode(args, shape: str, pk) -> dict:
    import torch
    cfg = SHAPES[shape]
    B = args.batch or BATCH[shape]
    context = CONTEXT[shape]
    point_batches = [b for b in ((1, 64) if shape != "32b" else (1,)) if b != B]
    big = max([B] + point_batches)
    eng = build_engine(cfg, args.layers or cfg["num_hidden_layers"], max_requests=big,
                       tokens_in_cache=big * (context + MAX_GROWTH + 16) + PREFILL_TOKENS,
                       max_batch_tokens=PREFILL_TOKENS, graphs=not args.no_graphs)
    if args.only_prefill:
        return {"prefill_ms": time_prefill(eng, PREFILL_TOKENS, 5), "tokens": PREFILL_TOKENS}
    randomize_cache(eng)
    slots = fill_contexts(eng, B, context)
    with ClockSampler() as clocks:
        d = time_decode(eng, slots, context, args.steps, args.warmup, args.min_seconds)
    ms = d["ms_per_step"]
    nbytes = decode_bytes(eng, B, d["mean_context"])
    achieved = nbytes / (ms / 1000.0) / 1e9
    layers = len(eng.spec.run_order)
    out = {
        "metric": "decode_tokens_per_second", "value": round(B / (ms / 1000.0), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, random cache contents",
        "impl": "ours",
        "config": config_record(shape, cfg, layers, B, context, "decode"),
        "clocks": clocks.summary(),
        "gpu_launches": d["launches"],
        "timing": {"what": "median block of --steps whole steps (host and device half), CUDA events",
                   "blocks": d["blocks"], "timed_seconds": round(d["timed_seconds"], 2),
                   "device_half_ms": round(d["device_half_ms"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes,
                     "peak_source": pk["source"]},
    }
    if args.skip_extras:
        return out
    # the same step launched kernel by kernel (no CUDA graph), and where its time goes
    graphs, eng.use_graphs = eng.use_graphs, False
    eager = time_decode(eng, slots, context, min(args.steps, 20), 3, 0.0)
    eng.use_graphs = graphs
    out["timing"]["eager_ms"] = round(eager["ms_per_step"], 4)
    out["kernels"] = {"decode_step_eager": kernel_table(eng, slots, context)}
    for s in slots:
        eng.close_request(s)
    points = {}
    for b in point_batches:
        sl = fill_contexts(eng, b, context)
        p = time_decode(eng, sl, context, max(5, args.steps // 2), 3, 1.0)
        points[f"decode_b{b}"] = round(b / (p["ms_per_step"] / 1000.0), 1)
        frac = decode_bytes(eng, b, p["mean_context"]) / (p["ms_per_step"] / 1000.0) / 1e9 / pk["hbm_gbs"]
        points[f"decode_b{b}_hbm_frac"] = round(frac, 4)
        for s in sl:
            eng.close_request(s)
    pf_ms = time_prefill(eng, PREFILL_TOKENS, 5)
    flops = prefill_flops(eng.spec, PREFILL_TOKENS)
    out["prefill"] = {"value": round(PREFILL_TOKENS / (pf_ms / 1000.0), 1), "tokens": PREFILL_TOKENS,
                      "ms": round(pf_ms, 3),
                      "frac": round(flops / (pf_ms / 1000.0) / (pk["bf16_tflops"] * 1e12), 4),
                      "frac_of_sustained": round(flops / (pf_ms / 1000.0) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                      "tflops": round(flops / (pf_ms / 1000.0) / 1e12, 1),
                      "regime": "sustained: median of 5 runs after 3 warm-ups, back to back"}
    out["kernels"]["prefill"] = prefill_kernel_table(eng, PREFILL_TOKENS)
    e2e, h2d, d2h, nb = time_e2e(eng, B, context, args.steps, args.warmup, ms, args.min_seconds)
    e2e_bytes = decode_bytes(eng, B, context + args.warmup + nb * args.steps // 2)
    out["e2e"] = {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                  "blocks": nb, "hbm_frac": round(e2e_bytes * e2e / B / 1e9 / pk["hbm_gbs"], 4),
                  "sm_mhz": time_e2e.clocks.get("sm_mhz"), "reasons": time_e2e.clocks.get("reasons")}
    for b in point_batches:
        v, _, _, nbp = time_e2e(eng, b, context, max(5, args.steps // 2), 3, 1000.0 * b / points[f"decode_b{b}"], 1.0)
        points[f"e2e_b{b}"] = round(v, 1)
    out["points"] = points
    return out


def run_mixed(args, shape: str, pk) -> dict:
    """32 requests, prompt lengths uniform in [128, 3072] from a seed, prefilled in portions of up to 512
    tokens beside the decoding requests, through the scheduler; every request generates --new-tokens."""
    import random

    import torch
    from safetyraise_lmengine_b200 import LLM, EngineConfig, SamplingParams
    from safetyraise_lmengine_b200.engine.scheduler import GenerationRequest
    cfg = SHAPES[shape]
    n_req, chunk, new = 32, 512, args.new_tokens
    rng = random.Random(0)
    lens = [rng.randint(128, 3072) for _ in range(n_req)]
    eng = build_engine(cfg, args.layers or cfg["num_hidden_layers"], max_requests=n_req,
                       tokens_in_cache=sum(lens) + n_req * (new + PAGE_SIZE), max_batch_tokens=chunk,
                       graphs=not args.no_graphs)
    spec = eng.spec
    ecfg = EngineConfig(max_context=4096, max_active=n_req, queue_capacity=n_req, prefill_chunk=chunk,
                        max_batch_tokens=chunk, page_size=PAGE_SIZE)
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, spec.vocab_size, (n,), generator=gen).tolist() for n in lens]

    def one_pass(timed: bool):
        llm = LLM(eng, ecfg)
        llm.eos = set()
        for p in prompts:
            llm.submit(GenerationRequest(p, SamplingParams(temperature=0.0, max_new_tokens=new)))
        steps = []
        torch.cuda.synchronize()
        t_all = time.perf_counter()
        while True:
            t0 = time.perf_counter()
            llm.last_step = None
            if not llm.step():
                break
            torch.cuda.synchronize()
            if llm.last_step is not None:
                steps.append((time.perf_counter() - t0, llm.last_step))
        return time.perf_counter() - t_all, steps, llm.metrics()

    from safetyraise_lmengine_b200.kernels import ops
    one_pass(False)                                   # warm-up: graphs recorded, buffers sized
    launches_before = ops.launches
    with ClockSampler() as clocks:
        seconds, steps, metrics = one_pass(True)
    launches = ops.launches - launches_before         # (a replayed graph counts the launches it holds)
    per_token = linear_flops_per_token(spec)
    weight_bytes = eng.model.weight_bytes() - spec.vocab_size * spec.hidden_size * 2
    kv_bytes_per_token = eng.cache.bytes_per_page() // eng.cache.page_size
    kinds = {"decode": [0.0, 0, 0.0], "portion": [0.0, 0, 0.0]}       # seconds, steps, work (bytes or flops)
    for sec, st in steps:
        counts, starts = st["counts"], st["starts"]
        if max(counts) == 1:
            k = kinds["decode"]
            k[2] += weight_bytes + sum(s + 1 for s in starts) * kv_bytes_per_token
        else:
            k = kinds["portion"]
            k[2] += sum(counts) * per_token + sum(attention_flops(spec, c, s) for c, s in zip(counts, starts)) \
                + 2.0 * len(counts) * spec.vocab_size * spec.hidden_size      # at most one logits row an entry
        k[0] += sec
        k[1] += 1
    total_tokens = sum(lens) + n_req * new
    dec, por = kinds["decode"], kinds["portion"]
    return {
        "metric": "mixed_tokens_per_second", "value": round(total_tokens / seconds, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": len(steps), "warmup": 1, "ms_per_step": round(1000.0 * seconds / len(steps), 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), prompts of uniform random token ids, lengths uniform in "
                "[128, 3072] from seed 0",
        "impl": "ours",
        "config": dict(config_record(shape, cfg, len(spec.run_order), n_req, 0, "mixed"), prefill_chunk=chunk,
                       new_tokens=new, prompt_tokens=sum(lens)),
        "clocks": clocks.summary(),
        "gpu_launches": launches,
        "generated_tokens_per_second": round(n_req * new / seconds, 1),
        "seconds": round(seconds, 3),
        "decode_steps": {"steps": dec[1], "mean_ms": round(1000.0 * dec[0] / max(dec[1], 1), 3),
                         "hbm_frac": round(dec[2] / max(dec[0], 1e-9) / 1e9 / pk["hbm_gbs"], 4)},
        "portion_steps": {"steps": por[1], "mean_ms": round(1000.0 * por[0] / max(por[1], 1), 3),
                          "tflops": round(por[2] / max(por[0], 1e-9) / 1e12, 1),
                          "frac": round(por[2] / max(por[0], 1e-9) / (pk["bf16_tflops"] * 1e12), 4),
                          "frac_of_sustained": round(por[2] / max(por[0], 1e-9) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "scheduler": {k: int(v) for k, v in metrics.items()},
        "peak_source": pk["source"],
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES))
    ap.add_argument("--workload", default=None, choices=["decode", "mixed"],
                    help="decode (default; with prefill and the batch points) or mixed (default of --shape 14b)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=0, help="decode batch (default 8; 64 for --shape 32b)")
    ap.add_argument("--new-tokens", type=int, default=128, help="mixed workload: tokens every request generates")
    ap.add_argument("--skip-extras", action="store_true", help="only the default decode measurement")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host (for profilers)")
    ap.add_argument("--only-prefill", action="store_true", help="run just the 2,048-token prefill (for profilers)")
    ap.add_argument("--streaming-kernel", action="store_true",
                    help="steps of up to 8 tokens on the weight-streaming mma.sync kernel instead of the tensor-core one")
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="repeat the block of --steps steps until this much is timed (0: one block, for profilers)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not offered")
        return 2
    args.warmup = max(args.warmup, 3)
    workload = args.workload or ("mixed" if args.shape == "14b" else "decode")
    if args.streaming_kernel:
        from safetyraise_lmengine_b200.kernels import ops
        ops.skinny_max_tokens = 8
    pk = peaks()
    out = run_mixed(args, args.shape, pk) if workload == "mixed" else run_decode(args, args.shape, pk)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
