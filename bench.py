"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step: every request of the batch gets its next token.
The default run has the sizes of the 8B configuration (36 layers, hidden 4096,
32/8 heads of 128, intermediate 12288, vocabulary 151936), random weights in
bfloat16, a batch of 8 and 2,048 tokens of context per request.  It prints one
JSON line: decoded tokens a second on the device (`value`: CUDA events around
the device half of each step -- the upload of the batch and the forward; the
host half, checks and batch layout, is done before the first event), the same
through the Python entry point by the wall clock with host tokens in and out
(`e2e`), a 2,048-token prefill (the median of runs back to back: the GPU is at
its power cap by then), the decode step's fraction of the HBM roofline, and
decode at batch 1 and 64.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36,
    "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
FULL_LAYERS = CONFIG_8B["num_hidden_layers"]
CONTEXT = 2048            # tokens each request holds while decoding; the benchmark context is 4096
PREFILL_TOKENS = 2048
PAGE_SIZE = 16


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


def build_engine(layers: int, max_requests: int, tokens_in_cache: int, max_batch_tokens: int, graphs=True):
    import torch
    from safetyraise_lmengine_b200 import Engine, spec_from_config
    from safetyraise_lmengine_b200.parts.model import tensor_decls
    from safetyraise_lmengine_b200.weights.random_init import RandomWeights
    cfg = dict(CONFIG_8B, num_hidden_layers=layers)
    spec = spec_from_config(cfg)
    src = RandomWeights(tensor_decls(spec), seed=0, device="cuda:0")
    num_pages = (tokens_in_cache + PAGE_SIZE - 1) // PAGE_SIZE + max_requests
    eng = Engine.from_source(cfg, src, dtype="bfloat16", page_size=PAGE_SIZE, num_pages=num_pages,
                             max_requests=max_requests, max_batch_tokens=max_batch_tokens, max_context=4096,
                             options={"cuda_graphs": graphs})
    torch.cuda.synchronize()
    return eng


def fill_contexts(eng, batch: int, context: int):
    """Opens `batch` requests that each hold `context` tokens.  The cache contents are random
    (attention time does not depend on the values); the page accounting is the real one."""
    import torch
    for pool in eng.cache.kv_pools.values():
        flat = pool.view(-1)
        step = 1 << 26
        for lo in range(0, flat.numel(), step):
            flat[lo:lo + step].normal_(0.0, 1.0)
    slots = []
    for _ in range(batch):
        s = eng.open_request()
        assert eng.cache.reserve(s, context)
        eng.cache.commit(s, context)
        slots.append(s)
    torch.cuda.synchronize()
    return slots


def time_decode(eng, slots, steps: int, warmup: int):
    """Device time of `steps` decode steps (CUDA events around each step); returns (ms list, launches)."""
    import torch
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.kernels import ops
    gen = torch.Generator().manual_seed(0)
    vocab = eng.spec.vocab_size
    def prepared():                     # the host half of a step: checks, page reservation, batch layout
        toks = torch.randint(0, vocab, (len(slots),), generator=gen).tolist()
        return eng.prepare([StepEntry(s, [t], [0]) for s, t in zip(slots, toks)])
    for _ in range(warmup):
        eng.run(prepared())
    torch.cuda.synchronize()
    ms = []
    launches0 = ops.launches
    for _ in range(steps):
        prep = prepared()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.run(prep)                   # the device half: one upload of the batch, then the forward
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
    # the contexts grew by warmup+steps tokens; put them back so that every measurement sees `context`
    return ms, ops.launches - launches0


def reset_contexts(eng, slots, context):
    for s in slots:
        eng.cache.truncate(s, context)


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


def prefill_flops(spec, tokens: int) -> float:
    m = spec.layers[0].mixer
    ff = spec.layers[0].feed_forward
    H = spec.hidden_size
    per_layer = 2 * tokens * ((m.heads + 2 * m.kv_heads) * m.head_dim * H + m.heads * m.head_dim * H
                              + 3 * H * ff.intermediate_size)
    attention = 2 * tokens * tokens * m.heads * m.head_dim        # causal: QK^T and PV, half of the square each
    return len(spec.run_order) * (per_layer + attention) + 2 * spec.vocab_size * H


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
    times.sort()
    return times[len(times) // 2]      # the median: after the warm-ups the GPU sits at its power cap (sustained clocks)


def time_e2e(eng, batch: int, context: int, steps: int, warmup: int):
    """Decode through the Python entry point: requests are submitted as token ids, prefilled by the
    scheduler, and each timed step copies its token ids and batch layout from pinned host memory
    and reads the sampled tokens back to the host."""
    import torch
    from safetyraise_lmengine_b200 import LLM, EngineConfig, SamplingParams
    from safetyraise_lmengine_b200.engine.scheduler import GenerationRequest
    cfg = EngineConfig(max_context=4096, max_active=batch, queue_capacity=batch, prefill_chunk=2048,
                       max_batch_tokens=eng.mctx.max_batch_tokens, page_size=PAGE_SIZE)
    llm = LLM(eng, cfg)
    llm.eos = set()
    gen = torch.Generator().manual_seed(2)
    for _ in range(batch):
        prompt = torch.randint(0, eng.spec.vocab_size, (context,), generator=gen).tolist()
        llm.submit(GenerationRequest(prompt, SamplingParams(temperature=0.0, max_new_tokens=warmup + steps + 8)))
    decoding = lambda: all(len(st.tokens) > st.usage.prompt_tokens for st in llm._live.values())
    while not decoding():
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        llm.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    h2d = eng.last_h2d_bytes
    for rid in list(llm._live):
        llm.cancel(rid)
    llm.step()
    return batch * steps / seconds, h2d, batch * 4


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-extras", action="store_true", help="only the default decode measurement")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host (for profilers)")
    ap.add_argument("--only-prefill", action="store_true", help="run just the 2,048-token prefill (for profilers)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not offered")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from safetyraise_lmengine_b200.kernels import ops
    pk = peaks()
    B = args.batch
    big = max(64, B)
    room = max(256, args.warmup + args.steps + 72)        # tokens a request may grow by during a measurement
    eng = build_engine(args.layers, max_requests=big, tokens_in_cache=big * (CONTEXT + room) + PREFILL_TOKENS,
                       max_batch_tokens=PREFILL_TOKENS, graphs=not args.no_graphs)
    if args.only_prefill:
        pf_ms = time_prefill(eng, PREFILL_TOKENS, 5)
        print(json.dumps({"prefill_ms": pf_ms, "tokens": PREFILL_TOKENS}))
        return 0
    slots = fill_contexts(eng, B, CONTEXT)
    with ClockSampler() as clocks:
        ms, launches = time_decode(eng, slots, args.steps, args.warmup)
    ms_per_step = sum(ms) / len(ms)
    value = B / (ms_per_step / 1000.0)
    # the contexts grow by one token a step: the cache read in the timed steps is that of the mean length
    nbytes = decode_bytes(eng, B, CONTEXT + args.warmup + args.steps // 2)
    achieved = nbytes / (ms_per_step / 1000.0) / 1e9
    out = {
        "metric": "decode_tokens_per_second", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, random cache contents",
        "impl": "ours",
        "config": {"model": "Qwen3-8B layer sizes", "layers": args.layers, "layers_of_config": FULL_LAYERS,
                   "hidden": 4096, "heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288,
                   "vocab": 151936, "global_batch": B, "seq_len": CONTEXT, "benchmark_context": 4096,
                   "page_size": PAGE_SIZE, "parallelism": "single GPU",
                   "l2": "not flushed: each step reads >15 GB of weights, far more than the 126 MB L2"},
        "clocks": clocks.summary(),
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes,
                     "peak_source": pk["source"]},
    }
    for s in slots:
        eng.close_request(s)

    if not args.skip_extras:
        points = {}
        for b in (1, 64):
            sl = fill_contexts(eng, b, CONTEXT)
            pms, _ = time_decode(eng, sl, max(5, args.steps // 2), 3)
            points[f"decode_b{b}"] = round(b / (sum(pms) / len(pms) / 1000.0), 1)
            for s in sl:
                eng.close_request(s)
        out["points"] = points
        pf_ms = time_prefill(eng, PREFILL_TOKENS, 5)
        flops = prefill_flops(eng.spec, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pf_ms / 1000.0), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(pf_ms, 3),
                          "frac": round(flops / (pf_ms / 1000.0) / (pk["bf16_tflops"] * 1e12), 4),
                          "frac_of_sustained": round(flops / (pf_ms / 1000.0) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                          "tflops": round(flops / (pf_ms / 1000.0) / 1e12, 1),
                          "regime": "sustained: median of 5 runs after 3 warm-ups, back to back"}
        e2e, h2d, d2h = time_e2e(eng, B, CONTEXT, args.steps, args.warmup)
        out["e2e"] = {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": d2h}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
