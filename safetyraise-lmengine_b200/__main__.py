"""Command line in the manner of the reference's ``rsinfer`` (src/cli.rs:24-57):

    python -m safetyraise_lmengine_b200 inspect   --model-path DIR [--context N]
    python -m safetyraise_lmengine_b200 run       --config FILE [--request FILE | --prompt-ids 1,2,3]
    python -m safetyraise_lmengine_b200 benchmark --config FILE --request FILE [--iterations N]
    python -m safetyraise_lmengine_b200 replay    --model DIR --dtype D --out DIR --max-tokens N

``serve`` (the HTTP server) is not part of this engine.  Text is not handled:
prompts are token ids, results are token ids.  The config file is a JSON object
``{"model_path": ..., "model_name": ..., "engine": {...}}``; a relative
model_path is resolved against the file (src/cli.rs:83-97); unknown keys are
refused.  A request file is ``{"prompt_ids": [...], "max_tokens": n,
"temperature": t, "top_p": p, "top_k": k, "repetition_penalty": r, "seed": s}``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

from .errors import ConfigError, EngineError

MAX_CONFIG_BYTES = 1 << 20


def _read_bounded(path: str, limit: int = MAX_CONFIG_BYTES) -> str:
    with open(path) as f:
        data = f.read(limit + 1)
    if len(data) > limit:
        raise ConfigError(f"{path}: larger than {limit} bytes")
    return data


def load_service_config(path: str):
    from .engine.llm import EngineConfig
    cfg = json.loads(_read_bounded(path))
    unknown = set(cfg) - {"model_path", "model_name", "engine"}
    if unknown:
        raise ConfigError(f"{path}: unknown key(s) {sorted(unknown)}")
    if "model_path" not in cfg:
        raise ConfigError(f"{path}: model_path is required")
    model_path = cfg["model_path"]
    if not os.path.isabs(model_path):
        model_path = os.path.join(os.path.dirname(os.path.abspath(path)), model_path)
    return model_path, cfg.get("model_name", os.path.basename(model_path.rstrip("/"))), \
        EngineConfig.from_dict(cfg.get("engine", {}))


def load_request(text: str):
    from .engine.scheduler import GenerationRequest
    from .sampling.params import SamplingParams
    req = json.loads(text)
    known = {"prompt_ids", "max_tokens", "temperature", "top_p", "top_k", "repetition_penalty", "seed", "model"}
    unknown = set(req) - known
    if unknown:
        raise ConfigError(f"request: unknown key(s) {sorted(unknown)}")
    sp = SamplingParams()
    for key, attr in (("max_tokens", "max_new_tokens"), ("temperature", "temperature"), ("top_p", "top_p"),
                      ("top_k", "top_k"), ("repetition_penalty", "repetition_penalty"), ("seed", "seed")):
        if req.get(key) is not None:
            setattr(sp, attr, req[key])
    return GenerationRequest(list(req.get("prompt_ids", [])), sp)


def cmd_inspect(args) -> int:
    """Reads configuration and tensors; never runs the model (src/cli.rs:100-124)."""
    from .config.registry import read_config_json, spec_from_config
    from .parts.model import tensor_decls
    from .weights.loader import check_against, logical_bytes
    from .weights.safetensors_io import WeightFolder
    spec = spec_from_config(read_config_json(args.model_path))
    if not 0 < args.context <= spec.max_position_embeddings:
        raise ConfigError("inspect: --context is outside the model's positions")
    folder = WeightFolder(args.model_path)
    check_against(tensor_decls(spec), {n: folder.meta(n)[1] for n in folder.names()})
    count, total = logical_bytes(folder)
    per_token = 0
    seen = set()
    for step in spec.run_order:
        m = spec.layers[step.layer].mixer
        if step.writes_cache and step.cache not in seen and hasattr(m, "kv_heads"):
            seen.add(step.cache)
            per_token += 2 * m.kv_heads * m.head_dim
    elem = 4 if args.dtype == "float32" else 2
    out = {"spec": spec.to_json(), "tensors": count, "logical_weight_bytes": total, "context": args.context,
           "state_bytes_per_request": per_token * elem * args.context, "state_dtype": args.dtype,
           "validation": "configuration and weights parsed and matched only; the model was not run"}
    print(json.dumps(out, indent=1, default=str))
    return 0


def _make_llm(config_path):
    from .engine.llm import LLM
    t0 = time.monotonic()
    model_path, name, engine_cfg = load_service_config(config_path)
    llm = LLM.from_folder(model_path, engine_cfg)
    return llm, name, (time.monotonic() - t0) * 1000.0


def _one(llm, request):
    import copy
    t0 = time.monotonic()
    rid = llm.submit(copy.deepcopy(request))
    llm.run_until_idle()
    res = llm.take_result(rid)
    return res, time.monotonic() - t0


def cmd_run(args) -> int:
    llm, name, _ = _make_llm(args.config)
    if args.request:
        text = _read_bounded(args.request, 8 << 20)
    elif args.prompt_ids:
        text = json.dumps({"prompt_ids": [int(t) for t in args.prompt_ids.split(",") if t.strip()]})
    else:
        text = sys.stdin.read(8 << 20)
    res, _ = _one(llm, load_request(text))
    print(json.dumps({"model": name, "tokens": res.tokens, "finish_reason": res.finish_reason,
                      "usage": vars(res.usage), "error": res.error}, indent=1))
    return 0 if res.error is None else 1


def cmd_benchmark(args) -> int:
    """End-to-end seconds per run of one request (src/cli.rs:166-202)."""
    if not 1 <= args.iterations <= 100:
        raise ConfigError("benchmark: --iterations must lie in 1..=100")
    request = load_request(_read_bounded(args.request, 8 << 20))
    llm, name, load_ms = _make_llm(args.config)
    runs = []
    for _ in range(args.iterations):
        res, seconds = _one(llm, request)
        n = res.usage.completion_tokens
        runs.append({"seconds": seconds, "completion_tokens": n,
                     "end_to_end_tokens_per_second": n / seconds if seconds > 0 else 0.0,
                     "usage": vars(res.usage), "finish_reason": res.finish_reason})
    print(json.dumps({"capabilities": {"model": name, "dtype": llm.config.dtype, "metrics": llm.metrics()},
                      "load_ms": load_ms, "runs": runs,
                      "scope": "end-to-end time of the given request through queue, prefill and decode; "
                               "not pure decode throughput"}, indent=1))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="safetyraise_lmengine_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("inspect", help="parse configuration and weights; do not run the model")
    p.add_argument("--model-path", required=True)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.set_defaults(fn=cmd_inspect)
    p = sub.add_parser("run", help="run one request, print JSON")
    p.add_argument("--config", required=True)
    g = p.add_mutually_exclusive_group()
    g.add_argument("--request")
    g.add_argument("--prompt-ids", help="comma-separated token ids (text prompts need a tokenizer: not here)")
    p.set_defaults(fn=cmd_run)
    p = sub.add_parser("benchmark", help="time one request end to end")
    p.add_argument("--config", required=True)
    p.add_argument("--request", required=True)
    p.add_argument("--iterations", type=int, default=3)
    p.set_defaults(fn=cmd_benchmark)
    p = sub.add_parser("replay", help="feed given token ids step by step, dump logits (see bin/trace_run)")
    p.add_argument("rest", nargs=argparse.REMAINDER)
    p.set_defaults(fn=None)
    args = ap.parse_args(argv)
    try:
        if args.command == "replay":
            from .engine.replay import main as replay_main
            return replay_main(args.rest)
        return args.fn(args)
    except EngineError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
