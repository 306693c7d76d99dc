"""Command line in the manner of the reference's ``rsinfer`` (src/cli.rs:24-57):

    python -m safetyraise_lmengine_b200 inspect   --model-path DIR [--context N]
    python -m safetyraise_lmengine_b200 run       --config FILE [--request FILE | --prompt-ids 1,2,3]
    python -m safetyraise_lmengine_b200 benchmark --config FILE --request FILE [--iterations N]
    python -m safetyraise_lmengine_b200 replay    --model DIR --dtype D --out DIR --max-tokens N

In place of a model folder, ``inspect``, ``run`` and ``benchmark`` take
``--random-weights SEED --config-json FILE``: the architecture's config.json
alone, every tensor filled from the seed and the tensor's name (``--config`` is
then optional and gives the engine options only).

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


def load_service_config(path: str, need_model: bool = True):
    from .engine.llm import EngineConfig
    cfg = json.loads(_read_bounded(path))
    unknown = set(cfg) - {"model_path", "model_name", "engine"}
    if unknown:
        raise ConfigError(f"{path}: unknown key(s) {sorted(unknown)}")
    if "model_path" not in cfg:
        if need_model:
            raise ConfigError(f"{path}: model_path is required")
        return None, cfg.get("model_name", "random"), EngineConfig.from_dict(cfg.get("engine", {}))
    model_path = cfg["model_path"]
    if not os.path.isabs(model_path):
        model_path = os.path.join(os.path.dirname(os.path.abspath(path)), model_path)
    return model_path, cfg.get("model_name", os.path.basename(model_path.rstrip("/"))), \
        EngineConfig.from_dict(cfg.get("engine", {}))


def _random_source(args):
    """(config.json dict, weight source) of --random-weights SEED --config-json FILE, or None."""
    if args.random_weights is None and not args.config_json:
        return None
    if args.random_weights is None or not args.config_json:
        raise ConfigError("--random-weights SEED and --config-json FILE go together")
    from .config.registry import spec_from_config
    from .parts.model import tensor_decls
    from .weights.random_init import RandomWeights
    config = json.loads(_read_bounded(args.config_json))
    if not isinstance(config, dict):
        raise ConfigError(f"{args.config_json}: top level must be an object")
    return config, RandomWeights(tensor_decls(spec_from_config(config)), args.random_weights)


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
    from .config.registry import architecture_of, read_config_json
    from .engine.step import DTYPES
    from .parts.model import cache_groups_of, tensor_decls
    from .weights.loader import check_against, logical_bytes
    from .weights.safetensors_io import WeightFolder
    rnd = _random_source(args)
    if (rnd is None) == (args.model_path is None):
        raise ConfigError("inspect: give --model-path DIR, or --random-weights SEED --config-json FILE")
    config = rnd[0] if rnd else read_config_json(args.model_path)
    arch = architecture_of(config)
    spec = arch.read_spec(config)
    if not 0 < args.context <= spec.max_position_embeddings:
        raise ConfigError("inspect: --context is outside the model's positions")
    source = rnd[1] if rnd else arch.source_for(WeightFolder(args.model_path))
    check_against(tensor_decls(spec), {n: source.meta(n)[1] for n in source.names()})
    count, total = logical_bytes(source)
    # what a request holds: the keys and values of every paged group and the fixed-size state of the others
    dtype = DTYPES[args.dtype]
    groups = cache_groups_of(spec)
    state = sum(g.bytes_per_request(dtype, args.context) for g in groups)
    out = {"spec": spec.to_json(), "tensors": count, "logical_weight_bytes": total, "context": args.context,
           "state_bytes_per_request": state, "state_dtype": args.dtype,
           "cache_groups": [{"name": g.name, "kind": g.kind, "entries": len(g.entries),
                             "bytes_per_request": g.bytes_per_request(dtype, args.context)} for g in groups],
           "validation": "configuration and weights parsed and matched only; the model was not run"}
    print(json.dumps(out, indent=1, default=str))
    return 0


def _make_llm(args):
    from .engine.llm import LLM, EngineConfig
    t0 = time.monotonic()
    rnd = _random_source(args)
    if args.config:
        model_path, name, engine_cfg = load_service_config(args.config, need_model=rnd is None)
    elif rnd is not None:
        model_path, name, engine_cfg = None, "random", EngineConfig()
    else:
        raise ConfigError("give --config FILE, or --random-weights SEED --config-json FILE")
    if rnd is not None:
        if model_path is not None:
            raise ConfigError("--random-weights stands in place of model_path: the config file names a folder")
        llm = LLM.from_source(rnd[0], rnd[1], engine_cfg)
    else:
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
    llm, name, _ = _make_llm(args)
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
    llm, name, load_ms = _make_llm(args)
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
    def random_options(p):
        p.add_argument("--random-weights", type=int, metavar="SEED",
                       help="fill every tensor from this seed instead of reading a folder")
        p.add_argument("--config-json", metavar="FILE", help="the architecture's config.json for --random-weights")

    p = sub.add_parser("inspect", help="parse configuration and weights; do not run the model")
    p.add_argument("--model-path")
    random_options(p)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.set_defaults(fn=cmd_inspect)
    p = sub.add_parser("run", help="run one request, print JSON")
    p.add_argument("--config")
    random_options(p)
    g = p.add_mutually_exclusive_group()
    g.add_argument("--request")
    g.add_argument("--prompt-ids", help="comma-separated token ids (text prompts need a tokenizer: not here)")
    p.set_defaults(fn=cmd_run)
    p = sub.add_parser("benchmark", help="time one request end to end")
    p.add_argument("--config")
    random_options(p)
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
