"""Trace replay: feeds given token ids through the engine step by step and
writes the logits that a step asks for.  It samples nothing and has no model
code of its own: it builds the same ``Engine`` that generation uses and calls
its ``step``.

Input, one JSON object a line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step with wanted places it writes ``<out>/<step>.f32``: float32
little-endian [wanted, vocab], in the order of the entries and of ``want``.
After every step it prints ``done <step>``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_SIZE = 16          # divides 64, so a request's 64-token rounding is a whole number of pages
MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    os.makedirs(args.out, exist_ok=True)

    print("trace_run: loading (the first call compiles the CUDA kernels)", file=sys.stderr, flush=True)
    from .step import Engine, StepEntry
    num_pages = (args.max_tokens + PAGE_SIZE - 1) // PAGE_SIZE
    engine = Engine.from_folder(args.model, dtype=args.dtype, page_size=PAGE_SIZE, num_pages=num_pages,
                                max_requests=MAX_LIVE, max_batch_tokens=max(args.max_tokens, 64),
                                max_context=None)
    print("trace_run: ready", file=sys.stderr, flush=True)

    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.open_request()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                logits.cpu().numpy().astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            if rid in slots:
                engine.close_request(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
