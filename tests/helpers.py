"""Shared helpers of the GPU tests: tolerances, replay of cut-up requests, the oracle."""
import functools

import numpy as np

import plain_qwen3

# Largest |engine - plain| allowed, as a fraction of the largest |plain logit| compared.
# float32: summation order is the only difference.  bfloat16: activations and the cache are
# rounded to 8 bits of mantissa at every kernel boundary.  Twice the largest error any comparison of
# the whole GPU suite has shown (5.4e-6 and 8.9e-3, both on one block at 14B / 32B layer sizes; the
# run prints its own figures at its end).
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


# The largest error every comparison of this run has seen, per dtype (printed at the end of the run).
WORST = {}


def note_error(dtype: str, err: float, where: str = "") -> None:
    if err > WORST.get(dtype, (0.0, ""))[0]:
        WORST[dtype] = (err, where)


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


@functools.lru_cache(maxsize=64)
def _plain_cached(folder: str, tokens: tuple):
    cfg, w = plain_qwen3.read_model_folder(folder)
    return plain_qwen3.model_logits(cfg, w, list(tokens), np.float64)


def plain_logits(folder: str, tokens) -> np.ndarray:
    return _plain_cached(folder, tuple(int(t) for t in tokens))


def random_tokens(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def replay(engine, steps):
    """steps: list of {"entries": [(rid, tokens, want)], "end": [rid]}.
    Returns {(rid, position): float32 logits row}."""
    from safetyraise_lmengine_b200.engine.step import StepEntry
    slots, fed, out = {}, {}, {}
    for st in steps:
        entries, where = [], []
        for rid, tokens, want in st["entries"]:
            if rid not in slots:
                slots[rid] = engine.open_request()
                fed[rid] = 0
            entries.append(StepEntry(slots[rid], tokens, want))
            where += [(rid, fed[rid] + w) for w in want]
            fed[rid] += len(tokens)
        if entries:
            logits = engine.step(entries).cpu().numpy().copy()
            assert logits.shape[0] == len(where)
            for key, row in zip(where, logits):
                out[key] = row
        for rid in st.get("end", []):
            engine.close_request(slots.pop(rid))
    for rid in list(slots):
        engine.close_request(slots.pop(rid))
    return out


def cut_whole(rid, tokens):
    return [{"entries": [(rid, tokens, list(range(len(tokens))))], "end": [rid]}]


def cut_bulk_tail(rid, tokens, tail=32):
    tail = min(tail, len(tokens) - 1)
    head = len(tokens) - tail
    steps = [{"entries": [(rid, tokens[:head], list(range(head)))]}]
    for i in range(head, len(tokens)):
        steps.append({"entries": [(rid, tokens[i:i + 1], [0])]})
    steps[-1]["end"] = [rid]
    return steps


def cut_portions(rid, tokens, sizes=(7, 2, 13, 3, 2, 5, 31, 2, 64, 3)):
    steps, i, k = [], 0, 0
    while i < len(tokens):
        n = min(sizes[k % len(sizes)], len(tokens) - i)
        if len(tokens) - i - n == 1:        # never leave a single-token portion by accident
            n += 1
        steps.append({"entries": [(rid, tokens[i:i + n], list(range(n)))]})
        i += n
        k += 1
    steps[-1]["end"] = [rid]
    return steps


def check_against_plain(got: dict, folder: str, requests: dict, dtype: str):
    """got: {(rid, pos): row}; requests: {rid: tokens}.  Every position of every request must be there."""
    worst = 0.0
    for rid, tokens in requests.items():
        ref = plain_logits(folder, tokens)
        rows = np.stack([got[(rid, p)] for p in range(len(tokens))])
        err = np.abs(rows.astype(np.float64) - ref).max(axis=1) / np.abs(ref).max()
        bad = np.nonzero(err > TOL[dtype])[0]
        assert bad.size == 0, (f"request {rid}: first wrong position {bad[0]} of {len(tokens)} "
                               f"(rel err {err[bad[0]]:.3e} > {TOL[dtype]:.0e}); wrong positions {bad[:20]}")
        worst = max(worst, float(err.max()))
    note_error(dtype, worst, folder.rsplit("/", 1)[-1])
    return worst
