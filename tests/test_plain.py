"""The plain implementation itself (no GPU): the reference's hand-computed cases, its C linear
operator's outputs, and invariants of the whole model."""
import json
import math
import os

import numpy as np
import pytest
from conftest import TINY_A, TINY_B

import plain_qwen3 as P


def test_attention_known_weighted_average():
    # src/model/math.rs:246-253: q = [1, 0] (2 heads, dim 1), keys 0 and ln 2, values 2 and 8 -> 6 and 5
    q = np.array([[[0.0], [0.0]], [[1.0], [0.0]]])          # two tokens; the second is the reference's query
    k = np.array([[[0.0]], [[math.log(2.0)]]])
    v = np.array([[[2.0]], [[8.0]]])
    out = P.causal_attention(q, k, v)
    assert abs(out[1, 0, 0] - 6.0) < 1e-12 and abs(out[1, 1, 0] - 5.0) < 1e-12
    assert out[0, 0, 0] == 2.0                               # the first token sees only itself


def test_partial_rope_keeps_the_tail():
    # src/model/math.rs:295-307: rotary_dim 2 of head_dim 4 at position 1
    x = np.array([[[1.0, 0.0, 7.0, 9.0]]])
    y = P.rope(x, np.array([1]), 10000.0, 2)
    assert abs(y[0, 0, 0] - math.cos(1.0)) < 1e-12 and abs(y[0, 0, 1] - math.sin(1.0)) < 1e-12
    assert list(y[0, 0, 2:]) == [7.0, 9.0]


def test_rope_pairs_are_half_split():
    # src/model/math.rs:91-95: (left, right) = (head[i], head[i + half]) with half = rotary_dim / 2.
    # rotary_dim 4 of head_dim 6, theta 1 (every angle equals the position), position 1: the pairs
    # are (0, 2) and (1, 3), not (0, 1) and (2, 3); elements 4 and 5 pass
    x = np.array([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]])
    y = P.rope(x, np.array([1]), 1.0, 4)[0, 0]
    c, s = math.cos(1.0), math.sin(1.0)
    want = [1 * c - 3 * s, 2 * c - 4 * s, 3 * c + 1 * s, 4 * c + 2 * s, 5.0, 6.0]
    assert np.allclose(y, want, rtol=0, atol=1e-12)
    assert P.rotary_dim_of({"partial_rotary_factor": 0.5}, 64) == 32
    assert P.rotary_dim_of({"rope_parameters": {"partial_rotary_factor": 0.25}, "partial_rotary_factor": 0.5}, 64) == 16
    assert P.rotary_dim_of({}, 48) == 48


def test_rms_norm_and_silu():
    x = np.array([[3.0, 4.0]])
    y = P.rms_norm(x, np.array([1.0, 2.0]), 1e-6)
    inv = 1 / math.sqrt(12.5 + 1e-6)
    assert np.allclose(y, [[3 * inv, 8 * inv]], rtol=1e-12)
    for v in (-30.0, -1.0, 0.0, 2.5, 40.0):
        assert abs(P.silu(np.array([v]))[0] - v / (1 + math.exp(-v))) < 1e-12


def test_linear_against_the_references_c_operator():
    path = os.path.join(os.path.dirname(__file__), "golden", "linear_golden.json")
    for case in json.load(open(path))["cases"]:
        w = np.array(case["weight"], dtype=np.float32)
        x = np.array(case["input"], dtype=np.float32)
        ref = np.array(case["output"], dtype=np.float32)
        assert np.allclose(P.linear(x.astype(np.float64), w), ref, rtol=1e-5, atol=1e-6), case["name"]
    assert json.load(open(path))["cases"][0]["output"] == [[-2.0, 20.0], [-2.0, 47.0]]


@pytest.mark.parametrize("name", ["A", "B"])
def test_model_is_causal_and_float32_agrees(name, folder_a, folder_b):
    folder = folder_a if name == "A" else folder_b
    cfg, w = P.read_model_folder(folder)
    rng = np.random.default_rng(0)
    toks = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=40)]
    full = P.model_logits(cfg, w, toks)
    assert full.shape == (40, cfg["vocab_size"]) and np.isfinite(full).all()
    head = P.model_logits(cfg, w, toks[:23])
    assert np.allclose(full[:23], head, rtol=1e-10, atol=1e-12)      # later tokens change nothing earlier
    f32 = P.model_logits(cfg, w, toks, np.float32)
    assert np.abs(f32 - full).max() <= 1e-4 * np.abs(full).max()   # the formulas' own float32 rounding
    other = list(toks)
    other[5] = (other[5] + 1) % cfg["vocab_size"]
    changed = P.model_logits(cfg, w, other)
    assert np.array_equal(changed[:5], full[:5]) and not np.allclose(changed[5:], full[5:])


def test_sampling_order_of_operations():
    logits = np.array([0.2, 1.1, 0.7, -0.3], dtype=np.float32)
    assert P.sample(logits, [], 0.0, 0, 1.0, 1.0, 0.5) == 1
    assert P.sample(np.array([1.0, 1.5], np.float32), [1], 0.0, 0, 1.0, 2.0, 0.0) == 0   # sampling.rs:232-241
    out = P.apply_repetition_penalty(np.array([4.0, -4.0], np.float32), [0, 0, 1, 1], 2.0)
    assert list(out) == [2.0, -8.0]                                                       # sampling.rs:243-248
    ids, wts, kept = P.sample_distribution(logits, 1.0, 2, 1.0)
    assert list(ids) == [1, 2] and abs(kept - 1.0) < 1e-6
    ids, _, _ = P.sample_distribution(logits, 1.0, 0, 0.3)
    assert list(ids) == [1]                                   # top-p can cut to the first token
    ids, _, _ = P.sample_distribution(np.array([1.0, 1.0, 1.0], np.float32), 1.0, 2, 1.0)
    assert list(ids) == [0, 1]                                # ties by ascending id
    assert P.sample(logits, [], 1.0, 0, 1.0, 1.0, 0.0) == 1 and P.sample(logits, [], 1.0, 0, 1.0, 1.0, 0.9999) == 3
