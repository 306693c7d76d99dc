"""Plain, slow Qwen3 dense decoder: the oracle every engine test compares with.

Whole sequences, no cache, one function per part, NumPy only.  It shares no
code with the product package: it reads ``config.json`` keys and tensor names by
itself.  It rests on the reference's formulas (the reference is a Rust crate
that cannot be compiled without a Rust toolchain, so there is no reference
output to diff against); every function cites the reference file:line that it
restates.

All arithmetic runs in the dtype given (float64 by default, which makes this
the exact-math oracle; float32 reproduces the reference's own precision).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ----------------------------------------------------------------------------
# reading a model folder (independent of the product loader)
# ----------------------------------------------------------------------------

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32}


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_model_folder(path: str):
    """Returns (config dict, {tensor name: float32/int32 array}).

    Container format as parsed by src/artifact/mod.rs:706-851: u64 LE header
    length, JSON header, raw little-endian tensor bytes.
    """
    with open(os.path.join(path, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    base = 8 + hlen
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[base + lo:base + hi]
        if meta["dtype"] == "BF16":
            arr = _bf16_to_f32(np.frombuffer(raw, dtype=np.uint16))
        else:
            arr = np.frombuffer(raw, dtype=_ST_DTYPES[meta["dtype"]])
        tensors[name] = arr.reshape(meta["shape"]).copy()
    return config, tensors


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embedding(table: np.ndarray, ids) -> np.ndarray:
    """x[t,:] = E[id_t,:]; an id outside the table is an error.
    src/model/native.rs:213-229."""
    ids = np.asarray(ids, dtype=np.int64)
    if ids.size == 0 or ids.min() < 0 or ids.max() >= table.shape[0]:
        raise ValueError("token id outside the vocabulary")
    return table[ids]


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """var = mean(x^2); y = x * 1/sqrt(var+eps) * w, over the last axis.
    src/model/math.rs:28-50 (offset=false for Qwen3, src/model/native.rs:534)."""
    dt = x.dtype
    var = (x * x).sum(axis=-1, keepdims=True) / dt.type(x.shape[-1])
    inv = dt.type(1.0) / np.sqrt(var + dt.type(eps))
    return x * inv * weight.astype(dt)


def rope(x: np.ndarray, positions: np.ndarray, theta: float, rotary_dim: int) -> np.ndarray:
    """Half-split rotary encoding on x[T, heads, head_dim].

    angle = pos / theta^(2i/rotary_dim); (l, r) = (v[i], v[i+half]);
    v[i] = l cos - r sin; v[i+half] = r cos + l sin.  src/model/math.rs:52-99
    (axis 0 of the position triple is used when there is no mrope_section)."""
    dt = x.dtype
    half = rotary_dim // 2
    i = np.arange(half, dtype=dt)
    denom = np.power(dt.type(theta), (dt.type(2) * i) / dt.type(rotary_dim))
    angle = positions.astype(dt)[:, None] / denom[None, :]          # [T, half]
    sin, cos = np.sin(angle)[:, None, :], np.cos(angle)[:, None, :]
    out = x.copy()
    left, right = x[..., :half], x[..., half:2 * half]
    out[..., :half] = left * cos - right * sin
    out[..., half:2 * half] = right * cos + left * sin
    return out


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """q[T,nq,hd], k/v[T,nkv,hd] of one whole sequence -> [T,nq,hd].

    Query head h reads KV head h // (nq/nkv); scores scaled by 1/sqrt(hd);
    query t sees keys 0..t; softmax in the working dtype.
    src/model/math.rs:102-155 (the online form there equals this closed form)."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    dt = q.dtype
    scale = dt.type(1.0) / np.sqrt(dt.type(hd))
    out = np.zeros_like(q)
    mask = np.tril(np.ones((T, T), dtype=bool))
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale                     # [T, T]
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def sigmoid(x: np.ndarray) -> np.ndarray:
    """Branch-stable logistic.  src/model/math.rs:11-18."""
    pos = x >= 0
    e = np.exp(np.where(pos, -x, x))
    return np.where(pos, 1.0 / (1.0 + e), e / (1.0 + e)).astype(x.dtype)


def silu(x: np.ndarray) -> np.ndarray:
    """x * sigmoid(x).  src/model/math.rs:20-22."""
    return x * sigmoid(x)


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """x[T,in] . W[out,in]^T, no bias.  src/artifact/mod.rs:377-405."""
    return x @ w.astype(x.dtype).T


def attention_part(n1, positions, w, prefix, cfg) -> np.ndarray:
    """q/k/v projections, per-head RMSNorm of q and k, RoPE, causal GQA
    attention, output projection.  src/model/native.rs:611-646."""
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    hd = cfg.get("head_dim", cfg["hidden_size"] // nq)
    eps = cfg.get("rms_norm_eps", 1e-6)
    theta = rope_theta(cfg)
    rotary_dim = rotary_dim_of(cfg, hd)
    T = n1.shape[0]
    q = linear(n1, w[prefix + "q_proj.weight"]).reshape(T, nq, hd)
    k = linear(n1, w[prefix + "k_proj.weight"]).reshape(T, nkv, hd)
    v = linear(n1, w[prefix + "v_proj.weight"]).reshape(T, nkv, hd)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    q = rope(q, positions, theta, rotary_dim)
    k = rope(k, positions, theta, rotary_dim)
    a = causal_attention(q, k, v).reshape(T, nq * hd)
    return linear(a, w[prefix + "o_proj.weight"])


def feed_forward_part(n2, w, prefix) -> np.ndarray:
    """down(silu(gate(x)) * up(x)).  src/model/native.rs:552-557."""
    g = linear(n2, w[prefix + "gate_proj.weight"])
    u = linear(n2, w[prefix + "up_proj.weight"])
    return linear(silu(g) * u, w[prefix + "down_proj.weight"])


def block(x, positions, w, layer: int, cfg) -> np.ndarray:
    """Pre-norm residual block.  src/model/native.rs:526-562."""
    p = f"model.layers.{layer}."
    eps = cfg.get("rms_norm_eps", 1e-6)
    n1 = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    r = x + attention_part(n1, positions, w, p + "self_attn.", cfg)
    n2 = rms_norm(r, w[p + "post_attention_layernorm.weight"], eps)
    return r + feed_forward_part(n2, w, p + "mlp.")


def rope_theta(cfg) -> float:
    """rope_parameters/rope_scaling first, then the top level, default 1e6.
    src/model/spec.rs:283-293."""
    for key in ("rope_parameters", "rope_scaling"):
        sub = cfg.get(key)
        if isinstance(sub, dict) and "rope_theta" in sub:
            return float(sub["rope_theta"])
    return float(cfg.get("rope_theta", 1e6))


def rotary_dim_of(cfg, head_dim: int) -> int:
    """floor(head_dim * partial_rotary_factor), the factor looked up like rope_theta, default 1.
    src/model/spec.rs:266-282; elements beyond it pass unrotated (src/model/math.rs:66-67, 93-95)."""
    fraction = cfg.get("partial_rotary_factor", 1.0)
    for key in ("rope_parameters", "rope_scaling"):
        sub = cfg.get(key)
        if isinstance(sub, dict) and "partial_rotary_factor" in sub:
            fraction = sub["partial_rotary_factor"]
    return int(head_dim * float(fraction))


def model_logits(cfg: dict, w: dict, tokens, dtype=np.float64) -> np.ndarray:
    """Logits [T, V] of one whole sequence at positions 0..T-1.
    src/model/native.rs:231-312."""
    w = {k: (a.astype(dtype) if a.dtype.kind == "f" else a) for k, a in w.items()}
    x = embedding(w["model.embed_tokens.weight"], tokens)
    positions = np.arange(len(tokens))
    for layer in range(cfg["num_hidden_layers"]):
        x = block(x, positions, w, layer, cfg)
    hn = rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(hn, head)


def greedy_generate(cfg, w, prompt, steps: int, dtype=np.float64):
    """Whole-sequence recompute per token; ties go to the lowest id
    (src/frontend/sampling.rs:181-189)."""
    tokens = list(prompt)
    out = []
    for _ in range(steps):
        logits = model_logits(cfg, w, tokens, dtype)[-1]
        nxt = int(np.argmax(logits))
        out.append(nxt)
        tokens.append(nxt)
    return out


# ----------------------------------------------------------------------------
# sampling (src/frontend/sampling.rs:92-189) with an explicit uniform draw
# ----------------------------------------------------------------------------

def apply_repetition_penalty(logits: np.ndarray, history, penalty: float) -> np.ndarray:
    """Once per unique id: negative logits times p, others divided by p.
    src/frontend/sampling.rs:161-179."""
    out = logits.astype(np.float32).copy()
    if penalty == 1.0:
        return out
    for tok in set(int(t) for t in history):
        if 0 <= tok < out.shape[0]:
            out[tok] = out[tok] * np.float32(penalty) if out[tok] < 0 else out[tok] / np.float32(penalty)
    return out


def sample_distribution(logits, temperature, top_k, top_p):
    """Returns (candidate ids in draw order, weights, kept_sum): sort by value
    descending and id ascending, cut to top_k, softmax, cut at the first
    prefix whose mass >= top_p.  src/frontend/sampling.rs:104-147."""
    scaled = logits.astype(np.float32) / np.float32(temperature)
    order = np.lexsort((np.arange(scaled.shape[0]), -scaled))
    if top_k > 0:
        order = order[:top_k]
    vals = scaled[order]
    wts = np.exp(vals - vals.max()).astype(np.float32)
    wts = wts / wts.sum(dtype=np.float32)
    cum = np.cumsum(wts, dtype=np.float32)
    hit = np.nonzero(cum >= np.float32(top_p))[0]
    cutoff = int(hit[0]) + 1 if hit.size else len(wts)
    cutoff = max(1, min(cutoff, len(wts)))
    return order[:cutoff], wts[:cutoff], float(wts[:cutoff].sum(dtype=np.float32))


def sample(logits, history, temperature, top_k, top_p, penalty, uniform: float) -> int:
    """uniform in [0,1) stands for the generator's draw.
    src/frontend/sampling.rs:92-158."""
    adj = apply_repetition_penalty(np.asarray(logits), history, penalty)
    if temperature == 0.0:
        return int(np.argmax(adj))
    ids, wts, kept = sample_distribution(adj, temperature, top_k, top_p)
    draw = uniform * kept
    for tok, wt in zip(ids, wts):
        draw -= float(wt)
        if draw <= 0.0:
            return int(tok)
    return int(ids[-1])
