"""Safetensors reading and writing, the loader's one error, random weights (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch
from conftest import TINY_A, TINY_B

import plain_qwen3
from safetyraise_lmengine_b200 import spec_from_config
from safetyraise_lmengine_b200.errors import WeightError
from safetyraise_lmengine_b200.parts.model import tensor_decls
from safetyraise_lmengine_b200.weights.loader import check_against, load_tensors
from safetyraise_lmengine_b200.weights.random_init import RandomWeights, write_model_folder
from safetyraise_lmengine_b200.weights.safetensors_io import SafetensorsFile, WeightFolder, write_safetensors


def test_round_trip_and_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4, 2).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "d": torch.randn(7).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t)
    for k, v in t.items():
        got = f.get(k)
        assert got.dtype == v.dtype and torch.equal(got, v)


def test_random_folder_matches_config_and_is_seeded(tmp_path):
    d0 = write_model_folder(TINY_B, 1, str(tmp_path / "m0"))
    d1 = write_model_folder(TINY_B, 1, str(tmp_path / "m1"))
    d2 = write_model_folder(TINY_B, 2, str(tmp_path / "m2"))
    w0, w1, w2 = WeightFolder(d0), WeightFolder(d1), WeightFolder(d2)
    names = set(w0.names())
    assert len(names) == 11 * 3 + 3                      # 11 per layer + embed, norm, lm_head
    assert "lm_head.weight" in names
    for n in names:
        assert torch.equal(w0.get(n), w1.get(n))
    assert not torch.equal(w0.get("model.embed_tokens.weight"), w2.get("model.embed_tokens.weight"))
    emb = w0.get("model.embed_tokens.weight")
    assert emb.dtype == torch.bfloat16 and abs(emb.float().std().item() - 0.02) < 0.002
    nw = w0.get("model.layers.0.self_attn.q_norm.weight")
    assert nw.dtype == torch.float32 and abs(nw.mean().item() - 1.0) < 0.1
    cfg, tensors = plain_qwen3.read_model_folder(d0)      # the plain reader sees the same bytes
    assert cfg == TINY_B
    assert np.array_equal(tensors["model.embed_tokens.weight"], emb.float().numpy())


def test_tied_model_has_no_head(tmp_path):
    d = write_model_folder(TINY_A, 0, str(tmp_path / "m"))
    assert "lm_head.weight" not in set(WeightFolder(d).names())
    assert len(set(WeightFolder(d).names())) == 11 * 2 + 2


def test_one_error_lists_missing_unexpected_and_shapes():
    spec = spec_from_config(TINY_A)
    decls = tensor_decls(spec)
    have = {d.name: d.shape for d in decls}
    have.pop("model.norm.weight")
    have.pop("model.layers.1.mlp.up_proj.weight")
    have["model.layers.0.extra.weight"] = (3,)
    have["model.embed_tokens.weight"] = (255, 64)
    with pytest.raises(WeightError) as e:
        check_against(decls, have)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.norm.weight" in msg and "up_proj" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.extra.weight" in msg
    assert "wrong shapes (1)" in msg and "[255, 64]" in msg and "[256, 64]" in msg


def test_precision_policy():
    spec = spec_from_config(TINY_A)
    decls = tensor_decls(spec)
    src = RandomWeights(decls, 0)
    t16 = load_tensors(src, decls, torch.bfloat16, "cpu")
    t32 = load_tensors(src, decls, torch.float32, "cpu")
    assert t16["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t16["model.norm.weight"].dtype == torch.float32          # stored in 32-bit: stays so
    assert t32["model.embed_tokens.weight"].dtype == torch.float32
    assert torch.equal(t32["model.embed_tokens.weight"], t16["model.embed_tokens.weight"].float())

    class F32Source(RandomWeights):                                  # a matrix stored in 32-bit stays so
        def meta(self, n):
            dt, shape, nbytes = super().meta(n)
            return torch.float32, shape, nbytes
        def get(self, n):
            return super().get(n).float()
    t = load_tensors(F32Source(decls, 0), decls, torch.bfloat16, "cpu")
    assert t["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32


def _write_raw(path, header: dict, data: bytes, dup=None):
    text = json.dumps(header)
    if dup:
        text = text[:-1] + "," + dup + "}"
    raw = text.encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)) + raw + data)


@pytest.mark.parametrize("header, data, dup", [
    ({"a": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 8, None),
    ({"a": {"dtype": "F32", "shape": [], "data_offsets": [0, 4]}}, b"\0" * 4, None),
    ({"a": {"dtype": "F32", "shape": [0], "data_offsets": [0, 0]}}, b"", None),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8, None),       # byte length
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, None),       # out of range
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
      "b": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 8, None),       # overlap
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4,
     '"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}'),                        # duplicate key
])
def test_malformed_files_are_refused(tmp_path, header, data, dup):
    p = str(tmp_path / "bad.safetensors")
    _write_raw(p, header, data, dup)
    with pytest.raises(WeightError):
        SafetensorsFile(p)


def test_folder_needs_exactly_one_container(tmp_path):
    with pytest.raises(WeightError):
        WeightFolder(str(tmp_path))
    write_safetensors(str(tmp_path / "model.safetensors"), {"a": torch.zeros(1)})
    (tmp_path / "model.safetensors.index.json").write_text('{"weight_map": {}}')
    with pytest.raises(WeightError):
        WeightFolder(str(tmp_path))


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    w = WeightFolder(str(tmp_path))
    assert set(w.names()) == {"a", "b"} and w.get("b").shape == (3,)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "../s1.safetensors"}}))
    with pytest.raises(WeightError):
        WeightFolder(str(tmp_path))


def _renamed_folder(tmp_path, config, seed):
    """A folder whose text model is stored as model.language_model.* (the output head keeps its name)."""
    spec = spec_from_config(config)
    src = RandomWeights(tensor_decls(spec), seed)
    tensors = {}
    for n in src.names():
        stored = "model.language_model." + n[len("model."):] if n.startswith("model.") else n
        tensors[stored] = src.get(n)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    (tmp_path / "config.json").write_text(json.dumps(config))
    return str(tmp_path), src


def test_language_model_prefix_is_read_as_the_plain_names(tmp_path):
    """src/model/native.rs:156-165: model.language_model.embed_tokens.weight present -> that prefix."""
    from conftest import TINY_B
    from safetyraise_lmengine_b200.config.registry import architecture_of
    folder, src = _renamed_folder(tmp_path, TINY_B, 4)
    arch = architecture_of(TINY_B)
    raw = WeightFolder(folder)
    assert "model.language_model.layers.2.mlp.down_proj.weight" in set(raw.names()) and "lm_head.weight" in set(raw.names())
    decls = tensor_decls(arch.read_spec(TINY_B))
    with pytest.raises(WeightError):                                 # as stored, nothing matches
        check_against(decls, {n: raw.meta(n)[1] for n in raw.names()})
    seen = arch.source_for(raw)
    check_against(decls, {n: seen.meta(n)[1] for n in seen.names()})
    t = load_tensors(seen, decls, torch.bfloat16, "cpu")
    assert torch.equal(t["model.layers.2.mlp.down_proj.weight"], src.get("model.layers.2.mlp.down_proj.weight"))
    assert torch.equal(t["lm_head.weight"], src.get("lm_head.weight"))
    # a folder under the plain names passes through unchanged
    plain = RandomWeights(decls, 4)
    assert arch.source_for(plain) is plain


def test_stored_types_of_random_folders(tmp_path):
    from conftest import TINY_A
    from safetyraise_lmengine_b200.weights.random_init import write_model_folder
    for store, dt in (("F32", torch.float32), ("F16", torch.float16), ("BF16", torch.bfloat16)):
        folder = write_model_folder(TINY_A, 9, str(tmp_path / store), store=store)
        w = WeightFolder(folder)
        assert w.meta("model.layers.0.mlp.up_proj.weight")[0] == dt
        assert w.meta("model.norm.weight")[0] == torch.float32
    t = load_tensors(WeightFolder(str(tmp_path / "F32")), tensor_decls(spec_from_config(TINY_A)), torch.bfloat16, "cpu")
    m = t["model.layers.0.mlp.up_proj.weight"]
    assert m.dtype == torch.float32 and not torch.equal(m, m.to(torch.bfloat16).float())
    with pytest.raises(ValueError):
        write_model_folder(TINY_A, 9, str(tmp_path / "x"), store="F8")
