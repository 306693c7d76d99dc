"""Random weights from a configuration and a seed.

Every tensor is a function of (seed, tensor name) alone, so the order of
generation does not matter.  Matrices and embedding tables are N(0, 0.02)
stored as BF16 (or, on request, as F16 or F32: the values are then rounded to
that type only, so most of them are not representable in bfloat16); norm
scales are 1 + N(0, 0.1) stored as F32.  The reference
has only a hand-made test fixture here (src/model/native.rs:322-417); the
distributions are those of the benchmark configurations.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Sequence

import torch

from .loader import INT_TABLE, MATRIX, TABLE, VECTOR, TensorDecl
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


STORAGE = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32}


def random_tensor(decl: TensorDecl, seed: int, device="cpu", matrix_dtype=torch.bfloat16) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, decl.name))
    if decl.role == VECTOR:
        return 1.0 + 0.1 * torch.randn(decl.shape, generator=gen, device=device, dtype=torch.float32)
    if decl.role == INT_TABLE:
        return torch.randint(0, 2 ** 31 - 1, decl.shape, generator=gen, device=device, dtype=torch.int32)
    t = torch.empty(decl.shape, device=device, dtype=matrix_dtype)
    # generated in slabs so that a large table needs no float32 copy of itself
    flat = t.view(-1)
    step = 1 << 26
    for lo in range(0, flat.numel(), step):
        n = min(step, flat.numel() - lo)
        flat[lo:lo + n] = (0.02 * torch.randn(n, generator=gen, device=device, dtype=torch.float32)
                           ).to(matrix_dtype)
    return t


class RandomWeights:
    """A weight source (names/meta/get) that makes tensors on demand, on any device."""

    def __init__(self, decls: Sequence[TensorDecl], seed: int, device="cpu", matrix_dtype=torch.bfloat16):
        self._decls = {d.name: d for d in decls}
        self.seed, self.device, self.matrix_dtype = seed, device, matrix_dtype

    def names(self):
        return self._decls.keys()

    def meta(self, name):
        d = self._decls[name]
        n = 1
        for s in d.shape:
            n *= s
        dt = torch.float32 if d.role == VECTOR else torch.int32 if d.role == INT_TABLE else self.matrix_dtype
        return dt, tuple(d.shape), n * dt.itemsize

    def get(self, name):
        return random_tensor(self._decls[name], self.seed, self.device, self.matrix_dtype)


def write_model_folder(config: dict, seed: int, out_dir: str, store: str = "BF16") -> str:
    """Writes config.json and model.safetensors for ``config`` with random weights; matrices and
    tables are stored as ``store`` (BF16, F16 or F32)."""
    from ..config.registry import architecture_of
    from ..parts.model import tensor_decls
    spec = architecture_of(config).read_spec(config)
    decls = tensor_decls(spec)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    if store not in STORAGE:
        raise ValueError(f"store {store!r}: one of {sorted(STORAGE)}")
    tensors: Dict[str, torch.Tensor] = {d.name: random_tensor(d, seed, matrix_dtype=STORAGE[store]) for d in decls}
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return out_dir
