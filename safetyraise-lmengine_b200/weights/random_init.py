"""Random weights from a configuration and a seed.

Every tensor is a function of (seed, tensor name) alone, so the order of
generation does not matter.  Matrices and embedding tables are N(0, 0.02)
stored as BF16; norm scales are 1 + N(0, 0.1) stored as F32.  The reference
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


def random_tensor(decl: TensorDecl, seed: int, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, decl.name))
    if decl.role == VECTOR:
        return 1.0 + 0.1 * torch.randn(decl.shape, generator=gen, device=device, dtype=torch.float32)
    if decl.role == INT_TABLE:
        return torch.randint(0, 2 ** 31 - 1, decl.shape, generator=gen, device=device, dtype=torch.int32)
    t = torch.empty(decl.shape, device=device, dtype=torch.bfloat16)
    # generated in slabs so that a large table needs no float32 copy of itself
    flat = t.view(-1)
    step = 1 << 26
    for lo in range(0, flat.numel(), step):
        n = min(step, flat.numel() - lo)
        flat[lo:lo + n] = (0.02 * torch.randn(n, generator=gen, device=device, dtype=torch.float32)
                           ).to(torch.bfloat16)
    return t


class RandomWeights:
    """A weight source (names/meta/get) that makes tensors on demand, on any device."""

    def __init__(self, decls: Sequence[TensorDecl], seed: int, device="cpu"):
        self._decls = {d.name: d for d in decls}
        self.seed, self.device = seed, device

    def names(self):
        return self._decls.keys()

    def meta(self, name):
        d = self._decls[name]
        n = 1
        for s in d.shape:
            n *= s
        dt = torch.float32 if d.role == VECTOR else torch.int32 if d.role == INT_TABLE else torch.bfloat16
        return dt, tuple(d.shape), n * (2 if dt == torch.bfloat16 else 4)

    def get(self, name):
        return random_tensor(self._decls[name], self.seed, self.device)


def write_model_folder(config: dict, seed: int, out_dir: str) -> str:
    """Writes config.json and model.safetensors for ``config`` with random weights."""
    from ..config.registry import architecture_of
    from ..parts.model import tensor_decls
    spec = architecture_of(config).read_spec(config)
    decls = tensor_decls(spec)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    tensors: Dict[str, torch.Tensor] = {d.name: random_tensor(d, seed) for d in decls}
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return out_dir
