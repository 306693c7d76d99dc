"""Loading tensors by name for a model.

A model declares what it needs as ``TensorDecl`` records; ``load_tensors``
checks the whole list against a source in one pass and raises ONE WeightError
that lists every missing tensor, every unexpected tensor and every wrong shape.
Lookup is by exact name and shapes must match exactly, as in the reference
(src/model/native.rs:100-117, src/artifact/mod.rs:126-133).

Storage precision: a float tensor stored in 16 bits is kept in bfloat16 (or
widened to float32 when the engine runs its float32 path); a tensor stored in
32 bits stays in 32 bits; integer tables are int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Sequence, Tuple

import torch

from ..errors import WeightError

MATRIX, VECTOR, TABLE, INT_TABLE = "matrix", "vector", "table", "int_table"


@dataclass(frozen=True)
class TensorDecl:
    name: str
    shape: Tuple[int, ...]
    role: str = MATRIX        # MATRIX | VECTOR (norm scale) | TABLE (embedding rows) | INT_TABLE


def check_against(decls: Sequence[TensorDecl], available: Dict[str, Tuple[int, ...]]) -> None:
    """available: name -> shape.  Raises one error naming everything wrong."""
    wanted = {d.name: d for d in decls}
    missing = [n for n in wanted if n not in available]
    unexpected = [n for n in available if n not in wanted]
    misshaped = [(n, tuple(available[n]), wanted[n].shape) for n in wanted
                 if n in available and tuple(available[n]) != tuple(wanted[n].shape)]
    if not (missing or unexpected or misshaped):
        return
    lines = ["weights do not match the configuration:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if misshaped:
        lines.append(f"  wrong shapes ({len(misshaped)}): " + "; ".join(
            f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in sorted(misshaped)))
    raise WeightError("\n".join(lines))


def device_dtype(stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if stored == torch.int32:
        return torch.int32
    if compute == torch.float32 or stored == torch.float32:
        return torch.float32
    return torch.bfloat16


def load_tensors(source, decls: Sequence[TensorDecl], compute_dtype: torch.dtype,
                 device) -> Dict[str, torch.Tensor]:
    """source: object with names(), meta(name) -> (dtype, shape, nbytes), get(name) -> tensor."""
    names = list(source.names())
    check_against(decls, {n: source.meta(n)[1] for n in names})
    out = {}
    for d in decls:
        t = source.get(d.name)
        if d.role == INT_TABLE:
            if t.dtype != torch.int32:
                raise WeightError(f"tensor {d.name} must be stored as I32, found {t.dtype}")
            out[d.name] = t.to(device)
            continue
        if not t.dtype.is_floating_point:
            raise WeightError(f"tensor {d.name} must be a float tensor, found {t.dtype}")
        if d.role == VECTOR and not bool(torch.isfinite(t.float()).all()):
            raise WeightError(f"tensor {d.name} holds non-finite values")   # src/model/native.rs:111-117
        target = torch.float32 if d.role == VECTOR else device_dtype(t.dtype, compute_dtype)
        out[d.name] = t.to(device=device, dtype=target).contiguous()
    return out


class PrefixedSource:
    """A weight source seen under other names: a stored name that begins with ``stored_prefix`` is
    offered with ``prefix`` in its place; every other name is offered as it is."""

    def __init__(self, source, prefix: str, stored_prefix: str):
        self._source = source
        self._stored = {}
        for n in source.names():
            shown = prefix + n[len(stored_prefix):] if n.startswith(stored_prefix) else n
            if shown in self._stored:
                raise WeightError(f"tensors {self._stored[shown]} and {n} would both be read as {shown}")
            self._stored[shown] = n

    def names(self):
        return self._stored.keys()

    def meta(self, name):
        return self._source.meta(self._stored[name])

    def get(self, name):
        return self._source.get(self._stored[name])


def logical_bytes(source) -> Tuple[int, int]:
    """(tensor count, total stored bytes), as ``inspect`` reports them (src/cli.rs:100-124)."""
    count = total = 0
    for n in source.names():
        total += source.meta(n)[2]
        count += 1
    return count, total
