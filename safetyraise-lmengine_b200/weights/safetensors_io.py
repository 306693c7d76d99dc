"""Reading and writing the safetensors container without a library.

Layout: u64 little-endian header length, a JSON header {name: {dtype, shape,
data_offsets}}, then the raw little-endian bytes.  The checks are those of the
reference's own parser (src/artifact/mod.rs:576-851): header size bound,
duplicate keys, known dtype, non-empty shape without zero extents, offsets in
range and not overlapping, byte length equal to elements times element size;
a folder holds either model.safetensors or model.safetensors.index.json.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

from ..errors import WeightError

MAX_HEADER_BYTES = 64 << 20

_DTYPES = {
    "F32": (torch.float32, np.float32, 4),
    "F16": (torch.float16, np.float16, 2),
    "BF16": (torch.bfloat16, np.uint16, 2),
    "I32": (torch.int32, np.int32, 4),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32"}


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise WeightError(f"safetensors header: duplicate key {k!r}")
        seen[k] = v
    return seen


class SafetensorsFile:
    """One mapped file; ``get(name)`` returns a CPU tensor that views the mapping."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._file = open(path, "rb")
        except OSError as e:
            raise WeightError(f"{path}: {e.strerror}") from None
        size = os.fstat(self._file.fileno()).st_size
        if size < 8:
            raise WeightError(f"{path}: shorter than a safetensors header")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen == 0 or hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise WeightError(f"{path}: header length {hlen} is out of range")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"),
                                object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise WeightError(f"{path}: header must be a JSON object")
        self._base = 8 + hlen
        data_len = size - self._base
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        spans = []
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (lo, hi) = meta["dtype"], tuple(meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise WeightError(f"{path}: malformed entry for tensor {name!r}") from None
            if dtype not in _DTYPES:
                raise WeightError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
            if len(shape) == 0 or any((not isinstance(d, int)) or d <= 0 for d in shape):
                raise WeightError(f"{path}: tensor {name!r} has an empty or zero-sized shape {shape}")
            if not (isinstance(lo, int) and isinstance(hi, int) and 0 <= lo <= hi <= data_len):
                raise WeightError(f"{path}: tensor {name!r} has data offsets out of range")
            count = 1
            for d in shape:
                count *= d
            if hi - lo != count * _DTYPES[dtype][2]:
                raise WeightError(f"{path}: tensor {name!r} holds {hi - lo} bytes, "
                                  f"its shape {shape} needs {count * _DTYPES[dtype][2]}")
            self.entries[name] = (dtype, shape, lo, hi)
            spans.append((lo, hi, name))
        spans.sort()
        for (_, hi0, n0), (lo1, _, n1) in zip(spans, spans[1:]):
            if lo1 < hi0:
                raise WeightError(f"{path}: tensors {n0!r} and {n1!r} overlap")

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def meta(self, name: str):
        dtype, shape, lo, hi = self.entries[name]
        return _DTYPES[dtype][0], shape, hi - lo

    def get(self, name: str) -> torch.Tensor:
        dtype, shape, lo, hi = self.entries[name]
        tdt, ndt, _ = _DTYPES[dtype]
        arr = np.frombuffer(self._map, dtype=ndt, count=(hi - lo) // np.dtype(ndt).itemsize,
                            offset=self._base + lo)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # read-only mapping: tensors are only read
            t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(shape)


class WeightFolder:
    """A model folder: model.safetensors, or the shards of model.safetensors.index.json."""

    def __init__(self, model_dir: str):
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        has_single, has_index = os.path.isfile(single), os.path.isfile(index)
        if has_single and has_index:
            raise WeightError(f"{model_dir}: holds both model.safetensors and an index; which one counts?")
        if not has_single and not has_index:
            raise WeightError(f"{model_dir}: holds neither model.safetensors nor model.safetensors.index.json")
        self._where: Dict[str, SafetensorsFile] = {}
        if has_single:
            f = SafetensorsFile(single)
            for n in f.names():
                self._where[n] = f
            return
        with open(index) as fh:
            try:
                weight_map = json.load(fh, object_pairs_hook=_no_duplicates)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as e:
                raise WeightError(f"{index}: no readable weight_map ({e})") from None
        shards: Dict[str, SafetensorsFile] = {}
        for name, shard in weight_map.items():
            if os.path.isabs(shard) or ".." in shard.split("/"):       # src/artifact/mod.rs:680-696
                raise WeightError(f"{index}: shard path {shard!r} leaves the model folder")
            if shard not in shards:
                shards[shard] = SafetensorsFile(os.path.join(model_dir, shard))
            if name not in shards[shard].entries:
                raise WeightError(f"{index}: tensor {name!r} is not in shard {shard!r}")
            self._where[name] = shards[shard]
        for shard, f in shards.items():
            for n in f.names():
                if weight_map.get(n) != shard:
                    raise WeightError(f"{index}: shard {shard!r} holds tensor {n!r} that the index does not list")

    def names(self):
        return self._where.keys()

    def meta(self, name):
        return self._where[name].meta(name)

    def get(self, name) -> torch.Tensor:
        return self._where[name].get(name)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 \
            else t.view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
