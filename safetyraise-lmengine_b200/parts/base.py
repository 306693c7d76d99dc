"""Interfaces of the parts a model is put together from, and their registries.

A part is built from its own specification (sizes and constants as fields) and
the tensors it declared; it never learns which model it is in.  Five kinds:

* Norm:             ``apply(residual, delta, out, rows=None)``
* PositionEncoding: says how it is applied (``applies``): ``rotation(ctx)`` gives a mixer the step's
                    rotation of q and k; ``add_to_embedding(ctx, residual)`` adds to the embedded tokens
* Mixer:            ``cache_need()``, ``forward(ctx, x, run_step) -> [T, hidden]``
* FeedForward:      ``forward(ctx, x) -> [T, hidden]``
* Block:            ``forward(ctx, residual, pending, run_step, next_block) -> pending`` (see ``Block``)

Each kind has a registry from the ``kind`` string of its specification to the
class; ``register_*`` adds to it, from inside or outside this package.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import Unsupported
from ..weights.loader import TensorDecl

NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}


def _register(table, what):
    def deco(kind: str):
        def wrap(cls):
            table[kind] = cls
            cls.kind = kind
            return cls
        return wrap
    deco.__doc__ = f"Class decorator: registers a {what} under a kind string."
    return deco


register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_block = _register(BLOCKS, "block")


def lookup(table, kind: str, what: str):
    if kind not in table:
        raise Unsupported(f"{what} kind {kind!r} is not registered (registered: {sorted(table)})")
    return table[kind]


@dataclass(frozen=True)
class CacheNeed:
    """What one run step of a mixer needs from the cache manager."""
    kind: str                                 # cache.manager.PAGED_ALL | PAGED_WINDOW | FIXED_STATE | "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: torch.dtype = torch.float32


@dataclass
class ModelContext:
    """What every part of one model instance shares."""
    device: torch.device
    dtype: torch.dtype                        # activation / cache dtype: float32 or bfloat16
    max_batch_tokens: int
    options: dict = field(default_factory=dict)


class Workspace:
    """Named activation buffers, allocated once at their largest size and reused every step."""

    def __init__(self, device, max_tokens: int):
        self.device, self.max_tokens = device, max_tokens
        self._bufs: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}     # (name, width, dtype, rows) -> buf[:rows]: slicing costs 1.5 us
        self.generation = 0      # grows whenever a buffer moves: recorded CUDA graphs are stale then

    def get(self, name: str, rows: int, width: int, dtype: torch.dtype, reserve=None) -> torch.Tensor:
        """A [rows, width] view of the buffer ``name``; the buffer is made for ``reserve`` rows
        (default: the most tokens a step may hold) and grows if a step ever needs more."""
        view = self._views.get((name, width, dtype, rows))
        if view is not None:
            return view
        key = (name, width, dtype)
        buf = self._bufs.get(key)
        cap = max(rows, self.max_tokens if reserve is None else reserve, 1)
        if buf is None or buf.shape[0] < rows:
            if buf is not None:
                self.generation += 1
                self._views = {k: v for k, v in self._views.items() if k[:3] != key}
            buf = torch.empty((cap, width), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[(name, width, dtype, rows)] = buf[:rows]
        return view


# Words of a step's status buffer (int32, on the device; zero = fine).  The engine reads them back
# with the step's result and fails the step if one is set.
FAULT_WAIT, FAULT_TOKEN, FAULT_ACTIVATION, FAULT_LOGITS = 0, 1, 2, 3
STATUS_WORDS = 8
FAULT_NAMES = {FAULT_WAIT: "a kernel gave up on a bounded wait",
               FAULT_TOKEN: "a token id outside the embedding table",
               FAULT_ACTIVATION: "a non-finite activation",
               FAULT_LOGITS: "a non-finite logit"}


@dataclass
class StepContext:
    """The ragged batch of one step, flattened, on the device.

    Entry e feeds q_lens[e] tokens of the request in slot slots[e], at positions
    starts[e] .. starts[e]+q_lens[e]-1.  Paged groups add a block table per entry
    and, for every token, the flat cache row it is written to.
    """
    T: int
    n_entries: int
    token_ids: torch.Tensor                   # int32 [T]
    positions: torch.Tensor                   # int32 [T]
    entry_of_token: torch.Tensor              # int32 [T]
    slots: torch.Tensor                       # int32 [n_entries]
    cu_q: torch.Tensor                        # int32 [n_entries + 1]
    kv_lens: torch.Tensor                     # int32 [n_entries] (after this step)
    logit_rows: torch.Tensor                  # int32 [R]
    block_tables: Dict[str, torch.Tensor]     # group -> int32 [n_entries, pages]
    kv_slot: Dict[str, torch.Tensor]          # group -> int32 [T]
    host: dict                                # the same as Python lists, for parts that plan on the host
    cache: "object"
    workspace: Workspace
    dtype: torch.dtype
    tables: dict = field(default_factory=dict)    # position-encoding tables of this step
    max_q_len: int = 1
    max_kv_len: int = 1
    kv_bound: int = 1                         # an upper bound of max_kv_len that kernels may size their grids by
    options: dict = field(default_factory=dict)   # the engine's options, for parts that have switches
    status: Optional[torch.Tensor] = None     # int32 [STATUS_WORDS]: the step's fault words (None: the model's own)


@dataclass
class Rotation:
    """How a rotary position encoding turns the q and k heads of this step's tokens: the first
    2 * pairs elements of a head are rotated pair by pair, pair i by the angle whose cosine and sine
    are cos[t, i] and sin[t, i]; the rest of the head passes unchanged (a rotary fraction below one).
    The partners of pair i are the elements (i, i + pairs), or (2i, 2i + 1) when interleaved."""
    cos: torch.Tensor            # float32 [T, pairs]
    sin: torch.Tensor
    pairs: int
    interleaved: bool = False


ROTATION, EMBEDDING = "rotation", "embedding"      # PositionEncoding.applies


@dataclass
class NormedInput:
    """An activation on its way into a part, normalised lazily.

    ``xw`` holds residual * norm weight in the activation dtype.  If ``ss_parts`` is None it is already
    divided by its RMS (a plain normalised tensor).  Otherwise ``ss_parts`` [parts, 8] holds partial sums
    of squares of each token's residual row, and whoever consumes ``xw`` with a linear map scales the
    map's output by rsqrt(sum / width + eps) per token instead.  Produced by the epilogue of the product
    that wrote the residual, consumed by the first product of the next part: the norm kernel between
    the two disappears.
    """
    xw: torch.Tensor
    ss_parts: Optional[torch.Tensor]
    width: int
    eps: float


class Part:
    """Common behaviour: a part declares its tensors before it is built.

    A position encoding also says where it acts, in the class attribute ``applies``:
    ROTATION -- mixers call ``rotation(ctx) -> Rotation`` and turn q and k with it;
    EMBEDDING -- the model calls ``add_to_embedding(ctx, residual)`` once, after the token rows are
    gathered into the float32 residual stream (absolute and learned encodings).  An encoding that
    acts on the attention scores would need mixers whose kernels take a bias: none here does, and
    the attention part refuses such an encoding when it is built."""

    # Whether the kernels a forward launches depend on the step's device tensors only (block tables,
    # positions, slots), not on its host lists.  Decode-only steps of a model whose parts all say so
    # are recorded into CUDA graphs and replayed; a part that loops over ``ctx.host`` or branches on
    # values of the step sets this to False and its model always runs eagerly.
    replayable = True

    @classmethod
    def tensor_decls(cls, spec, prefix: str) -> List[TensorDecl]:
        return []

    # A mixer says what it needs from the cache manager from its specification alone, so that the
    # needs of a model are known before any weight is read (``inspect``, admission arithmetic).
    @classmethod
    def cache_need_of(cls, spec) -> "CacheNeed":
        return CacheNeed("none")

    def cache_need(self) -> "CacheNeed":
        return type(self).cache_need_of(self.spec)


class Block(Part):
    """One layer: an arrangement of norms, a mixer and a feed-forward around the float32 residual stream.

    ``forward(ctx, residual, pending, run_step, next_block) -> pending``.  ``residual`` [T, hidden] float32
    is updated in place.  ``pending`` is what the block before left behind: None, a tensor still to be
    added to the residual (the next norm kernel adds it while it norms), or a ``NormedInput`` -- the input
    of this block's first part, already prepared by the product that wrote the residual.  A block may
    hand its successor such a prepared input only if the successor says it takes one for this step:
    ``next_block.prepared_input_norm(ctx)`` returns the norm whose weight the input must carry, or None
    (the default: the successor wants a plain pending tensor).  ``next_block`` is None behind the last
    block; what the last block returns goes to the final norm, so it must be a tensor or None."""

    def prepared_input_norm(self, ctx):
        return None

    def forward(self, ctx, residual, pending, run_step, next_block=None):
        raise NotImplementedError
