"""The step function: one ragged batch through the model, from the cache.

``Engine.step(entries)`` takes, for each request in the batch, the request's
slot, its next tokens and the places among them whose logits are wanted.
Portions of prompts stand beside single decoded tokens, cut anywhere.  It
checks everything on the host first (a refused step launches nothing and
changes nothing), reserves pages, runs only the given tokens as one batch, and
commits the new lengths.  It returns float32 logits [wanted, vocab] in the
order of the entries and of their ``want`` lists.

Counterpart of NativeModel::forward (src/model/native.rs:231-312), which takes
one request at a time; batching several requests into one forward is this
engine's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.registry import architecture_of, read_config_json
from ..errors import ConfigError, ResourceExhausted, ShapeError, StepFailed, Unavailable
from ..parts.base import (FAULT_LOGITS, FAULT_NAMES, FAULT_TOKEN, STATUS_WORDS, ModelContext, StepContext,
                          Workspace)
from ..weights.safetensors_io import WeightFolder

DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16,
          "bf16": torch.bfloat16}


LATER = -1      # a token id that is filled in between prepare() and run()


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]             # LATER for an id that PreparedStep.set_token supplies before run()
    want: Sequence[int] = ()          # indices into ``tokens`` whose logits are returned
    generation: Optional[int] = None  # the slot's generation when the request opened it (``Engine.generation``);
                                      # given, a step refuses a slot that another request holds by now


@dataclass
class PreparedStep:
    """A step whose host work is done: checked, pages reserved, the batch laid out in a pinned buffer.
    Nothing has been copied to the device or launched yet."""
    entries: Sequence[StepEntry]
    starts: List[int]
    q_lens: List[int]
    kv_lens: List[int]
    sections: dict
    words: int
    pair: list                        # [pinned host buffer, event of its last copy]
    pages: int
    wanted: int
    token_at: List[int]               # offset of each entry's first token id in the buffer
    missing: int                      # token ids still to be set
    state_snapshot: Optional[dict] = None   # fixed-size state of the step's slots before the forward
    host: Optional[np.ndarray] = None       # the pinned buffer as an array (made once: set_token is called per token)

    def set_token(self, entry: int, index: int, token: int) -> None:
        h = self.host if self.host is not None else self.pair[0].numpy()
        at = self.token_at[entry] + index
        if h[at] == LATER:
            self.missing -= 1
        h[at] = token


def _round_up(a: int, b: int) -> int:
    return (a + b - 1) // b * b


class Engine:
    """A model, its cache and its workspace on one GPU."""

    def __init__(self, model, cache: CacheManager, mctx: ModelContext, max_context: int):
        self.model, self.cache, self.mctx = model, cache, mctx
        self.spec = model.spec
        self.max_context = min(max_context, self.spec.max_position_embeddings)
        self.workspace = Workspace(mctx.device, mctx.max_batch_tokens)
        self.max_pages_per_request = (self.max_context + cache.page_size - 1) // cache.page_size
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_hosts: list = []          # ring of pinned buffers, each with the event of its last copy
        self._meta_turn = 0
        self.steps_run = 0
        # decode-only steps (one token per entry) are recorded into CUDA graphs, one per
        # (batch size, wanted rows, block-table width); the second step of a kind records, later ones replay
        self.use_graphs = bool(mctx.options.get("cuda_graphs", True)) and getattr(model, "replayable", True)
        self._graphs: Dict[tuple, tuple] = {}
        self._graph_seen: set = set()
        self.graph_replays = 0
        self._graph_generation = 0
        self.last_h2d_bytes = 0          # bytes of batch layout the last step copied to the device
        # fault words of a step (parts.base.FAULT_*), then room for one sampled token per request: a
        # sampler bound to this buffer brings both back in one read
        self.status = torch.zeros(STATUS_WORDS + cache.max_requests, dtype=torch.int32, device=mctx.device)
        self._slot_generation = [0] * cache.max_requests    # the generation of each slot this engine last saw
        self.steps_failed = 0

    # ---- construction -----------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", **kw) -> "Engine":
        config = read_config_json(model_dir)
        return cls.from_source(config, WeightFolder(model_dir), dtype=dtype, **kw)

    @classmethod
    def from_source(cls, config: dict, source, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                    num_pages: Optional[int] = None, max_requests: int = 64,
                    max_batch_tokens: int = 2048, max_context: Optional[int] = None,
                    options: Optional[dict] = None) -> "Engine":
        if not torch.cuda.is_available():
            raise Unavailable("no CUDA device: this engine has no CPU path")
        tdtype = DTYPES.get(dtype, dtype)
        if tdtype not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"dtype {dtype!r}: float32 or bfloat16")
        arch = architecture_of(config)
        spec = arch.read_spec(config)
        source = arch.source_for(source)
        device = torch.device(device)
        mctx = ModelContext(device, tdtype, max_batch_tokens, dict(options or {}))
        with torch.cuda.device(device):
            model = arch.build_model(spec, mctx, source)
            max_context = min(max_context or spec.max_position_embeddings, spec.max_position_embeddings)
            groups = model.cache_groups()
            if num_pages is None:
                per_page = max(1, sum(g.bytes_per_token(tdtype) for g in groups) * page_size)
                free, _ = torch.cuda.mem_get_info(device)
                num_pages = max(1, min(int(free * 0.8) // per_page,
                                       max_requests * ((max_context + page_size - 1) // page_size)))
            cache = CacheManager(groups, page_size, num_pages, max_requests, tdtype, device)
        return cls(model, cache, mctx, max_context)

    # ---- requests ---------------------------------------------------------
    def open_request(self) -> int:
        return self.cache.open_request()

    def generation(self, slot: int) -> int:
        """Grows each time the slot is opened; a StepEntry that carries it is refused once the slot has
        passed to another request (the owner test of src/model/native.rs:259-261)."""
        return self.cache.generation(slot)

    def close_request(self, slot: int) -> None:
        self.cache.close_request(slot)

    # ---- the step -------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]):
        if not entries:
            raise ShapeError("a step needs at least one entry")
        seen = set()
        total = 0
        vocab = self.spec.vocab_size
        for e in entries:
            if e.slot in seen:
                raise ShapeError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise ShapeError("an entry without tokens")
            start = self.cache.length(e.slot)
            if start < 0:
                raise ShapeError(f"slot {e.slot} is not open")
            if e.generation is not None and e.generation != self.cache.generation(e.slot):
                raise ShapeError(f"slot {e.slot} was given to another request since this one opened it "
                                 f"(generation {self.cache.generation(e.slot)}, the entry holds {e.generation})")
            if start + n > self.max_context:
                raise ShapeError(f"slot {e.slot}: {start}+{n} tokens exceed the context of {self.max_context}")
            if n == 1:                               # a decoded token: no array for one number
                t = int(e.tokens[0])
                if not (0 <= t < vocab or t == LATER):
                    raise ShapeError(f"token id {t} is outside the vocabulary of {vocab}")
            else:
                ids = np.asarray(e.tokens, dtype=np.int64)
                wrong = ((ids < 0) | (ids >= vocab)) & (ids != LATER)
                if wrong.any():
                    raise ShapeError(f"token id {int(ids[wrong][0])} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ShapeError(f"wanted place {w} is outside the entry's {n} tokens")
            total += n
        if total > self.mctx.max_batch_tokens:
            raise ShapeError(f"{total} tokens in one step exceed max_batch_tokens={self.mctx.max_batch_tokens}")

    def _meta_buffers(self, words: int):
        """A pinned host buffer that no copy in flight still reads, and the device buffer."""
        if self._meta_dev is None or self._meta_dev.numel() < words:
            cap = max(words, 4 * self.mctx.max_batch_tokens + 64 * (self.max_pages_per_request + 8) + 1024)
            torch.cuda.synchronize(self.mctx.device)
            self._graphs.clear()                      # they point into the old buffer
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.mctx.device)
            self._meta_hosts = [[torch.empty(cap, dtype=torch.int32, pin_memory=True), None]
                                for _ in range(4)]
        self._meta_turn = (self._meta_turn + 1) % len(self._meta_hosts)
        pair = self._meta_hosts[self._meta_turn]
        if pair[1] is not None:
            pair[1].synchronize()
        return pair, self._meta_dev

    def _lay_out(self, entries: Sequence[StepEntry], starts: List[int]) -> PreparedStep:
        """Flattens the batch into a pinned host buffer (no device work)."""
        n = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        groups = self.cache.paged_groups
        ps = self.cache.page_size
        kv_lens = [s + q for s, q in zip(starts, q_lens)]
        # decode-only steps round the table width coarsely: its value is part of a graph's identity
        decode_only = max(q_lens) == 1
        pages = _round_up(max(1, max((l + ps - 1) // ps for l in kv_lens)), 16 if decode_only else 8)
        R = sum(len(e.want) for e in entries)
        # layout, in int32 words; every section starts on a 16-byte boundary
        sections, off = {}, 0
        def place(name, count):
            nonlocal off
            sections[name] = (off, count)
            off = _round_up(off + count, 4)
        for name in ("token_ids", "positions", "entry_of_token"):
            place(name, T)
        for g in groups:
            place("kv_slot:" + g.name, T)
        place("slots", n)
        place("cu_q", n + 1)
        place("kv_lens", n)
        place("logit_rows", R)
        for g in groups:
            place("table:" + g.name, n * pages)
        pair, _ = self._meta_buffers(off)
        h = pair[0].numpy()
        view = lambda name: h[sections[name][0]:sections[name][0] + sections[name][1]]
        tok, posv, eot = view("token_ids"), view("positions"), view("entry_of_token")
        cu = view("cu_q")
        rows = view("logit_rows")
        cu[0] = 0
        t0 = r0 = 0
        token_at, missing = [], 0
        slot_views = [(view("kv_slot:" + g.name), view("table:" + g.name), g.name) for g in groups]
        for i, e in enumerate(entries):
            q = q_lens[i]
            token_at.append(sections["token_ids"][0] + t0)
            if q == 1:                               # a decoded token: plain numbers
                t = int(e.tokens[0])
                missing += t == LATER
                tok[t0] = t
                posv[t0] = starts[i]
                eot[t0] = i
            else:
                ids = np.asarray(e.tokens, dtype=np.int32)
                missing += int((ids == LATER).sum())
                tok[t0:t0 + q] = ids
                posv[t0:t0 + q] = np.arange(starts[i], starts[i] + q, dtype=np.int32)
                eot[t0:t0 + q] = i
            for w in e.want:
                rows[r0] = t0 + int(w)
                r0 += 1
            for kvs, tabs, name in slot_views:
                tv = tabs[i * pages:(i + 1) * pages]
                held = self.cache.table_into(name, e.slot, tv)      # the block table, straight into its row
                if held > pages:
                    raise ShapeError(f"slot {e.slot} holds {held} pages, the step laid out {pages}")
                tv[held:] = 0
                if q == 1:
                    p = starts[i]
                    kvs[t0] = int(tv[p // ps]) * ps + p % ps
                else:
                    p = posv[t0:t0 + q]
                    kvs[t0:t0 + q] = tv[p // ps] * ps + p % ps
            t0 += q
            cu[i + 1] = t0
        view("slots")[:] = [e.slot for e in entries]
        view("kv_lens")[:] = kv_lens
        return PreparedStep(entries=entries, starts=starts, q_lens=q_lens, kv_lens=kv_lens, sections=sections,
                            words=off, pair=pair, pages=pages, wanted=R, token_at=token_at, missing=missing, host=h)

    def _upload(self, prep: PreparedStep) -> StepContext:
        """Copies the laid-out batch to the device in one copy and returns the device views."""
        sections, off, pair = prep.sections, prep.words, prep.pair
        dev = self._meta_dev
        dev[:off].copy_(pair[0][:off], non_blocking=True)
        self.last_h2d_bytes = off * 4
        pair[1] = torch.cuda.Event()
        pair[1].record()
        groups = self.cache.paged_groups
        n, pages = len(prep.entries), prep.pages
        d = lambda name: dev[sections[name][0]:sections[name][0] + sections[name][1]]
        return StepContext(
            T=sum(prep.q_lens), n_entries=n, token_ids=d("token_ids"), positions=d("positions"),
            entry_of_token=d("entry_of_token"), slots=d("slots"), cu_q=d("cu_q"), kv_lens=d("kv_lens"),
            logit_rows=d("logit_rows"),
            block_tables={g.name: d("table:" + g.name).view(n, pages) for g in groups},
            kv_slot={g.name: d("kv_slot:" + g.name) for g in groups},
            host={"q_lens": prep.q_lens, "starts": prep.starts, "kv_lens": prep.kv_lens,
                  "slots": [e.slot for e in prep.entries]},
            cache=self.cache, workspace=self.workspace, dtype=self.mctx.dtype,
            max_q_len=max(prep.q_lens), max_kv_len=max(prep.kv_lens), kv_bound=pages * self.cache.page_size,
            options=self.mctx.options, status=self.status[:STATUS_WORDS])

    def build_context(self, entries: Sequence[StepEntry], starts: List[int]) -> StepContext:
        """Flattens the batch, uploads it in one copy and returns the device views."""
        return self._upload(self._lay_out(entries, starts))

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        """Runs the model on the batch: eagerly, or by replaying the CUDA graph of this kind of step."""
        from ..kernels import ops
        if not self.use_graphs or ctx.max_q_len != 1:
            return self.model.forward(ctx)
        if self._graph_generation != self.workspace.generation:   # a buffer moved since recording
            self._graphs.clear()
            self._graph_generation = self.workspace.generation
        key = (ctx.T, ctx.n_entries, int(ctx.logit_rows.shape[0]), ctx.kv_bound)
        hit = self._graphs.get(key)
        if hit is None:
            if key not in self._graph_seen:           # first time: run eagerly (this also sizes every buffer)
                self._graph_seen.add(key)
                return self.model.forward(ctx)
            if len(self._graphs) >= 64:
                self._graphs.clear()
            graph = torch.cuda.CUDAGraph()
            before = ops.launches
            torch.cuda.synchronize(self.mctx.device)
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
            hit = self._graphs[key] = (graph, logits, ops.launches - before)
            ops.launches = before
        graph, logits, launches = hit
        graph.replay()
        ops.launches += launches
        self.graph_replays += 1
        return logits

    def prepare(self, entries: Sequence[StepEntry]) -> PreparedStep:
        """The host half of a step: checks, page reservation, batch layout.  Token ids given as LATER
        may be supplied afterwards (``PreparedStep.set_token``).  Between prepare() and run() or
        discard() of a step no other step may be prepared or run."""
        self._validate(entries)
        starts = [self.cache.length(e.slot) for e in entries]
        self._greet_new_occupants(entries)
        done = []
        for e, s in zip(entries, starts):
            if not self.cache.reserve(e.slot, s + len(e.tokens)):
                for e2, s2 in done:                     # give back what this step took
                    self.cache.truncate(e2.slot, s2)
                raise ResourceExhausted(f"no free cache pages for slot {e.slot} "
                                        f"({s}+{len(e.tokens)} tokens); nothing was run")
            done.append((e, s))
        try:
            with torch.cuda.device(self.mctx.device):
                return self._lay_out(entries, starts)
        except Exception:
            self.discard_reservation(entries, starts)
            raise

    def _greet_new_occupants(self, entries) -> None:
        """A slot that changed hands since this engine last ran it starts from a zero fixed-size state,
        whoever opened it (this engine, or the scheduler when it admits or re-admits a request)."""
        for e in entries:
            g = self.cache.generation(e.slot)
            if g != self._slot_generation[e.slot]:
                self._slot_generation[e.slot] = g
                for pool in self.cache.state_pools.values():
                    pool[:, e.slot].zero_()

    def discard_reservation(self, entries, starts) -> None:
        for e, s in zip(entries, starts):
            self.cache.truncate(e.slot, s)

    def discard(self, prep: PreparedStep) -> None:
        """Gives back what a prepared step reserved; nothing of it ran."""
        self.discard_reservation(prep.entries, prep.starts)

    def launch(self, prep: PreparedStep, patch: Optional[Sequence[tuple]] = None) -> torch.Tensor:
        """The device half without its book-keeping: one copy of the layout, then the forward.  The
        lengths do not move; ``commit`` or ``revoke`` must follow.

        patch: token ids left open as LATER that the device fills in itself, as (entry, index, row) --
        token ``index`` of entry ``entry`` is the token that the sampler bound to this engine's status
        buffer wrote for its row ``row`` (the step before this one, which the host has not read yet)."""
        patch = list(patch or ())
        if prep.missing != len(patch):
            self.discard(prep)
            raise ShapeError(f"{prep.missing} token ids of the prepared step were never set "
                             f"({len(patch)} are taken on the device)")
        try:
            with torch.cuda.device(self.mctx.device):
                from ..kernels import ops
                ops.bind_error_flag(self.status[:1])
                if patch:
                    # the pairs (word of the token id, sampler row) ride behind the layout in the same copy
                    at = _round_up(prep.words, 4)
                    h = prep.host if prep.host is not None else prep.pair[0].numpy()
                    if at + 2 * len(patch) > h.shape[0]:
                        raise ShapeError("the step's layout leaves no room for the token pairs")
                    for k, (entry, index, row) in enumerate(patch):
                        word = prep.token_at[entry] + index
                        if h[word] != LATER or not 0 <= row < self.cache.max_requests:
                            raise ShapeError(f"token {index} of entry {entry} is not open, or row {row} does not exist")
                        h[at + 2 * k], h[at + 2 * k + 1] = word, row
                    layout_words, prep.words = prep.words, at + 2 * len(patch)
                ctx = self._upload(prep)
                if patch:
                    prep.words = layout_words
                    ops.patch_words(self._meta_dev, self._meta_dev[at:at + 2 * len(patch)],
                                    self.status[STATUS_WORDS:], len(patch), self.status[FAULT_TOKEN:FAULT_TOKEN + 1])
                if self.cache.state_pools:
                    # fixed-size state cannot be truncated: keep what the step's slots held
                    # (src/engine/state.rs:222-224 clones the whole state for the same reason)
                    idx = ctx.slots.long()
                    prep.state_snapshot = {name: (idx, pool.index_select(1, idx))
                                           for name, pool in self.cache.state_pools.items()}
                return self._forward(ctx)
        except Exception:
            self.discard(prep)
            raise

    def commit(self, prep: PreparedStep) -> None:
        for e, s in zip(prep.entries, prep.starts):
            self.cache.commit(e.slot, s + len(e.tokens))
        self.steps_run += 1

    def revoke(self, prep: PreparedStep) -> None:
        """Takes a launched step back: the fixed-size state of its slots as it was, lengths and pages as
        before the step.  (After ``commit`` a window group may already have let go of pages the old
        length needs; such a request can only be closed, which is what the generation loop does.)"""
        with torch.cuda.device(self.mctx.device):
            for name, (idx, saved) in (prep.state_snapshot or {}).items():
                self.cache.state_pools[name].index_copy_(1, idx, saved)
        prep.state_snapshot = None
        for e, s in zip(prep.entries, prep.starts):
            try:
                self.cache.truncate(e.slot, s)
            except ValueError:
                pass

    def read_faults(self):
        """The fault words, read from the device (waits for it)."""
        return self.status[:STATUS_WORDS].tolist()

    def fault_of(self, words) -> Optional[StepFailed]:
        """None if no word is raised; else the error of the failed step, with the words cleared on
        the device and every recorded graph kept (they write into the same words)."""
        if not any(words):
            return None
        self.status[:STATUS_WORDS].zero_()
        self.steps_failed += 1
        what = [f"{FAULT_NAMES.get(i, 'fault word %d' % i)} ({w})" for i, w in enumerate(words) if w]
        return StepFailed("the step failed and nothing of it was kept: " + "; ".join(what), words)

    def run(self, prep: PreparedStep, patch: Optional[Sequence[tuple]] = None) -> torch.Tensor:
        """The device half for a caller that reads the step's fault words itself, together with what
        it reads back anyway (the generation loop: ``Sampler.collect``): launches, advances the
        lengths at once so that the next step can be laid out while this one runs, and returns.
        A raised word then means ``revoke``.  patch: see ``launch``."""
        logits = self.launch(prep, patch)
        self.commit(prep)
        return logits

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one batch; returns float32 logits [wanted, vocab] (valid until the next step).
        The lengths advance only after the step's fault words read clean; otherwise everything is
        taken back and StepFailed is raised (src/model/native.rs:272-306)."""
        prep = self.prepare(entries)
        logits = self.launch(prep)
        with torch.cuda.device(self.mctx.device):
            from ..kernels import ops
            if logits.shape[0]:
                ops.check_finite(logits, None, self.status[FAULT_LOGITS:FAULT_LOGITS + 1])
        fault = self.fault_of(self.read_faults())
        if fault is not None:
            self.revoke(prep)
            raise fault
        self.commit(prep)
        return logits
