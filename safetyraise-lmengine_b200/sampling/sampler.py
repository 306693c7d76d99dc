"""Batch sampler over the logits a step returned: one kernel for all rows.

The random draw of a request's i-th generated token is a function of (seed, i)
alone, so the same seed gives the same tokens however the requests were batched,
cut or preempted.  The reference draws from ``rand::StdRng`` seeded per request
(src/frontend/sampling.rs:72-80); its bit stream is not reproduced, its
distribution and order of operations are.
"""
from __future__ import annotations

import os
from typing import List, Sequence

import numpy as np
import torch

from ..kernels import ops
from ..parts.base import FAULT_LOGITS, FAULT_TOKEN, STATUS_WORDS
from .params import SamplingParams

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_for(seed: int, index: int) -> float:
    """A float32 in [0, 1) for the index-th draw of a request with this seed."""
    bits = _splitmix64(_splitmix64(seed & _MASK) ^ ((index + 1) * 0xD1B54A32D192ED03 & _MASK))
    return float(np.float32((bits >> 40) * (1.0 / (1 << 24))))


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


class Sampler:
    """``status``: an engine's status buffer (int32: STATUS_WORDS fault words, then room for one token per
    request).  With it the sampled tokens are written behind the fault words and one read-back
    fetches both; a non-finite logit raises the word FAULT_LOGITS (src/frontend/sampling.rs:97-99).
    Without it the sampler keeps words of its own."""

    def __init__(self, device, vocab_size: int, max_rows: int = 64, status: torch.Tensor = None):
        self.device, self.vocab = device, vocab_size
        self._shared = status is not None
        self._status = status
        if status is None:
            self._status = torch.zeros(STATUS_WORDS + max_rows, dtype=torch.int32, device=device)
        self._words = STATUS_WORDS
        self.bad = self._status[FAULT_LOGITS:FAULT_LOGITS + 1]
        self.last_words = [0] * STATUS_WORDS      # the fault words as the last collect() read them
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, rows: int):
        if rows <= self._cap:
            return
        if self._words + rows > self._status.numel():
            if self._shared:
                raise ValueError(f"{rows} rows to sample exceed the engine's {self._status.numel() - self._words}")
            old = self._status
            self._status = torch.zeros(self._words + rows, dtype=torch.int32, device=self.device)
            self._status[:self._words].copy_(old[:self._words])
            self.bad = self._status[FAULT_LOGITS:FAULT_LOGITS + 1]
        self._cap = rows
        # the rows' parameters go through pinned buffers taken in turn: a launch may be queued while the copy
        # of the launch before it has not run yet; each buffer waits for the event behind its last copy
        self._hosts = [[torch.empty(5 * rows, dtype=torch.float32, pin_memory=True), None] for _ in range(3)]
        self._host_turn = 0
        self._dev = torch.empty(5 * rows, dtype=torch.float32, device=self.device)
        self._out = self._status[self._words:self._words + rows]
        self._scratch = None               # [rows, vocab] float32, made when a row is first sampled
        if not hasattr(self, "_hist_host"):
            self._hist_host = self._hist_dev = None

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int], histories: Sequence[Sequence[int]]) -> List[int]:
        """logits [n, V] float32 on the device; one token id per row, as Python ints."""
        return self.collect(self.launch(logits, params, seeds, indices, histories))

    def collect(self, n) -> List[int]:
        """The tokens of the last launch(): waits for the device and reads them back, the fault words
        with them (``last_words``; the caller decides what a raised word means).  ``n``: the number of
        rows that launch() returned, or what snapshot() returned for them."""
        if isinstance(n, tuple):
            host, event, rows = n
            event.synchronize()
            got = host[:self._words + rows].tolist()
        else:
            got = self._status[:self._words + n].tolist()
        self.last_words = got[:self._words]
        return got[self._words:]

    def snapshot(self, n: int):
        """Copies the fault words and the ``n`` tokens of the last launch() to pinned host memory behind
        what the stream holds so far, so that collect() of the returned handle waits for that copy alone
        and further work may be queued behind it meanwhile (it may overwrite the words and the tokens).
        At most two handles are alive at a time."""
        ring = self.__dict__.setdefault("_snapshots", [])
        need = self._words + self._cap
        if not ring or ring[0].numel() < need:
            ring[:] = [torch.empty(need, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self._snapshot_turn = (getattr(self, "_snapshot_turn", 0) + 1) % len(ring)
        host = ring[self._snapshot_turn]
        host[:self._words + n].copy_(self._status[:self._words + n], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return host, event, n

    def clear_words(self) -> None:
        self._status[:self._words].zero_()
        self.last_words = [0] * self._words

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int], histories: Sequence[Sequence[int]], pending=None) -> int:
        """Starts the sampling kernel for the rows of ``logits``; returns the number of rows.  The host
        does not wait: collect() does.

        pending: per row, None or the row of the launch before this one whose token (still on the device,
        behind the fault words) is the last of this row's history: a repetition penalty counts it, the
        device puts it in place."""
        n = logits.shape[0]
        if n == 0:
            return 0
        self._grow(n)
        if all(p.is_greedy for p in params):
            ops.argmax(logits, self._out[:n], self.bad)
            return n
        self._host_turn = (self._host_turn + 1) % len(self._hosts)
        pair = self._hosts[self._host_turn]
        if pair[1] is not None:
            pair[1].synchronize()
        h = pair[0].numpy()
        c = self._cap
        for i, p in enumerate(params):
            h[i] = p.temperature
            h[c + i] = p.top_p
            h[2 * c + i] = p.repetition_penalty
            h[3 * c + i] = uniform_for(seeds[i], indices[i]) if p.temperature > 0 else 0.0
        h[4 * c:4 * c + n].view(np.int32)[:] = [p.top_k for p in params]
        self._dev.copy_(pair[0], non_blocking=True)
        pair[1] = torch.cuda.Event()
        pair[1].record()
        d = self._dev
        hist = offs = None
        if any(p.repetition_penalty != 1.0 for p in params):
            # ids and row offsets go through one pinned buffer and one asynchronous copy: a pageable
            # copy would make the host wait for the forward that is still running on the device
            late = [pending is not None and pending[i] is not None and p.repetition_penalty != 1.0
                    for i, p in enumerate(params)]
            lens = [len(hh) + late[i] if p.repetition_penalty != 1.0 else 0
                    for i, (p, hh) in enumerate(zip(params, histories))]
            total = sum(lens)
            words = n + 1 + max(total, 1) + 2 * sum(late)            # (the pairs of patch_words ride behind)
            if self._hist_host is None or self._hist_host[0][0].numel() < words:
                cap = max(words, 2 * (self._hist_host[0][0].numel() if self._hist_host is not None else 4096))
                # pinned buffers taken in turn, like the parameters' (a launch may be queued before the copy of
                # the launch ahead of it has run)
                self._hist_host = [[torch.empty(cap, dtype=torch.int32, pin_memory=True), None] for _ in range(3)]
                self._hist_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
                self._hist_turn = 0
            self._hist_turn = (self._hist_turn + 1) % len(self._hist_host)
            hist_pair = self._hist_host[self._hist_turn]
            if hist_pair[1] is not None:
                hist_pair[1].synchronize()
            hh_np = hist_pair[0].numpy()
            hh_np[0] = 0
            np.cumsum(lens, out=hh_np[1:n + 1])
            at = n + 1
            pairs = []
            for i, (ln, hist_ids) in enumerate(zip(lens, histories)):
                if ln:
                    hh_np[at:at + ln - late[i]] = hist_ids
                    if late[i]:
                        hh_np[at + ln - 1] = -1                       # an id the kernel skips, until it is put in place
                        pairs += [at + ln - 1, int(pending[i])]
                    at += ln
            if total == 0:
                hh_np[n + 1] = 0
            ids_end = n + 1 + max(total, 1)
            hh_np[ids_end:ids_end + len(pairs)] = pairs
            self._hist_dev[:words].copy_(hist_pair[0][:words], non_blocking=True)
            hist_pair[1] = torch.cuda.Event()
            hist_pair[1].record()
            if pairs:
                ops.patch_words(self._hist_dev, self._hist_dev[ids_end:ids_end + len(pairs)],
                                self._status[self._words:], len(pairs) // 2, self._status[FAULT_TOKEN:FAULT_TOKEN + 1])
            offs = self._hist_dev[:n + 1]
            hist = self._hist_dev[n + 1:ids_end]
        if self._scratch is None or self._scratch.shape[0] < self._cap:
            self._scratch = torch.empty(self._cap, self.vocab, dtype=torch.float32, device=self.device)
        ops.sample(logits, d[:n], d[4 * c:4 * c + n].view(torch.int32), d[c:c + n], d[2 * c:2 * c + n],
                   d[3 * c:3 * c + n], hist, offs, self._out[:n], self.bad, self._scratch)
        return n
