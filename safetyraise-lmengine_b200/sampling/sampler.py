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
from ..parts.base import FAULT_LOGITS, STATUS_WORDS
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
        self._host = torch.empty(5 * rows, dtype=torch.float32, pin_memory=True)
        self._dev = torch.empty(5 * rows, dtype=torch.float32, device=self.device)
        self._out = self._status[self._words:self._words + rows]
        self._scratch = None               # [rows, vocab] float32, made when a row is first sampled
        if not hasattr(self, "_hist_host"):
            self._hist_host = self._hist_dev = None

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int], histories: Sequence[Sequence[int]]) -> List[int]:
        """logits [n, V] float32 on the device; one token id per row, as Python ints."""
        return self.collect(self.launch(logits, params, seeds, indices, histories))

    def collect(self, n: int) -> List[int]:
        """The tokens of the last launch(): waits for the device and reads them back, the fault words
        with them (``last_words``; the caller decides what a raised word means)."""
        got = self._status[:self._words + n].tolist()
        self.last_words = got[:self._words]
        return got[self._words:]

    def clear_words(self) -> None:
        self._status[:self._words].zero_()
        self.last_words = [0] * self._words

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int], histories: Sequence[Sequence[int]]) -> int:
        """Starts the sampling kernel for the rows of ``logits``; returns the number of rows.  The host
        does not wait: collect() does."""
        n = logits.shape[0]
        if n == 0:
            return 0
        self._grow(n)
        if all(p.is_greedy for p in params):
            ops.argmax(logits, self._out[:n], self.bad)
            return n
        h = self._host.numpy()
        c = self._cap
        for i, p in enumerate(params):
            h[i] = p.temperature
            h[c + i] = p.top_p
            h[2 * c + i] = p.repetition_penalty
            h[3 * c + i] = uniform_for(seeds[i], indices[i]) if p.temperature > 0 else 0.0
        h[4 * c:4 * c + n].view(np.int32)[:] = [p.top_k for p in params]
        # the previous call ended by reading its tokens back, so its copy has left the pinned buffer
        self._dev.copy_(self._host, non_blocking=True)
        d = self._dev
        hist = offs = None
        if any(p.repetition_penalty != 1.0 for p in params):
            # ids and row offsets go through one pinned buffer and one asynchronous copy: a pageable
            # copy would make the host wait for the forward that is still running on the device
            lens = [len(hh) if p.repetition_penalty != 1.0 else 0 for p, hh in zip(params, histories)]
            total = sum(lens)
            words = n + 1 + max(total, 1)
            if self._hist_host is None or self._hist_host.numel() < words:
                cap = max(words, 2 * (self._hist_host.numel() if self._hist_host is not None else 4096))
                self._hist_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
                self._hist_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            hh_np = self._hist_host.numpy()
            hh_np[0] = 0
            np.cumsum(lens, out=hh_np[1:n + 1])
            at = n + 1
            for ln, hist_ids in zip(lens, histories):
                if ln:
                    hh_np[at:at + ln] = hist_ids
                    at += ln
            if total == 0:
                hh_np[n + 1] = 0
            self._hist_dev[:words].copy_(self._hist_host[:words], non_blocking=True)
            offs = self._hist_dev[:n + 1]
            hist = self._hist_dev[n + 1:words]
        if self._scratch is None or self._scratch.shape[0] < self._cap:
            self._scratch = torch.empty(self._cap, self.vocab, dtype=torch.float32, device=self.device)
        ops.sample(logits, d[:n], d[4 * c:4 * c + n].view(torch.int32), d[c:c + n], d[2 * c:2 * c + n],
                   d[3 * c:3 * c + n], hist, offs, self._out[:n], self.bad, self._scratch)
        return n
