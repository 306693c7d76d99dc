"""Python face of the native scheduler (csrc/host/scheduler.cpp) and the request records.

The native scheduler decides: admission, portions under the token budget,
decoding, preemption when pages run out.  This module keeps what it does not:
the token ids, the sampling options, deadlines and the finish reasons
(src/engine/scheduler.rs:185-219).
"""
from __future__ import annotations

import ctypes as C
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..cache.manager import CacheManager, runtime
from ..errors import ConfigError, ResourceExhausted
from ..sampling.params import SamplingParams

FINISH_STOP, FINISH_LENGTH, FINISH_CANCELLED, FINISH_DEADLINE, FINISH_ERROR = (
    "stop", "length", "cancelled", "deadline", "error")

SUBMIT_ERRORS = {
    -1: (ResourceExhausted, "the request queue is full"),
    -2: (ConfigError, "prompt plus max_new_tokens exceeds max_context"),
    -3: (ResourceExhausted, "the request would not fit the cache pool even alone"),
    -4: (ConfigError, "empty prompt, max_new_tokens <= 0, or a request id that is already live"),
}


@dataclass
class GenerationRequest:
    prompt: List[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)
    request_id: Optional[int] = None
    deadline_ms: Optional[int] = None


@dataclass
class Usage:                         # src/engine/scheduler.rs:206-212
    prompt_tokens: int = 0
    completion_tokens: int = 0
    queue_ms: float = 0.0
    elapsed_ms: float = 0.0
    preemptions: int = 0


@dataclass
class RequestState:
    request: GenerationRequest
    tokens: List[int]                 # prompt + generated
    seed: int
    submitted_at: float
    first_step_at: Optional[float] = None
    deadline_at: Optional[float] = None
    cancelled: bool = False
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    usage: Usage = field(default_factory=Usage)

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.usage.prompt_tokens:]


@dataclass
class PlanEntry:
    request_id: int
    slot: int
    start: int
    count: int
    want_logits: bool


class Scheduler:
    def __init__(self, cache: CacheManager, max_active: int, queue_capacity: int, prefill_chunk: int,
                 max_batch_tokens: int, max_context: int):
        self._lib = runtime()
        self._cache = cache                      # keeps the native manager alive
        self._h = self._lib.srlm_sched_create(cache.handle, max_active, queue_capacity, prefill_chunk,
                                              max_batch_tokens, max_context)
        if not self._h:
            raise ConfigError("scheduler options must all be positive")
        self._cap = max(max_active, 1) + 8
        self._entries = (C.c_int64 * (5 * self._cap))()
        self._pre = (C.c_int64 * self._cap)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.srlm_sched_destroy(h)

    def submit(self, request_id: int, prompt_len: int, max_new: int) -> None:
        r = self._lib.srlm_sched_submit(self._h, request_id, prompt_len, max_new)
        if r != 0:
            exc, msg = SUBMIT_ERRORS[r]
            raise exc(f"request {request_id}: {msg}")

    def plan(self) -> Tuple[List[PlanEntry], List[int]]:
        npre = C.c_int(0)
        n = self._lib.srlm_sched_plan(self._h, self._entries, self._cap, self._pre, C.byref(npre))
        e = self._entries
        plan = [PlanEntry(e[5 * i], e[5 * i + 1], e[5 * i + 2], e[5 * i + 3], bool(e[5 * i + 4]))
                for i in range(n)]
        return plan, [self._pre[i] for i in range(npre.value)]

    def advance(self, request_id: int, count: int) -> None:
        r = self._lib.srlm_sched_advance(self._h, request_id, count)
        if r != 0:
            raise ValueError(f"advance({request_id}, {count}) is invalid ({r})")

    def rollback(self, request_id: int) -> None:
        self._lib.srlm_sched_rollback(self._h, request_id)

    def append_token(self, request_id: int) -> int:
        return self._lib.srlm_sched_append_token(self._h, request_id)

    def retract_token(self, request_id: int) -> int:
        """Undoes the last append_token of a request whose token was not fed yet (it was a stop token)."""
        return self._lib.srlm_sched_retract_token(self._h, request_id)

    def finish(self, request_id: int) -> None:
        self._lib.srlm_sched_finish(self._h, request_id)

    def has_work(self) -> bool:
        return bool(self._lib.srlm_sched_has_work(self._h))

    def counters(self) -> Dict[str, int]:
        out = (C.c_int64 * 9)()
        self._lib.srlm_sched_counters(self._h, out)
        names = ("submitted", "rejected", "completed", "preempted", "steps", "batched_tokens",
                 "generated_tokens", "active", "queued")
        return dict(zip(names, out))
