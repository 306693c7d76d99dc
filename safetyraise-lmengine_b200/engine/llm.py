"""The Python entry point: load a model, submit requests of token ids, get token ids.

``LLM`` ties the step function, the scheduler and the sampler together the way
the reference's Engine ties its worker loop (src/engine/scheduler.rs:319-488,
830-940).  ``EngineConfig`` keeps the reference's option names where it has
them (src/engine/scheduler.rs:27-61) and adds the ones a paged, batched engine
needs.
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from ..errors import ConfigError, EngineError, ResourceExhausted
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, fresh_seed
from .scheduler import (FINISH_CANCELLED, FINISH_DEADLINE, FINISH_ERROR, FINISH_LENGTH, FINISH_STOP,
                        GenerationRequest, RequestState, Scheduler, Usage)
from .step import LATER, Engine, StepEntry


@dataclass
class EngineConfig:
    # names of the reference's EngineConfig
    max_context: int = 4096
    max_active: int = 8
    queue_capacity: int = 8
    prefill_chunk: int = 2048              # tokens of a prompt per step: large portions run the tensor cores
                                           # best (2,048 tokens: 26 ms; four portions of 512: 38 ms on
                                           # B200); smaller ones let decoding requests step more often
    max_request_ms: int = 300_000
    # this engine's own
    max_batch_tokens: int = 2048
    page_size: int = 16
    num_pages: Optional[int] = None        # None: sized from free device memory
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    plan_ahead: bool = True                # the next decode step's host work runs while the device works
    launch_ahead: bool = True              # ... and the step itself is queued before this one's tokens are read

    def validate(self) -> None:            # src/engine/scheduler.rs:124-141
        for name in ("max_context", "max_active", "queue_capacity", "prefill_chunk", "max_request_ms",
                     "max_batch_tokens", "page_size"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive")
        if self.max_active > 1024 or self.queue_capacity > 65536:
            raise ConfigError("max_active <= 1024 and queue_capacity <= 65536")
        if self.num_pages is not None and self.num_pages <= 0:
            raise ConfigError("num_pages must be positive")

    @classmethod
    def from_dict(cls, d: dict) -> "EngineConfig":
        unknown = set(d) - set(cls.__dataclass_fields__)
        if unknown:                        # unknown fields are refused, as serde(deny_unknown_fields) does
            raise ConfigError(f"unknown engine option(s): {sorted(unknown)}")
        return cls(**d)


@dataclass
class GenerationResult:
    request_id: int
    tokens: List[int]
    finish_reason: str
    usage: Usage
    error: Optional[str] = None


class LLM:
    def __init__(self, engine: Engine, config: EngineConfig):
        config.validate()
        self.engine, self.config = engine, config
        self.scheduler = Scheduler(engine.cache, config.max_active, config.queue_capacity,
                                   config.prefill_chunk, config.max_batch_tokens,
                                   min(config.max_context, engine.max_context))
        self.sampler = Sampler(engine.mctx.device, engine.spec.vocab_size,
                               min(config.max_active, engine.cache.max_requests), status=engine.status)
        self.eos = set(engine.spec.eos_token_ids)
        self._live: Dict[int, RequestState] = {}
        self._done: Dict[int, RequestState] = {}
        self._ids = itertools.count(1)
        self.failed = self.cancelled = 0
        self._prepared = None          # (plan, PreparedStep, open token places) of a step laid out ahead
        self._inflight = None          # (plan, PreparedStep, sampler rows) of a step queued on the device ahead
        self.steps_ahead = 0           # steps that were queued on the device before the step ahead of them was read
        self.steps_dropped = 0         # ... and those of them that were taken back (a stop token, a fault, a cancel)
        self.last_step: Optional[dict] = None   # what the last step ran: {"starts": [...], "counts": [...]} per entry

    # ---- construction ---------------------------------------------------------
    @classmethod
    def from_folder(cls, model_path: str, config: Optional[EngineConfig] = None, **overrides) -> "LLM":
        config = config or EngineConfig()
        for k, v in overrides.items():
            if k not in EngineConfig.__dataclass_fields__:
                raise ConfigError(f"unknown engine option {k!r}")
            setattr(config, k, v)
        config.validate()
        engine = Engine.from_folder(model_path, dtype=config.dtype, device=config.device,
                                    page_size=config.page_size, num_pages=config.num_pages,
                                    max_requests=config.max_active, max_batch_tokens=config.max_batch_tokens,
                                    max_context=config.max_context)
        return cls(engine, config)

    @classmethod
    def from_source(cls, config_json: dict, source, config: Optional[EngineConfig] = None) -> "LLM":
        """A model from its config.json (as a dict) and any weight source, for instance
        ``weights.random_init.RandomWeights``: the random-weights mode."""
        config = config or EngineConfig()
        config.validate()
        engine = Engine.from_source(config_json, source, dtype=config.dtype, device=config.device,
                                    page_size=config.page_size, num_pages=config.num_pages,
                                    max_requests=config.max_active, max_batch_tokens=config.max_batch_tokens,
                                    max_context=config.max_context)
        return cls(engine, config)

    # ---- requests -----------------------------------------------------------------
    def submit(self, request: GenerationRequest) -> int:
        """Admission checks of the reference's submit (src/engine/scheduler.rs:389-487)."""
        request.sampling.validate()
        vocab = self.engine.spec.vocab_size
        if not request.prompt:
            raise ConfigError("the prompt holds no tokens")
        for t in request.prompt:
            if not 0 <= int(t) < vocab:
                raise ConfigError(f"prompt token {t} is outside the vocabulary of {vocab}")
        deadline = request.deadline_ms if request.deadline_ms is not None else self.config.max_request_ms
        if not 0 < deadline <= self.config.max_request_ms:
            raise ConfigError(f"deadline_ms must lie in (0, {self.config.max_request_ms}]")
        rid = request.request_id if request.request_id is not None else next(self._ids)
        self.scheduler.submit(rid, len(request.prompt), request.sampling.max_new_tokens)
        now = time.monotonic()
        seed = request.sampling.seed if request.sampling.seed is not None else fresh_seed()
        self._live[rid] = RequestState(request, [int(t) for t in request.prompt], seed, now,
                                       deadline_at=now + deadline / 1000.0,
                                       usage=Usage(prompt_tokens=len(request.prompt)))
        return rid

    def cancel(self, request_id: int) -> None:
        st = self._live.get(request_id)
        if st is not None:
            st.cancelled = True

    def _finish(self, rid: int, reason: str, error: Optional[str] = None) -> None:
        st = self._live.pop(rid)
        self.scheduler.finish(rid)
        st.finish_reason, st.error = reason, error
        st.usage.completion_tokens = len(st.tokens) - st.usage.prompt_tokens
        st.usage.elapsed_ms = (time.monotonic() - st.submitted_at) * 1000.0
        if reason == FINISH_ERROR:
            self.failed += 1
        if reason in (FINISH_CANCELLED, FINISH_DEADLINE):
            self.cancelled += 1
        self._done[rid] = st

    # ---- the loop ---------------------------------------------------------------------
    def _discard_prepared(self) -> None:
        """Takes back a step that was prepared ahead and will not run as planned."""
        if self._prepared is None:
            return
        plan, prep, _ = self._prepared
        self._prepared = None
        self.engine.discard(prep)
        for p in plan:
            self.scheduler.rollback(p.request_id)

    def _fail_plan(self, plan, error: Exception) -> None:
        for p in plan:                                 # src/engine/scheduler.rs:882-895
            self.scheduler.rollback(p.request_id)
            self._finish(p.request_id, FINISH_ERROR, str(error))

    def _plan_ahead(self, plan, sampled, states) -> bool:
        """While the device runs a decode step, does the host half of the next one: bookkeeping of this
        step, the scheduler's plan, page reservation and batch layout, with the ids of the tokens being
        sampled left open.  Only when no token value can change the plan: nobody reaches its length in
        this step (whoever waits in the queue is then admitted by the same rule a turn later would apply
        to the same state).  A stop token still can: then the prepared step is taken back.  Returns
        whether this step's bookkeeping (advance, append_token) was done."""
        if not self.config.plan_ahead:
            return False
        for st in states:
            if len(st.tokens) - st.usage.prompt_tokens + 1 >= st.request.sampling.max_new_tokens:
                return False
        samples = {p.request_id for p in sampled}
        for p in plan:
            self.scheduler.advance(p.request_id, p.count)
            if p.request_id in samples:
                self.scheduler.append_token(p.request_id)
        nxt, preempted = self.scheduler.plan()
        for rid in preempted:
            self._live[rid].usage.preemptions += 1
        if not nxt:
            return True
        entries, later = [], []
        for i, p in enumerate(nxt):
            st = self._live[p.request_id]
            known = len(st.tokens)                     # the token being sampled will sit at this index
            toks = [st.tokens[j] if j < known else LATER for j in range(p.start, p.start + p.count)]
            if p.start + p.count > known:
                later.append((i, known - p.start, p.request_id))
            entries.append(StepEntry(p.slot, toks, [p.count - 1] if p.want_logits else []))
        try:
            prep = self.engine.prepare(entries)
        except EngineError:
            for p in nxt:                              # planned normally at the next turn
                self.scheduler.rollback(p.request_id)
            return True
        self._prepared = (nxt, prep, later)
        return True

    def _drop_ahead(self) -> None:
        """Takes back whatever was done for the step after the current one: a step laid out ahead, or
        one already queued on the device (it is waited for, then revoked: lengths, pages and state as
        before it; the fault words it may have raised are of no interest)."""
        self._discard_prepared()
        if self._inflight is None:
            return
        plan, prep, _ = self._inflight
        self._inflight = None
        self.steps_dropped += 1
        with torch.cuda.device(self.engine.mctx.device):
            torch.cuda.synchronize()
            self.engine.revoke(prep)
            self.sampler.clear_words()
        for p in plan:
            self.scheduler.rollback(p.request_id)

    def _may_launch_ahead(self) -> bool:
        """The step laid out ahead may be queued before this step's tokens are read: its token ids are
        taken on the device, and so is the last id of a repetition penalty's history.  Only decode steps:
        launching a step with a prompt portion kernel by kernel takes the host milliseconds, by which this
        step's tokens would reach their readers later."""
        if not self.config.launch_ahead or self._prepared is None or not self.engine.use_graphs:
            return False                 # (without graphs a decode step is launched kernel by kernel too)
        nxt, _, _ = self._prepared
        return all(p.count == 1 for p in nxt)

    def _launch_ahead(self, sampled) -> None:
        """Queues the step that was laid out ahead behind this step's sampler: its open token ids are
        filled on the device from the sampler's rows."""
        nxt, prep, later = self._prepared
        self._prepared = None
        row_of = {p.request_id: k for k, p in enumerate(sampled)}
        try:
            logits = self.engine.run(prep, [(entry, index, row_of[rid]) for entry, index, rid in later])
        except EngineError:
            for p in nxt:                              # planned normally at the next turn
                self.scheduler.rollback(p.request_id)
            return
        ids = [p.request_id for p in nxt if p.want_logits]
        states = [self._live[rid] for rid in ids]
        # a request sampled in the step before has one token more than its list shows yet
        rows = self.sampler.launch(
            logits, [s.request.sampling for s in states], [s.seed for s in states],
            [len(s.tokens) - s.usage.prompt_tokens + (rid in row_of) for rid, s in zip(ids, states)],
            [s.tokens for s in states], pending=[row_of.get(rid) for rid in ids])
        self._inflight = (nxt, prep, rows)
        self.steps_ahead += 1

    def step(self, on_token: Optional[Callable[[int, int, int], None]] = None) -> bool:
        """One scheduler turn: interruptions, plan, one engine step, sampling.  False when idle."""
        now = time.monotonic()
        for rid, st in list(self._live.items()):      # checked between steps only
            reason = FINISH_CANCELLED if st.cancelled else \
                FINISH_DEADLINE if st.deadline_at is not None and now >= st.deadline_at else None
            if reason is not None:
                self._drop_ahead()
                self._finish(rid, reason)
        if self._inflight is not None:                # queued on the device during the turn before
            plan, prep, rows = self._inflight
            self._inflight = None
            sampled = [p for p in plan if p.want_logits]
            states = [self._live[p.request_id] for p in sampled]
        else:
            if self._prepared is not None:
                plan, prep, _ = self._prepared
                self._prepared = None
            else:
                if not self.scheduler.has_work():
                    return False
                plan, preempted = self.scheduler.plan()
                for rid in preempted:
                    self._live[rid].usage.preemptions += 1
                if not plan:
                    return self.scheduler.has_work() and bool(self._live)
                entries = []
                for p in plan:
                    st = self._live[p.request_id]
                    entries.append(StepEntry(p.slot, st.tokens[p.start:p.start + p.count],
                                             [p.count - 1] if p.want_logits else []))
                try:
                    prep = self.engine.prepare(entries)
                except EngineError as e:
                    self._fail_plan(plan, e)
                    return True
            for p in plan:
                st = self._live[p.request_id]
                if st.first_step_at is None:
                    st.first_step_at = now
                    st.usage.queue_ms = (now - st.submitted_at) * 1000.0
            try:
                logits = self.engine.run(prep)
            except EngineError as e:
                self._fail_plan(plan, e)
                return True
            sampled = [p for p in plan if p.want_logits]
            states = [self._live[p.request_id] for p in sampled]
            rows = self.sampler.launch(
                logits, [s.request.sampling for s in states], [s.seed for s in states],
                [len(s.tokens) - s.usage.prompt_tokens for s in states], [s.tokens for s in states])
        self.last_step = {"starts": [p.start for p in plan], "counts": [p.count for p in plan]}
        ahead = self._plan_ahead(plan, sampled, states)        # overlaps the device's work
        if ahead and self._may_launch_ahead():
            rows = self.sampler.snapshot(rows)                 # this step's tokens and words, read below
            self._launch_ahead(sampled)                        # the next step waits on the device already
        tokens = self.sampler.collect(rows)                     # waits for the device; the fault words come along
        fault = self.engine.fault_of(self.sampler.last_words)
        if fault is not None:
            # the step's result cannot be trusted: none of its tokens is published, every request of
            # the step ends with an error and gives its pages and its slot back
            # (src/engine/scheduler.rs:882-895)
            self._drop_ahead()
            prep.state_snapshot = None
            self._fail_plan(plan, fault)
            return True
        if not ahead:
            for p in plan:
                self.scheduler.advance(p.request_id, p.count)
        stopped = [p.request_id for p, tok in zip(sampled, tokens) if tok in self.eos]
        if ahead and stopped:
            self._drop_ahead()                         # a stop token changes who decodes next
        by_rid = {}
        for p, st, tok in zip(sampled, states, tokens):
            rid = p.request_id
            if tok in self.eos:                        # the stop token is neither kept nor fed
                if ahead:
                    self.scheduler.retract_token(rid)
                self._finish(rid, FINISH_STOP)
                continue
            st.tokens.append(tok)
            by_rid[rid] = tok
            n = len(st.tokens) - st.usage.prompt_tokens if ahead else self.scheduler.append_token(rid)
            if on_token is not None:
                on_token(rid, tok, n - 1)
            if n >= st.request.sampling.max_new_tokens:
                self._finish(rid, FINISH_LENGTH)       # no forward for a token nobody will read
        if self._prepared is not None:
            _, nxt_prep, later = self._prepared
            for entry, index, rid in later:
                nxt_prep.set_token(entry, index, by_rid[rid])
        return True

    def run_until_idle(self, on_token=None) -> None:
        while self.step(on_token):
            pass

    def take_result(self, request_id: int) -> Optional[GenerationResult]:
        st = self._done.pop(request_id, None)
        if st is None:
            return None
        return GenerationResult(request_id, st.generated, st.finish_reason, st.usage, st.error)

    def generate(self, prompts: Sequence[Sequence[int]], sampling: Optional[SamplingParams] = None
                 ) -> List[GenerationResult]:
        """Token ids in, token ids out; requests beyond the queue's capacity wait for room."""
        sampling = sampling or SamplingParams()
        pending = list(enumerate(prompts))
        ids: Dict[int, int] = {}
        while pending or self._live:
            while pending:
                if self.scheduler.counters()["queued"] >= self.config.queue_capacity:
                    break
                i, prompt = pending[0]
                try:
                    ids[i] = self.submit(GenerationRequest(list(prompt), SamplingParams(**vars(sampling))))
                except ResourceExhausted:
                    if not self._live:
                        raise
                    break
                pending.pop(0)
            if not self.step() and pending and not self._live:
                continue
        return [self.take_result(ids[i]) for i in range(len(prompts))]

    def metrics(self) -> dict:             # src/engine/scheduler.rs:221-272
        m = dict(self.scheduler.counters())
        m["failed"], m["cancelled"] = self.failed, self.cancelled
        return m
