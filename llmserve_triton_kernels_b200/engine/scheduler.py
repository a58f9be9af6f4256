"""Continuous batching above the step function: admit, cut prompts into portions, decode, finish, free.

Parity: src/llmserve/scheduler/engine.py:83-310.  Kept from the reference: first come first
served with no skipping; at most ``max_batch_size`` live requests; admission needs the pages
of what it will run plus one spare page per live request (engine.py:218-227); a finished
request leaves and frees its pages inside the step (engine.py:291-301); abort takes effect at
the start of the next step (engine.py:149-152, 197-210); when pages run out the newest
admitted request is preempted — its pages are freed, it goes back to the head of the queue and
is recomputed from its first token later, with unchanged results (engine.py:257-274); the
``static`` policy admits only when nothing is running (engine.py:213-214).

Different from the reference: a step is ONE mixed batch under a token budget
(``max_num_batched_tokens``).  Every running request that is decoding brings one token; what is
left of the budget goes to portions of prompts (at most ``chunk_size`` tokens of a request per
step), oldest request first; a request is sampled only in the step that holds the last token of
what it has to feed.  The reference runs whole prompts in one padded pass and decodes in a second
(engine.py:186-193).
"""

from __future__ import annotations

import random
import threading
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from time import perf_counter

from ..cache import CacheManager, OutOfPages
import torch

from ..sampling import Sampler, SamplingParams
from .batch import StepEntry


class Status(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(eq=False)  # a request is itself: `in` and `remove` go by identity, not by comparing every field
class Request:
    req_id: int
    prompt_ids: list[int]
    params: SamplingParams
    arrival_time: float
    seed: int
    generated: list[int] = field(default_factory=list)
    status: Status = Status.WAITING
    num_computed: int = 0  # tokens of prompt + generated that are in the cache
    token_times: list[float] = field(default_factory=list)
    finish_time: float | None = None
    finish_reason: str | None = None  # "stop" | "length" | "abort"
    num_preemptions: int = 0

    _all: list[int] | None = field(default=None, repr=False, compare=False)

    @property
    def all_ids(self) -> list[int]:
        """Prompt and generated tokens as one list, kept up to date by :meth:`append` (the scheduler asks for it
        many times a step: it is not rebuilt each time)."""
        if self._all is None or len(self._all) != len(self.prompt_ids) + len(self.generated):
            self._all = self.prompt_ids + self.generated
        return self._all

    @property
    def num_ids(self) -> int:
        return len(self.prompt_ids) + len(self.generated)

    def append(self, token: int) -> None:
        self.generated.append(token)
        if self._all is not None:
            self._all.append(token)

    @property
    def first_token_time(self) -> float | None:
        return self.token_times[0] if self.token_times else None


@dataclass
class TokenEvent:
    req_id: int
    token: int | None
    finished: bool
    finish_reason: str | None = None
    error: str | None = None


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0  # tokens run as portions of prompts (recomputation after preemption included)
    decode_tokens: int = 0
    tokens_generated: int = 0
    preemptions: int = 0
    last_batch_tokens: int = 0
    last_batch_requests: int = 0


@dataclass
class _Ahead:
    """A decode step that has been launched and whose tokens the host has not read yet."""

    reqs: list  # the requests of the step, in the order of its rows
    device_tokens: object  # int32 [rows] on the device: what the step chose
    host_tokens: object  # the same on the host (pinned memory, written by the sampling kernel), valid once `copied` has happened
    copied: object  # event after that kernel


class Scheduler:
    def __init__(
        self,
        step_function,
        cache: CacheManager,
        sampler: Sampler,
        *,
        max_position: int,
        max_batch_size: int = 8,
        max_num_batched_tokens: int = 4096,
        chunk_size: int | None = None,
        policy: str = "continuous",
        run_ahead: bool | None = None,
    ):
        if policy not in ("continuous", "static"):
            raise ValueError("policy must be 'continuous' or 'static'")
        if max_batch_size < 1 or max_num_batched_tokens < 1 or (chunk_size is not None and chunk_size < 1):
            raise ValueError("max_batch_size, max_num_batched_tokens and chunk_size must be positive")
        if max_batch_size > cache.max_requests:
            raise ValueError(f"max_batch_size {max_batch_size} exceeds the cache's {cache.max_requests} request slots")
        self.step_function = step_function
        self.cache = cache
        self.sampler = sampler
        self.max_position = int(max_position)
        self.max_batch_size = int(max_batch_size)
        self.max_num_batched_tokens = int(max_num_batched_tokens)
        self.chunk_size = int(chunk_size) if chunk_size else self.max_num_batched_tokens
        self.policy = policy
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: dict[int, Request] = {}
        self.stats = EngineStats()
        self._next_id = 0
        self._aborts: set[int] = set()
        self._lock = threading.Lock()
        # Decode steps that replay a graph run one step ahead of the host: the next step is fed the chosen tokens
        # on the device and launched before the host reads them, so the GPU does not wait for the host between
        # steps.  The host sees a step's tokens one call of step() later.
        self.run_ahead = bool(getattr(step_function, "use_graphs", False)) if run_ahead is None else bool(run_ahead)
        self._ahead: _Ahead | None = None

    # ------------------------------------------------------------------ public
    def validate_request(self, prompt_len: int, max_new_tokens: int) -> None:
        """Raise ValueError for a request that could never be served (src/llmserve/scheduler/engine.py:111-125)."""
        if prompt_len < 1:
            raise ValueError("prompt must contain at least one token")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        total = prompt_len + max_new_tokens
        if total > self.max_position:
            raise ValueError(f"prompt + max_new_tokens = {total} exceeds model limit {self.max_position}")
        need = self.cache.peak_pages_for(total, min(self.chunk_size, self.max_num_batched_tokens))
        if need > self.cache.num_pages:
            raise ValueError(f"request needs {need} pages but the pool has only {self.cache.num_pages}")

    def add_request(self, prompt_ids, params: SamplingParams, *, req_id: int | None = None, arrival_time: float | None = None) -> int:
        self.validate_request(len(prompt_ids), params.max_new_tokens)
        if req_id is None:
            req_id = self._next_id
        self._next_id = max(self._next_id, req_id + 1)
        seed = params.seed if params.seed is not None else random.getrandbits(63)
        self.waiting.append(
            Request(
                req_id=req_id,
                prompt_ids=[int(t) for t in prompt_ids],
                params=params,
                arrival_time=perf_counter() if arrival_time is None else arrival_time,
                seed=int(seed) & ((1 << 63) - 1),
            )
        )
        return req_id

    def abort(self, req_id: int) -> None:
        """Cancel a request at the start of the next step.  Thread-safe."""
        with self._lock:
            self._aborts.add(req_id)

    def reset(self) -> None:
        """Drop every request in flight and free all pages (error recovery)."""
        for r in self.running:
            if self.cache.has_request(r.req_id):
                self.cache.free_request(r.req_id)
        self.running.clear()
        self.waiting.clear()
        self._ahead = None

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def snapshot(self) -> dict:
        return {
            "running": len(self.running),
            "waiting": len(self.waiting),
            "free_blocks": self.cache.num_free_pages,
            "total_blocks": self.cache.num_pages,
            "kv_utilization": round(self.cache.utilization(), 4),
            "preemptions": self.stats.preemptions,
            "tokens_generated": self.stats.tokens_generated,
        }

    def run_until_complete(self) -> dict[int, Request]:
        while self.has_unfinished():
            self.step()
        self._ahead = None  # a step too many of requests that ended by their end-of-sequence token: nobody reads it
        return self.finished

    # ------------------------------------------------------------------ one step
    def step(self) -> list[TokenEvent]:
        events: list[TokenEvent] = []
        self.stats.steps += 1
        if self._ahead is not None:
            ahead, self._ahead = self._ahead, None
            if self._can_run_ahead(ahead):
                self._ahead = self._launch_ahead(ahead)  # the GPU goes on while the host catches up
            self._collect(ahead, events)
            if self._ahead is not None:
                return events
        self._process_aborts(events)
        plan = self._plan()
        if not plan:
            return events
        entries = []
        for req, n in plan:
            ids = req.all_ids
            last = req.num_computed + n == len(ids)
            entries.append(StepEntry(req.req_id, ids[req.num_computed : req.num_computed + n], [n - 1] if last else []))
        logits = self.step_function(entries)
        sampled = []
        for req, n in plan:
            decoding = n == 1 and req.num_computed + 1 == req.num_ids and req.generated and req.num_computed >= len(req.prompt_ids)
            if decoding:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += n
            req.num_computed += n
            if req.num_computed == req.num_ids:
                sampled.append(req)
        self.stats.last_batch_tokens = sum(n for _, n in plan)
        self.stats.last_batch_requests = len(plan)
        if sampled:
            params, seeds = [r.params for r in sampled], [r.seed for r in sampled]
            counters = [len(r.generated) for r in sampled]
            if self.run_ahead and len(sampled) == len(plan) and all(n == 1 for _, n in plan):
                # a decode step of every running request: its tokens stay on the device for now
                self._ahead = self._sample_ahead(sampled, logits, params, seeds, counters)
            else:
                self._append(sampled, self.sampler(logits, params, seeds, counters), events)
        return events

    # ------------------------------------------------------------------ one step ahead of the host
    def _sample_ahead(self, reqs: list[Request], logits, params, seeds, counters) -> _Ahead:
        """Tokens chosen and left on the device; the sampling kernel writes them into pinned host memory as well,
        where the host may read them once the event has happened."""
        if not logits.is_cuda:
            tokens = self.sampler.on_device(logits, params, seeds, counters)
            return _Ahead(reqs, tokens, tokens.clone(), None)
        host = torch.empty((logits.shape[0],), dtype=torch.int32, pin_memory=True)
        tokens = self.sampler.on_device(logits, params, seeds, counters, host_out=host)
        written = torch.cuda.Event()
        written.record()
        return _Ahead(reqs, tokens, host, written)

    def _can_run_ahead(self, ahead: _Ahead) -> bool:
        """The step after ``ahead`` can be launched before ``ahead``'s tokens are known: the same requests decode on
        (none ends by its length with the token that is on its way; one that ends by its end-of-sequence token
        does a step too many, whose result is dropped), nobody waits to be admitted or aborted, pages suffice."""
        with self._lock:
            if self._aborts:
                return False
        if self.waiting or len(ahead.reqs) != len(self.running) or any(a is not b for a, b in zip(ahead.reqs, self.running)):
            return False
        if any(len(r.generated) + 2 > r.params.max_new_tokens for r in ahead.reqs):
            return False
        need = sum(self.cache.extra_pages_needed(r.req_id, 1) for r in ahead.reqs)
        return need <= self.cache.num_free_pages

    def _launch_ahead(self, ahead: _Ahead) -> _Ahead:
        reqs = ahead.reqs
        logits = self.step_function.decode_ahead([r.req_id for r in reqs], ahead.device_tokens)
        for r in reqs:
            r.num_computed += 1
        self.stats.decode_tokens += len(reqs)
        self.stats.last_batch_tokens = self.stats.last_batch_requests = len(reqs)
        return self._sample_ahead(reqs, logits, [r.params for r in reqs], [r.seed for r in reqs], [len(r.generated) + 1 for r in reqs])

    def _collect(self, ahead: _Ahead, events: list[TokenEvent]) -> None:
        """The host reads the tokens of a step launched earlier.  A request that has ended meanwhile (its
        end-of-sequence token came with the step before, or it was aborted) drops its token."""
        if ahead.copied is not None:
            ahead.copied.synchronize()
        tokens = ahead.host_tokens.tolist()
        live = [(r, t) for r, t in zip(ahead.reqs, tokens) if r.status is Status.RUNNING and r in self.running]
        self._append([r for r, _ in live], [t for _, t in live], events)

    # ------------------------------------------------------------------ internals
    def _process_aborts(self, events: list[TokenEvent]) -> None:
        with self._lock:
            aborts, self._aborts = self._aborts, set()
        for rid in sorted(aborts):
            req = next((r for r in self.waiting if r.req_id == rid), None)
            if req is not None:
                self.waiting.remove(req)
            else:
                req = next((r for r in self.running if r.req_id == rid), None)
                if req is None:
                    continue  # already finished
                self.running.remove(req)
                self.cache.free_request(rid)
            self._finish(req, "abort", events, emit_token=None)

    def _portion(self, req: Request, budget: int) -> int:
        remaining = req.num_ids - req.num_computed
        return min(remaining, budget, self.chunk_size)

    def _plan(self) -> list[tuple[Request, int]]:
        """What this step runs: ``(request, number of its next tokens)``.  Preempts until the
        running requests' needs fit, then admits from the queue while pages and budget allow."""
        budget = self.max_num_batched_tokens
        plan: list[tuple[Request, int]] = []
        # decoding requests first (one token each), then portions of prompts, oldest first
        for pick_decodes in (True, False):
            for req in self.running:
                is_decode = req.num_ids - req.num_computed == 1
                if is_decode != pick_decodes or budget == 0:
                    continue
                n = self._portion(req, budget)
                plan.append((req, n))
                budget -= n
        order = {id(r): i for i, r in enumerate(self.running)}
        plan.sort(key=lambda item: order[id(item[0])])

        # pages run out: the newest admitted request gives its pages back and is recomputed later
        while plan:
            need = sum(self.cache.extra_pages_needed(r.req_id, n) for r, n in plan)
            if need <= self.cache.num_free_pages:
                break
            victim = self.running[-1]
            plan = [(r, n) for r, n in plan if r is not victim]
            self._preempt(victim)

        if self.policy == "static" and self.running:
            return plan
        reserved = sum(self.cache.extra_pages_needed(r.req_id, n) for r, n in plan)
        while self.waiting and len(self.running) < self.max_batch_size and budget > 0:
            req = self.waiting[0]
            n = self._portion(req, budget)
            need = self.cache.pages_for(n)
            headroom = len(self.running)  # one spare page per live request, so the next decode cannot starve
            if self.cache.num_free_pages - reserved - need < headroom:
                break
            self.waiting.popleft()
            self.cache.add_request(req.req_id)
            req.status = Status.RUNNING
            self.running.append(req)
            plan.append((req, n))
            reserved += need
            budget -= n
        return plan

    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        self.cache.free_request(req.req_id)
        req.status = Status.WAITING
        req.num_computed = 0
        req.num_preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(req)

    def _append(self, reqs: list[Request], tokens: list[int], events: list[TokenEvent]) -> None:
        now = perf_counter()
        for r, tok in zip(reqs, tokens):
            r.append(int(tok))
            r.token_times.append(now)
            self.stats.tokens_generated += 1
            reason = None
            if r.params.eos_token_id is not None and tok == r.params.eos_token_id:
                reason = "stop"
            elif len(r.generated) >= r.params.max_new_tokens:
                reason = "length"
            if reason:
                self.running.remove(r)
                self.cache.free_request(r.req_id)
                self._finish(r, reason, events, emit_token=int(tok))
            else:
                events.append(TokenEvent(r.req_id, int(tok), False))

    def _finish(self, req: Request, reason: str, events: list[TokenEvent], emit_token: int | None) -> None:
        req.status = Status.FINISHED
        req.finish_reason = reason
        req.finish_time = perf_counter()
        self.finished[req.req_id] = req
        events.append(TokenEvent(req.req_id, emit_token, True, reason))
