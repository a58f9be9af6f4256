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

import torch

from .. import ops
from ..cache import CacheManager, OutOfPages
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
        self._pinned: dict[int, dict] = {}

    # ------------------------------------------------------------------ requests in and out
    def _unservable(self, prompt_len: int, max_new_tokens: int) -> str | None:
        """Why a request of these lengths could never run here, or None.  The page need is the cache manager's: the
        most pages any group of layers holds for it at once, a windowed group giving pages back as it goes."""
        if prompt_len < 1:
            return "prompt must contain at least one token"
        if max_new_tokens < 1:
            return "max_new_tokens must be >= 1"
        longest = prompt_len + max_new_tokens
        if longest > self.max_position:
            return f"prompt + max_new_tokens = {longest} exceeds model limit {self.max_position}"
        portion = min(self.chunk_size, self.max_num_batched_tokens)
        peak = self.cache.peak_pages_for(longest, portion)
        if peak > self.cache.num_pages:
            return f"request needs {peak} pages but the pool has only {self.cache.num_pages}"
        return None

    def validate_request(self, prompt_len: int, max_new_tokens: int) -> None:
        """ValueError for a request that no amount of waiting would serve (the reference refuses the same four cases
        up front: src/llmserve/scheduler/engine.py:111-125)."""
        why = self._unservable(prompt_len, max_new_tokens)
        if why:
            raise ValueError(why)

    def add_request(self, prompt_ids, params: SamplingParams, *, req_id: int | None = None, arrival_time: float | None = None) -> int:
        self.validate_request(len(prompt_ids), params.max_new_tokens)
        rid = self._next_id if req_id is None else req_id
        self._next_id = max(self._next_id, rid + 1)
        drawn = random.getrandbits(63) if params.seed is None else int(params.seed)
        self.waiting.append(Request(
            req_id=rid, prompt_ids=[int(t) for t in prompt_ids], params=params, seed=drawn & ((1 << 63) - 1),
            arrival_time=perf_counter() if arrival_time is None else arrival_time,
        ))
        return rid

    def abort(self, req_id: int) -> None:
        """Cancel a request; it leaves at the start of the next step.  May be called from another thread."""
        with self._lock:
            self._aborts.add(req_id)

    def reset(self) -> None:
        """Error recovery: every request in flight is dropped (none is reported finished) and its pages come back."""
        self._ahead = None
        for req in list(self.running):
            self._leave(req, None)
        self.waiting.clear()

    def has_unfinished(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def snapshot(self) -> dict:
        """Counters under the names the reference's engine reports them by (src/llmserve/scheduler/engine.py:164-173)."""
        cache, stats = self.cache, self.stats
        return {
            "running": len(self.running), "waiting": len(self.waiting),
            "free_blocks": cache.num_free_pages, "total_blocks": cache.num_pages,
            "kv_utilization": round(cache.utilization(), 4),
            "preemptions": stats.preemptions, "tokens_generated": stats.tokens_generated,
        }

    def run_until_complete(self) -> dict[int, Request]:
        while self.has_unfinished():
            self.step()
        self._drop_ahead()  # a step too many of requests that ended by their end-of-sequence token: nobody reads it
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
                tokens = self.sampler(logits, params, seeds, counters)  # ends in a read by the host
                self._check_device()
                self._append(sampled, tokens, events)
        return events

    def _check_device(self) -> None:
        """Called where the host has just waited for the device: if a kernel reported that one of its bounded waits
        gave up, the step's results are not valid; everything in flight is dropped and the error raised."""
        try:
            ops.check_device_errors()
        except ops.KernelError:
            self.reset()
            raise

    # ------------------------------------------------------------------ one step ahead of the host
    def _sample_ahead(self, reqs: list[Request], logits, params, seeds, counters) -> _Ahead:
        """Tokens chosen and left on the device; the sampling kernel writes them into pinned host memory as well,
        where the host may read them once the event has happened."""
        if not logits.is_cuda:
            tokens = self.sampler.on_device(logits, params, seeds, counters)
            return _Ahead(reqs, tokens, tokens.clone(), None)
        host, written = self._pinned_tokens(logits.shape[0])
        tokens = self.sampler.on_device(logits, params, seeds, counters, host_out=host)
        written.record()
        return _Ahead(reqs, tokens, host, written)

    def _pinned_tokens(self, rows: int):
        """A pinned buffer for a step's tokens and the event that follows the kernel that writes it.  The sampling
        kernel writes the buffer itself, which torch's allocator of pinned memory knows nothing of, so the buffers
        are the scheduler's own: a ring of four per row count, each taken again only after its last kernel has run
        (at most two steps are in flight; a step that nobody collects leaves its buffer to come round)."""
        ring = self._pinned.setdefault(rows, {"at": 0, "slots": []})
        if len(ring["slots"]) < 4:
            ring["slots"].append((torch.empty((rows,), dtype=torch.int32, pin_memory=True), torch.cuda.Event()))
            return ring["slots"][-1]
        ring["at"] = (ring["at"] + 1) % 4
        host, event = ring["slots"][ring["at"]]
        event.synchronize()
        return host, event

    def _drop_ahead(self) -> None:
        self._ahead = None

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
        self._check_device()
        tokens = ahead.host_tokens.tolist()
        live = [(r, t) for r, t in zip(ahead.reqs, tokens) if r.status is Status.RUNNING and r in self.running]
        self._append([r for r, _ in live], [t for _, t in live], events)

    # ------------------------------------------------------------------ internals
    def _leave(self, req: Request, how: str | None, events: list[TokenEvent] | None = None, token: int | None = None) -> None:
        """Every way out of the running set goes through here, so that pages and state slot come back in one place.
        ``how``: "stop", "length" or "abort" end the request (an event says so, with the last token where there is
        one); "preempt" frees what it holds and puts it at the head of the queue, to be computed again from its
        first token; None drops it without a trace."""
        if any(r is req for r in self.running):
            self.running.remove(req)
        if self.cache.has_request(req.req_id):
            self.cache.free_request(req.req_id)
        if how is None:
            return
        if how == "preempt":
            req.status, req.num_computed = Status.WAITING, 0
            req.num_preemptions += 1
            self.stats.preemptions += 1
            self.waiting.appendleft(req)
            return
        req.status, req.finish_reason, req.finish_time = Status.FINISHED, how, perf_counter()
        self.finished[req.req_id] = req
        if events is not None:
            events.append(TokenEvent(req.req_id, token, True, how))

    def _process_aborts(self, events: list[TokenEvent]) -> None:
        with self._lock:
            wanted, self._aborts = self._aborts, set()
        if not wanted:
            return
        leaving = [r for r in list(self.waiting) + self.running if r.req_id in wanted]
        for req in sorted(leaving, key=lambda r: r.req_id):
            if req.status is Status.WAITING:
                self.waiting.remove(req)
            self._leave(req, "abort", events)
        # an id that is neither waiting nor running has ended already: nothing to do

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
        # Admission counts pages as the reference does, for the whole of what a request has to feed (its engine runs
        # whole prompts: src/llmserve/scheduler/engine.py:220-225), although here they are taken portion by portion:
        # what the running requests still need for their known tokens is spoken for.  A request that was admitted when
        # its first portion fitted would otherwise run out of pages halfway, be put back and computed again, over and over.
        spoken_for = sum(self._pages_still_needed(r) for r in self.running)
        while self.waiting and len(self.running) < self.max_batch_size and budget > 0:
            req = self.waiting[0]
            n = self._portion(req, budget)
            need = min(self.cache.pages_for(req.num_ids), self.cache.peak_pages_for(req.num_ids, min(self.chunk_size, self.max_num_batched_tokens)))
            headroom = len(self.running)  # one spare page per live request, so the next decode cannot starve
            if self.cache.num_free_pages - spoken_for - need < headroom:
                break
            self.waiting.popleft()
            self.cache.add_request(req.req_id)
            req.status = Status.RUNNING
            self.running.append(req)
            plan.append((req, n))
            spoken_for += need
            budget -= n
        return plan

    def _pages_still_needed(self, req: Request) -> int:
        """Pages that a running request has yet to take for the tokens it is known to hold (the rest of its prompt)."""
        return self.cache.extra_pages_needed(req.req_id, req.num_ids - req.num_computed) if req.num_ids > req.num_computed else 0

    def _preempt(self, req: Request) -> None:
        self._leave(req, "preempt")

    def _append(self, reqs: list[Request], tokens: list[int], events: list[TokenEvent]) -> None:
        """The tokens a step chose, one per request: each is recorded, and ends its request if it is the request's
        end-of-sequence token (which is emitted) or its last by length."""
        now = perf_counter()
        self.stats.tokens_generated += len(reqs)
        for req, token in zip(reqs, tokens):
            token = int(token)
            req.append(token)
            req.token_times.append(now)
            params = req.params
            if params.eos_token_id is not None and token == params.eos_token_id:
                self._leave(req, "stop", events, token)
            elif len(req.generated) >= params.max_new_tokens:
                self._leave(req, "length", events, token)
            else:
                events.append(TokenEvent(req.req_id, token, False))
