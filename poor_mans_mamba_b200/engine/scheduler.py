"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.  Pure host logic over the cache manager's accounting; it
plans steps and digests their results, the engine runs them.

Decisions, in order, every step:
 1. Requests that wait for exactly one token (decoding) go first, one token each.  If the
    pages they need are not free, the most recently admitted running request is
    *preempted*: everything it holds is given back and it returns to the front of the
    waiting queue, to be recomputed later from its prompt plus what it has generated
    (fixed-size state cannot be evicted in part).  A request that is alone and still
    cannot get a page ends with what it has (status ``cache_full``), as the reference ends
    a session on KV overflow with a partial result (src/runtime/cluster_scheduler.cpp:645-651).
 2. With the rest of the token budget, prompts that are partly computed continue, cut to
    the budget and to the pages that are free.
 3. Waiting requests are admitted first-come-first-served while a slot, the sequence cap
    and pages for their next portion allow.  A request whose tokens can never fit the pool
    fails at once (status ``oom``; the reference rejects a submit when no slot is free,
    src/runtime/cluster_scheduler.cpp:262-267).
 A request ends on its eos token (kept in the output) or at max_new_tokens
 (src/runtime/cluster_scheduler.cpp:474-499), or, with what it has and status ``max_seq``, when
 its context has reached ``max_seq_len`` and the token just sampled can no longer be fed (the
 reference: KV overflow on decode -> done with a partial result,
 src/runtime/cluster_scheduler.cpp:645-651).  A prompt longer than ``max_seq_len`` ends at once
 with status ``max_seq`` and no output (there the prefill fails, src/ops/cuda_backend.cu:578-579).
The plan is deterministic given the arrival order.
"""
from __future__ import annotations

import collections
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Tuple

from ..cache.manager import CacheManager


@dataclass
class SamplingParams:
    max_new_tokens: int = 32
    eos_id: int = -1          # -1: no stop token
    temperature: float = 0.0  # 0: greedy
    seed: int = 0


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    n_computed: int = 0      # tokens of prompt+output whose state is in the cache
    status: str = "waiting"  # waiting | running | done | max_seq | cache_full | oom
    preemptions: int = 0
    admitted_at: int = -1

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.n_computed

    @property
    def finished(self) -> bool:
        return self.status in ("done", "max_seq", "cache_full", "oom")


@dataclass
class PlannedEntry:
    req: Request
    start: int   # first token index (in prompt+output) of the portion
    count: int
    samples: bool  # the portion reaches the end of the known tokens, so a token is sampled


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Hashable] = field(default_factory=list)
    ended: List[Hashable] = field(default_factory=list)   # finished while planning (cache_full / oom)

    @property
    def n_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batched_tokens: int = 2048, max_seqs: int = 64,
                 max_seq_len: Optional[int] = None, release: Optional[Callable[[Hashable], None]] = None):
        """``max_seq_len``: longest context (prompt + generated) a request may reach; a request that
        would pass it ends with what it has (status ``max_seq``).  ``release``: called with a
        request id to give back everything the request holds (default: the cache manager's
        release); an engine passes its runner's `finish` so that per-request records kept beside
        the cache go too."""
        if max_batched_tokens <= 0 or max_seqs <= 0:
            raise ValueError("max_batched_tokens and max_seqs must be positive")
        if max_seq_len is not None and max_seq_len <= 0:
            raise ValueError("max_seq_len must be positive")
        self.cache = cache
        self.max_seq_len = max_seq_len
        self._release = release if release is not None else cache.release
        self.max_batched_tokens = int(max_batched_tokens)
        self.max_seqs = min(int(max_seqs), cache.num_slots)
        self.waiting: Deque[Request] = collections.deque()
        self.running: List[Request] = []  # in order of admission
        self.requests: Dict[Hashable, Request] = {}
        self._admissions = 0
        self.counters = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0,
                         "rejects": 0, "cache_full": 0}

    # ------------------------------------------------------------------ submissions
    def add(self, req_id: Hashable, prompt: List[int], params: SamplingParams) -> Request:
        if req_id in self.requests:
            raise ValueError(f"request id {req_id!r} is already known")
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if params.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        req = Request(req_id, list(prompt), params)
        self.requests[req_id] = req
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ helpers
    def _free(self) -> Dict[Tuple, int]:
        return dict(self.cache.free_pages())

    def _need(self, req: Request, new_len: int) -> Dict[Tuple, int]:
        if self.cache.has(req.id):
            return self.cache.pages_needed(req.id, new_len)
        return {k: g.blocks_for(new_len) for k, g in self.cache.groups.items()}

    @staticmethod
    def _fits(need: Dict[Tuple, int], free: Dict[Tuple, int]) -> bool:
        return all(need[k] <= free[k] for k in need)

    def _max_tokens_that_fit(self, req: Request, want: int, free: Dict[Tuple, int]) -> int:
        """The longest portion <= want whose pages are free."""
        lo, hi = 0, want
        while lo < hi:  # page need grows with the length: bisect
            mid = (lo + hi + 1) // 2
            if self._fits(self._need(req, req.n_computed + mid), free):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _never_fits(self, req: Request) -> bool:
        total = len(req.prompt) + len(req.output)
        return any(g.blocks_for(total) > g.num_pages for g in self.cache.groups.values() if g.window <= 0)

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self._release(req.id)
        self.running.remove(req)
        req.n_computed = 0
        req.status = "waiting"
        req.preemptions += 1
        self.waiting.appendleft(req)
        self.counters["preemptions"] += 1
        plan.preempted.append(req.id)

    def _end(self, req: Request, status: str, plan: Optional[StepPlan] = None) -> None:
        if self.cache.has(req.id):
            self._release(req.id)
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:  # preempted, then found to have ended (a stop token read late)
            self.waiting.remove(req)
        req.status = status
        if plan is not None:
            plan.ended.append(req.id)

    # ------------------------------------------------------------------ planning
    def plan(self) -> StepPlan:
        plan = StepPlan()
        while True:
            self._plan_once(plan)
            if plan.entries or not self.running:
                break
            # running requests exist but none can move: give the newest one's pages to the others
            victim = self.running[-1]
            if len(self.running) == 1:
                self.counters["cache_full"] += 1
                self._end(victim, "cache_full", plan)
            else:
                self._preempt(victim, plan)
        return plan

    def _plan_once(self, plan: StepPlan) -> None:
        plan.entries = []
        budget = self.max_batched_tokens

        # 1. decoding requests first; make room for them by preemption if needed
        while True:
            decoders = [r for r in self.running if r.pending == 1]
            free = self._free()
            need: Dict[Tuple, int] = {k: 0 for k in free}
            for r in decoders:
                for k, n in self._need(r, r.n_computed + 1).items():
                    need[k] += n
            if self._fits(need, free) or not self.running:
                break
            victim = self.running[-1]
            if len(self.running) == 1:
                self.counters["cache_full"] += 1
                self._end(victim, "cache_full", plan)
            else:
                self._preempt(victim, plan)
        free = self._free()
        for r in [r for r in self.running if r.pending == 1]:
            if budget == 0:
                break
            for k, n in self._need(r, r.n_computed + 1).items():
                free[k] -= n
            plan.entries.append(PlannedEntry(r, r.n_computed, 1, True))
            budget -= 1

        # 2. prompts that are partly computed
        for r in [r for r in self.running if r.pending > 1]:
            if budget == 0:
                break
            n = self._max_tokens_that_fit(r, min(r.pending, budget), free)
            if n == 0:
                continue
            for k, v in self._need(r, r.n_computed + n).items():
                free[k] -= v
            plan.entries.append(PlannedEntry(r, r.n_computed, n, n == r.pending))
            budget -= n

        # 3. admissions, first come first served
        free_slots = self.cache.free_slots
        while self.waiting and budget > 0 and len(self.running) < self.max_seqs and free_slots > 0:
            r = self.waiting[0]
            if self.max_seq_len is not None and len(r.prompt) + len(r.output) > self.max_seq_len:
                self.waiting.popleft()
                self.counters["rejects"] += 1
                self._end(r, "max_seq", plan)
                continue
            if self._never_fits(r):
                self.waiting.popleft()
                self.counters["rejects"] += 1
                self._end(r, "oom", plan)
                continue
            n = self._max_tokens_that_fit(r, min(r.pending, budget), free)
            if n == 0:
                break
            self.waiting.popleft()
            self.cache.admit(r.id)
            free_slots -= 1
            r.status = "running"
            r.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(r)
            for k, v in self._need(r, r.n_computed + n).items():
                free[k] -= v
            plan.entries.append(PlannedEntry(r, r.n_computed, n, n == r.pending))
            budget -= n

    # ------------------------------------------------------------------ results
    def complete(self, plan: StepPlan, sampled: List[int]) -> List[Request]:
        """Digest a step: ``sampled`` holds one token for every planned entry with
        ``samples`` set, in plan order.  Returns the requests that finished."""
        self.counters["steps"] += 1
        it = iter(sampled)
        finished: List[Request] = []
        for e in plan.entries:
            r = e.req
            r.n_computed += e.count
            self.counters["decode_tokens" if e.count == 1 and r.output else "prefill_tokens"] += e.count
            if not e.samples:
                continue
            tok = int(next(it))
            r.output.append(tok)
            hit_eos = r.params.eos_id >= 0 and tok == r.params.eos_id
            if hit_eos or len(r.output) >= r.params.max_new_tokens:
                self._end(r, "done")
                finished.append(r)
            elif self._at_max_seq(r):
                self._end(r, "max_seq")
                finished.append(r)
        return finished

    def _at_max_seq(self, r: Request) -> bool:
        """The cache holds max_seq_len tokens of this request: its next token cannot be computed."""
        return self.max_seq_len is not None and r.n_computed >= self.max_seq_len

    # ------------------------------------------------------------------ results that arrive late
    # A decode step whose sampled ids are still on their way to the host can be digested in two
    # halves, so that the next step is planned and launched meanwhile: `advance` does everything
    # that needs no token value (lengths, counters, ending by length) and leaves PENDING in the
    # outputs; `resolve` fills the values in and applies the stop token, one step late.
    PENDING = -1

    def advance(self, plan: StepPlan) -> List[Tuple[Request, int]]:
        """First half of `complete` for a step whose ids are not known yet.  Returns, for every
        sampling entry in plan order, (request, index in its output) for `resolve`."""
        self.counters["steps"] += 1
        slots: List[Tuple[Request, int]] = []
        for e in plan.entries:
            r = e.req
            r.n_computed += e.count
            self.counters["decode_tokens" if e.count == 1 and r.output else "prefill_tokens"] += e.count
            if not e.samples:
                continue
            slots.append((r, len(r.output)))
            r.output.append(self.PENDING)
            if len(r.output) >= r.params.max_new_tokens:
                self._end(r, "done")
            elif self._at_max_seq(r):
                self._end(r, "max_seq")
        return slots

    def resolve(self, slots: List[Tuple[Request, int]], sampled: List[int]) -> List[Request]:
        """Second half: the ids of the entries that `advance` listed.  A request that hits its
        stop token ends now; tokens it was given by later steps meanwhile are dropped."""
        finished: List[Request] = []
        for (r, idx), tok in zip(slots, sampled):
            if idx >= len(r.output) or r.output[idx] != self.PENDING:
                continue  # cut off by a stop token that an earlier step produced
            r.output[idx] = int(tok)
            if r.params.eos_id >= 0 and int(tok) == r.params.eos_id:
                del r.output[idx + 1:]
                if r.status != "done":  # still running, or ended by length meanwhile: the stop token decides
                    self._end(r, "done")
                finished.append(r)
        return finished
