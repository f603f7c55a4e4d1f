"""Continuous batching above the step function: admit requests, cut prompts into
portions under a token budget, decode, finish and free.

Knobs carry the reference's names and defaults (scheduler/scheduler.h:74-84):
max_batch_size 32, max_batch_tokens 16384, chunked_prefill_tokens 512,
mixed_prefill_budget_ratio 1.0.  As in the reference's step loop
(runtime/execution/batch_executor.cpp:422-439, 1288-1316) every live request
contributes either its next prompt portion or its one current token, and only the
last portion of a prompt asks for logits.  Unlike the reference, requests join and
leave at every step, not only between batches.

When pages run out (the reference falls back to a stateless path,
scheduler/scheduler.cpp:2418-2427): a request is admitted only if the pages of its
first portion are free; if a live request cannot get the pages of its next tokens,
the most recently admitted request is preempted: its pages and slot are given back
and it returns to the head of the waiting queue with the tokens it has generated
appended to its prompt, to be recomputed.  A request that could never fit (longer
than the longest sequence, or needing more pages than the pool has) is failed with
`context_overflow`, as the reference rejects it up front (scheduler.cpp:2298-2324).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..sampling.params import SamplingParams
from .batch import StepEntry

PENDING = -1        # stands in a request's output for a token that has been sampled on the device but not read yet


@dataclass
class SchedulerConfig:
    max_batch_size: int = 32              # requests in one step
    max_batch_tokens: int = 16384         # tokens in one step
    chunked_prefill_tokens: int = 512     # largest prompt portion
    mixed_prefill_budget_ratio: float = 1.0   # share of max_batch_tokens that prompt portions may take

    def validate(self) -> None:
        if self.max_batch_size <= 0 or self.max_batch_tokens <= 0 or self.chunked_prefill_tokens <= 0:
            raise ValueError("max_batch_size, max_batch_tokens and chunked_prefill_tokens must be positive")
        if not 0 < self.mixed_prefill_budget_ratio <= 1:
            raise ValueError("mixed_prefill_budget_ratio must be in (0, 1]")


@dataclass(eq=False)
class Request:
    request_id: Hashable
    prompt: List[int]
    params: SamplingParams
    max_tokens: int = 256
    eos_token_ids: Sequence[int] = ()
    seed: int = 0
    arrival: int = 0
    output: List[int] = field(default_factory=list)
    computed: int = 0                 # tokens of prompt + output whose keys and values are stored
    status: str = "waiting"           # waiting | running | finished
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1
    pending: int = 0                  # PENDING entries at the end of `output`
    discard: bool = False             # finished, but still part of the step in flight: that token is dropped

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed

    def token_slice(self, start: int, count: int) -> List[int]:
        """Tokens [start, start + count) of prompt + output, without joining the two lists."""
        n = len(self.prompt)
        end = start + count
        if end <= n:
            return self.prompt[start:end]
        if start >= n:
            return self.output[start - n:end - n]
        return self.prompt[start:] + self.output[:end - n]


@dataclass
class ScheduledEntry:
    request: Request
    start: int
    count: int
    wants_logits: bool


@dataclass
class StepPlan:
    entries: List[ScheduledEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)
    needs_drain: bool = False         # a request would have to be preempted while tokens are pending

    def step_entries(self) -> List[StepEntry]:
        out = []
        for e in self.entries:
            toks = e.request.token_slice(e.start, e.count)
            out.append(StepEntry(e.request.request_id, toks, [e.count - 1] if e.wants_logits else [], start=e.start))
        return out

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    """Decides each step's batch.  It reads and frees pages through the cache
    manager; the step function takes the pages it has been promised."""

    def __init__(self, config: SchedulerConfig, cache, max_seq_len: int):
        config.validate()
        self.config = config
        self.cache = cache
        self.max_seq_len = int(max_seq_len)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.finishing: List[Request] = []       # finished, but the step in flight still holds their pages
        self._arrivals = 0
        self._admissions = 0
        self.num_preemptions = 0
        self.num_steps = 0

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r}: empty prompt")
        if request.max_tokens <= 0:
            request.max_tokens = 1                       # scheduler.cpp:1763-1801: max_tokens <= 0 -> 1
        request.params.validate()
        request.arrival = self._arrivals
        self._arrivals += 1
        request.status = "waiting"
        self.waiting.append(request)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running or self.finishing)

    # ------------------------------------------------------------------ helpers
    def _never_fits(self, r: Request) -> Optional[str]:
        total = len(r.prompt) + r.max_tokens
        if len(r.prompt) + 1 > self.max_seq_len:
            return (f"context_overflow: the prompt of {len(r.prompt)} tokens leaves no room in the longest "
                    f"sequence of {self.max_seq_len}")
        need = -(-min(total, self.max_seq_len) // self.cache.page_size)
        # groups with a window need fewer pages in the long run; the full-attention bound is what counts
        for g in self.cache.groups:
            if g.spec.window is None and need > g.alloc.num_pages:
                return (f"context_overflow: {min(total, self.max_seq_len)} tokens need {need} pages, "
                        f"the pool has {g.alloc.num_pages}")
        return None

    def _fits(self, need: List[int], taken: List[int]) -> bool:
        free = self.cache.free_pages()
        return all(n + t <= f for n, t, f in zip(need, taken, free))

    def _pages_for(self, r: Request, new_len: int) -> List[int]:
        if r.request_id in self.cache:
            return self.cache.pages_needed(r.request_id, new_len)
        return self.cache.pages_needed_fresh(new_len)

    def _preempt(self, r: Request, plan: StepPlan) -> None:
        if r.request_id in self.cache:
            self.cache.free(r.request_id)
        self.running.remove(r)
        r.computed = 0
        r.status = "waiting"
        r.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(r)
        plan.preempted.append(r)
        plan.entries = [e for e in plan.entries if e.request is not r]

    def _finish(self, r: Request, reason: str) -> None:
        r.status, r.finish_reason = "finished", reason
        if r.request_id in self.cache:
            self.cache.free(r.request_id)
        if r in self.running:
            self.running.remove(r)
        if r in self.finishing:
            self.finishing.remove(r)
        self.finished.append(r)

    def abort(self, request_id) -> Optional[Request]:
        """End a request at once, whatever its state (the reference cancels between decode
        iterations, runtime/execution/batch_executor.cpp:1406-1443, and releases slot and blocks
        in scheduler/scheduler.cpp:2984-3001).  Returns the request if its pages and slot are free
        now; None if a token of it is still pending in the step in flight (it is then freed, and
        reported, when that step's tokens are read, like a request that met its end there) or if no
        live request has that id."""
        for r in self.waiting:
            if r.request_id == request_id:
                self.waiting.remove(r)
                r.status, r.finish_reason = "finished", "abort"
                self.finished.append(r)
                return r
        for r in self.running:
            if r.request_id != request_id:
                continue
            if r.pending:                                   # the step in flight will bring a token for it
                del r.output[len(r.output) - r.pending:]
                r.pending = 0
                r.discard = True
                r.finish_reason = "abort"
                r.status = "finishing"
                self.running.remove(r)
                self.finishing.append(r)
                return None
            # A prompt portion of it may be in flight too: its pages may still be given to the next
            # step's requests, because that step runs after the one in flight, in stream order.
            self._finish(r, "abort")
            return r
        return None

    # ---------------------------------------------------------------- schedule
    def _may_continue(self, r: Request) -> bool:
        """False while a request has to wait for its pending token: it may be the last one."""
        if not r.pending:
            return True
        return len(r.output) < r.max_tokens and len(r.prompt) + len(r.output) < self.max_seq_len

    def schedule(self, inflight: bool = False) -> StepPlan:
        """Decide the next step.  With `inflight` the previous step's tokens are not known yet
        (PENDING): requests go on with the pending token, which the step takes from the device;
        if a preemption would be needed the plan only says `needs_drain` and changes nothing."""
        cfg = self.config
        plan = StepPlan()
        # Plans are made against the pages that are free now; `taken` counts what this plan has promised.
        while True:
            plan.entries = []
            taken = [0] * len(self.cache.groups)
            budget = cfg.max_batch_tokens
            ok = True
            # 1. decoding requests: one token each, oldest admission first
            decoding = [r for r in self.running if r.remaining == 1 and r.output and self._may_continue(r)]
            prefilling = [r for r in self.running if not (r.remaining == 1 and r.output) and r.remaining > 0]
            for r in decoding:
                need = self._pages_for(r, r.computed + 1)
                if budget < 1 or not self._fits(need, taken):
                    ok = False
                    break
                taken = [a + b for a, b in zip(taken, need)]
                plan.entries.append(ScheduledEntry(r, r.computed, 1, True))
                budget -= 1
            if not ok:
                if inflight:
                    plan.entries = []
                    plan.needs_drain = True
                    return plan
                victim = max(self.running, key=lambda r: r.admitted_at)
                self._preempt(victim, plan)
                continue
            # 2. prompts under way: the next portion of each
            prefill_budget = min(budget, int(cfg.max_batch_tokens * cfg.mixed_prefill_budget_ratio) - len(decoding))
            for r in prefilling:
                n = min(r.remaining, cfg.chunked_prefill_tokens, prefill_budget)
                n = self._shrink_to_pages(r, n, taken)
                if n <= 0:
                    continue
                need = self._pages_for(r, r.computed + n)
                taken = [a + b for a, b in zip(taken, need)]
                plan.entries.append(ScheduledEntry(r, r.computed, n, n == r.remaining))
                prefill_budget -= n
            # 3. admissions, first come first served
            new_slots = 0
            while self.waiting and len(self.running) < cfg.max_batch_size and self.cache.num_free_slots > new_slots:
                r = self.waiting[0]
                why = self._never_fits(r)
                if why:
                    self.waiting.popleft()
                    r.status, r.finish_reason = "finished", why
                    self.finished.append(r)
                    plan.failed.append(r)
                    continue
                n = min(r.remaining, cfg.chunked_prefill_tokens, prefill_budget)
                n = self._shrink_to_pages(r, n, taken)
                if n <= 0:
                    break
                self.waiting.popleft()
                new_slots += 1
                r.status = "running"
                r.admitted_at = self._admissions
                self._admissions += 1
                self.running.append(r)
                need = self._pages_for(r, r.computed + n)
                taken = [a + b for a, b in zip(taken, need)]
                plan.entries.append(ScheduledEntry(r, r.computed, n, n == r.remaining))
                prefill_budget -= n
            if plan.entries or not self.running:
                break
            if inflight:                        # everyone may simply be waiting for pending tokens
                plan.needs_drain = True
                return plan
            # nothing can move although requests are live: free the newest one's pages
            victim = max(self.running, key=lambda r: r.admitted_at)
            self._preempt(victim, plan)
        self.num_steps += 1 if plan.entries else 0
        return plan

    def _shrink_to_pages(self, r: Request, n: int, taken: List[int]) -> int:
        """Largest portion <= n whose pages are free (0 if not even one token fits)."""
        if n <= 0:
            return 0
        if self._fits(self._pages_for(r, r.computed + n), taken):
            return n
        lo, hi = 0, n - 1
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self._fits(self._pages_for(r, r.computed + mid), taken):
                lo = mid
            else:
                hi = mid - 1
        return lo

    # ------------------------------------------------------------------- update
    def advance(self, plan: StepPlan) -> None:
        """The step has been launched: its tokens count as stored, and every entry that
        wanted logits has a token coming whose value is not known yet."""
        for e in plan.entries:
            r = e.request
            r.computed = e.start + e.count
            if e.wants_logits:
                r.output.append(PENDING)
                r.pending += 1

    def resolve(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """The tokens of a launched step are known: `sampled` holds one per entry that
        wanted logits, in order.  Returns the requests that are finished and freed."""
        done = []
        it = iter(sampled)
        for e in plan.entries:
            if not e.wants_logits:
                continue
            r = e.request
            tok = int(next(it))
            if r.discard:                                    # it had already finished when this step was launched
                r.discard = False
                self._finish(r, r.finish_reason)
                done.append(r)
                continue
            idx = len(r.output) - r.pending
            r.output[idx] = tok
            r.pending -= 1
            reason = None
            if tok in r.eos_token_ids:
                reason = "stop"
            elif idx + 1 >= r.max_tokens or len(r.prompt) + idx + 1 >= self.max_seq_len:
                reason = "length"
            if reason is None:
                continue
            del r.output[idx + 1:]
            if r.pending:                                    # the step in flight still works on its pages
                r.pending = 0
                r.discard = True
                r.finish_reason = reason
                r.status = "finishing"
                self.running.remove(r)
                self.finishing.append(r)
            else:
                self._finish(r, reason)
                done.append(r)
        return done

    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """advance + resolve in one go, for a step whose tokens are read right away."""
        self.advance(plan)
        return self.resolve(plan, sampled)
