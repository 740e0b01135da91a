"""The scheduler above the step function: it admits requests, cuts prompts into
portions under a token budget, decodes, finishes and frees.

One central loop owns the GPU (the reference has no central loop: every call
runs on its caller's thread and a leader batches pending passes,
src/core/engine.cpp:1483-1540, 1842-2041; what is kept of it is what a pass may
hold: prompt portions of some sequences beside single decode tokens of others,
engine.cpp:2017-2030, and the finishing rules of the generation loop,
engine.cpp:4351-4393).

Decisions, all made on the host from the cache manager's accounting, so they
run and are tested without a GPU:

* Every unfinished request has `tokens` (prompt + generated so far) of which
  `n_computed` are in the cache; it always has at least one token pending.  A
  request whose pending tokens all fit a step gets a new token sampled at the
  end of that step.
* A step's token budget (`max_batched_tokens`) is spent first on requests with
  one pending token (decoding), then on running requests in the middle of a
  prompt, then on newly admitted ones; the last portion is cut to what is left
  of the budget, down to a single token.
* A waiting request is admitted, first come first served, while fewer than
  `max_requests` are running and the free pages, after what the step already
  plans to take, would hold its whole prompt plus one token.
* When pages run out for the tokens that running requests need, the most
  recently admitted running request is preempted: its pages are given back and
  it returns to the front of the waiting queue, to be recomputed later from its
  prompt and the tokens it had generated (its random draws are indexed by
  position in its own stream, so it continues exactly as if never preempted).
  A request that is alone and still cannot get a page can never finish: it ends
  with CONTEXT_FULL.  (The reference fails the pass and clears that sequence's
  context, src/core/transformer.cpp:6652-6654, src/core/engine.cpp:3878-3882.)
* A request finishes on its end-of-sequence token (unless told to ignore it),
  at `max_tokens`, when its sequence fills the model's positions, when its
  callback returns False, or when cancelled; its pages and state slot are freed
  at once.  The last sampled token is returned but never run, as in the
  reference (engine.cpp:4388-4393).
* A step is accounted for in two halves, so that the host can run one step ahead of
  the GPU: `begin_step` (right after the step is launched) advances every request and
  appends a placeholder for each token the step will sample; `finish_step` (when the
  sampled ids have arrived) puts the real tokens in, calls callbacks and finishes
  requests.  Between the two, the next step may already be planned and launched with
  the placeholders standing for tokens that are still on the device.  What the length
  limits decide is known at `begin_step`; what depends on a token's value (end of
  sequence, a callback's verdict) is decided at `finish_step`, one step later, so a
  request may have run one token too many; that token is dropped.  `update` is both
  halves at once.
"""
from __future__ import annotations

import collections
import enum
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.pages import CacheManager
from ..sampling.params import SamplingParams, uniform_draw
from ..status import ErrorCode, LiyabError, invalid_argument


PLACEHOLDER = -1        # stands in a request's tokens for an id sampled by a step whose result is not back yet


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    callback: Optional[Callable[[int], bool]] = None      # called with each new token; False stops
    state: RequestState = RequestState.WAITING
    tokens: List[int] = field(default_factory=list)       # prompt + generated
    n_computed: int = 0                                   # tokens already in the cache
    finish_reason: Optional[str] = None                   # "eos", "length", "context", "stopped", "cancelled", "error"
    error: Optional[LiyabError] = None
    cancelled: bool = False
    preemptions: int = 0
    seed: int = 0
    stream: int = 0
    admitted_at: int = -1
    sample_slot: int = -1                                 # where the step in flight will put this request's token

    @property
    def generated(self) -> List[int]:
        return self.tokens[len(self.prompt):]

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.n_computed

    @property
    def unresolved(self) -> bool:
        """Whether the last token is still a placeholder for an id that has not come back from the device."""
        return bool(self.tokens) and self.tokens[-1] == PLACEHOLDER

    def next_uniform(self) -> float:
        """The draw for this request's next generated token."""
        return uniform_draw(self.seed, self.stream, len(self.tokens) - len(self.prompt))


@dataclass
class PlannedEntry:
    request: Request
    start: int          # first token of the portion (index into request.tokens)
    count: int
    sample: bool        # the portion ends the known tokens: a new token is sampled after it
    token_index: int = -1   # where in request.tokens the sampled token goes (set by begin_step)
    ends: Optional[str] = None  # the length limit that this very token reaches, if any (set by begin_step)

    @property
    def tokens(self) -> List[int]:
        return self.request.tokens[self.start:self.start + self.count]


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    preempted: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(e.count for e in self.entries)


@dataclass
class SchedulerStats:
    steps: int = 0
    batched_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    peak_running: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, max_positions: int, max_batched_tokens: int = 2048, max_requests: int = 64,
                 eos_token_id: Optional[int] = None):
        if max_batched_tokens <= 0 or max_requests <= 0:
            raise invalid_argument("max_batched_tokens and max_requests must be positive")
        self.cache = cache
        self.max_positions = max_positions
        self.max_batched_tokens = max_batched_tokens
        self.max_requests = min(max_requests, cache.max_requests)
        self.eos_token_id = eos_token_id
        self.waiting: Deque[Request] = collections.deque()
        self.running: List[Request] = []
        self.stats = SchedulerStats()
        self._admissions = 0
        self._streams = 0

    # -- requests ---------------------------------------------------------------

    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise invalid_argument(f"request {request.id!r} has an empty prompt")
        if len(request.prompt) > self.max_positions:
            raise LiyabError(ErrorCode.CONTEXT_FULL, f"request {request.id!r}: a prompt of {len(request.prompt)} "
                             f"tokens does not fit {self.max_positions} positions")
        request.tokens = list(request.prompt)
        request.n_computed = 0
        request.state = RequestState.WAITING
        request.seed = request.params.resolved_seed()
        request.stream = self._streams
        self._streams += 1
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def cancel(self, request_id: Hashable) -> None:
        for r in list(self.running) + list(self.waiting):
            if r.id == request_id:
                r.cancelled = True

    # -- planning -----------------------------------------------------------------

    def _pages_for(self, n_tokens: int) -> int:
        ps = self.cache.page_size
        return (n_tokens + ps - 1) // ps

    def _finish(self, r: Request, reason: str, error: Optional[LiyabError] = None) -> None:
        if r.state == RequestState.FINISHED:
            r.finish_reason = reason
            return
        if r.state == RequestState.RUNNING:
            self.running.remove(r)
            self.cache.close(r.id)
        elif r in self.waiting:
            self.waiting.remove(r)
        r.state = RequestState.FINISHED
        r.finish_reason = reason
        r.error = error
        self.stats.finished += 1

    def _preempt(self, r: Request) -> None:
        self.running.remove(r)
        self.cache.close(r.id)
        r.state = RequestState.WAITING
        r.n_computed = 0
        r.preemptions += 1
        self.waiting.appendleft(r)
        self.stats.preemptions += 1

    def plan(self) -> Tuple[StepPlan, List[Request]]:
        """The next step, and the requests that finished while planning (cancelled, or that can never fit)."""
        finished: List[Request] = []
        for r in [r for r in list(self.running) + list(self.waiting) if r.cancelled]:
            self._finish(r, "cancelled")
            finished.append(r)
        preempted: List[Request] = []
        while True:
            budget = self.max_batched_tokens
            entries: List[PlannedEntry] = []
            wants: Dict[Hashable, int] = {}
            order = [r for r in self.running if r.pending == 1] + [r for r in self.running if r.pending > 1]
            for r in order:
                if budget == 0:
                    break
                n = min(r.pending, budget)
                entries.append(PlannedEntry(r, r.n_computed, n, sample=(n == r.pending)))
                wants[r.id] = n
                budget -= n
            if self.cache.can_reserve(wants):
                break
            # Pages ran out for what running requests need: the most recently admitted one makes room.
            victim = max(self.running, key=lambda r: r.admitted_at)
            if len(self.running) == 1:
                self._finish(victim, "error", LiyabError(
                    ErrorCode.CONTEXT_FULL, f"request {victim.id!r} needs more pages than the cache has "
                    f"({victim.n_computed + victim.pending} tokens, {self.cache.free_pages()} pages free)"))
                finished.append(victim)
            else:
                self._preempt(victim)
                preempted.append(victim)
        # Admission: first come first served, only what fits whole.
        while self.waiting and len(self.running) < self.max_requests and budget > 0 and not preempted:
            r = self.waiting[0]
            whole = self._pages_for(min(len(r.tokens) + 1, self.max_positions))
            total_pages = min(g.pool.num_pages for g in self.cache.groups) if self.cache.groups else whole
            if whole > total_pages:
                self.waiting.popleft()
                r.state = RequestState.WAITING
                self._finish(r, "error", LiyabError(
                    ErrorCode.CONTEXT_FULL, f"request {r.id!r}: {len(r.tokens)} tokens need {whole} pages, the cache "
                    f"has {total_pages}"))
                finished.append(r)
                continue
            self.cache.open(r.id)
            n = min(r.pending, budget)
            probe = dict(wants)
            probe[r.id] = len(r.tokens) + 1 if len(r.tokens) < self.max_positions else len(r.tokens)
            if not self.cache.can_reserve(probe):
                self.cache.close(r.id)
                break
            self.waiting.popleft()
            r.state = RequestState.RUNNING
            r.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(r)
            entries.append(PlannedEntry(r, r.n_computed, n, sample=(n == r.pending)))
            wants[r.id] = n
            budget -= n
        self.stats.peak_running = max(self.stats.peak_running, len(self.running))
        return StepPlan(entries=entries, preempted=preempted), finished

    # -- after the step was launched, and after its tokens came back ---------------------

    def begin_step(self, plan: StepPlan) -> None:
        """The step is on its way: its tokens count as computed, a placeholder stands for each token it
        samples, and a request that its length limits end is taken out of the running set already."""
        self.stats.steps += 1
        self.stats.batched_tokens += plan.n_tokens
        for e in plan.entries:
            r = e.request
            r.n_computed += e.count
            if e.count == 1 and r.n_computed > len(r.prompt):
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += e.count
            if not e.sample:
                continue
            r.tokens.append(PLACEHOLDER)
            e.token_index = len(r.tokens) - 1
            if len(r.tokens) - len(r.prompt) >= r.params.max_tokens:
                e.ends = "length"
            elif len(r.tokens) > self.max_positions:
                e.ends = "context"                # the new token has no position left to run at
            if e.ends is not None:
                self._finish(r, e.ends)

    def finish_step(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """The ids sampled for the plan's entries with `sample`, in the plan's order, have arrived.
        Returns the requests whose generation is now complete."""
        done: List[Request] = []
        it = iter(sampled)
        for e in plan.entries:
            if not e.sample:
                continue
            token = int(next(it))
            r = e.request
            if e.token_index >= len(r.tokens):
                continue                           # the request ended on an earlier token; this one was one too many
            r.tokens[e.token_index] = token
            keep_going = True
            if r.callback is not None:
                keep_going = r.callback(token) is not False
            reason = None
            if not r.params.ignore_eos and self.eos_token_id is not None and token == self.eos_token_id:
                reason = "eos"
            elif e.ends is not None:
                reason = e.ends                      # this token reached a length limit (known since begin_step)
            elif not keep_going:
                reason = "stopped"
            elif r.cancelled:
                reason = "cancelled"
            if reason is not None:
                del r.tokens[e.token_index + 1:]     # a placeholder of the step after this one, if any
                self._finish(r, reason)
                done.append(r)
        return done

    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Both halves at once, for a caller that waits for every step's tokens before planning the next."""
        self.begin_step(plan)
        return self.finish_step(plan, sampled)
