"""The scheduler above ``step``: admits requests, cuts prompts into portions
under a token budget, decodes, finishes and frees.

It is the reference's server loop without sockets (src/kipp_server.c): FIFO
admission with head-of-line blocking (:2514-2531), a prompt portion for each
request still prefilling beside one token for each decoding request (step_eval,
:2044-2125), sample-then-eval (:2533-2535), "stop" on a stop token (the token
is not kept, :1937-1940) and "length" when max_tokens are made (:1970-1971).
Where the reference gives every prefilling request a fixed 32-token portion and
has no budget (:62, docs/ROADMAP.md:19-20), this one fills a per-step token
budget: decoded tokens first, then prompt portions in arrival order.

What happens when pages run out is decided by ``policy``:

``"reserve"``  (default, the reference's rule, src/kipp_server.c:1736-1777): a
    request is admitted only if every group's free pages cover its own peak
    need plus what the running requests may still take; so a step can never
    fail for pages, and requests wait in the queue instead.
``"preempt"``  a request is admitted as soon as its first portion fits.  If a
    later step does not fit, the youngest running request is put back at the
    head of the queue, its pages are freed, and it is recomputed from its
    prompt plus the tokens it had generated; the oldest request always
    proceeds.

The scheduler talks to the cache manager only (host bookkeeping) and never to
the device, so its decisions are tested without a GPU.
"""
from __future__ import annotations

import dataclasses
import enum
from collections import deque
from typing import Optional

from ..cache import CacheManager
from ..sampling.params import MASK64, RECENT_WINDOW, SamplingParams
from .batch import StepEntry


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclasses.dataclass
class Request:
    id: object
    prompt: list
    max_new_tokens: int
    sampling: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    stop_token_ids: tuple = ()
    # -- scheduler-owned ---------------------------------------------------------
    state: RequestState = RequestState.WAITING
    output: list = dataclasses.field(default_factory=list)
    finish_reason: Optional[str] = None
    fed: int = 0                       # tokens of prompt + output already in the cache
    rng_state: int = 1
    arrival: int = 0
    preemptions: int = 0
    last_logits = None                 # optional: logits of the last sampled position

    @property
    def all_tokens(self) -> list:
        return self.prompt + self.output

    def tokens_between(self, a: int, b: int) -> list:
        """Tokens [a, b) of prompt + output, without building the whole list
        (a decoding request asks for one token every step)."""
        n = len(self.prompt)
        if b <= n:
            return self.prompt[a:b]
        if a >= n:
            return self.output[a - n:b - n]
        return self.prompt[a:] + self.output[:b - n]

    @property
    def pending(self) -> int:
        """Tokens known but not yet in the cache."""
        return len(self.prompt) + len(self.output) - self.fed

    @property
    def total_budget(self) -> int:
        """Most tokens the request can ever hold in the cache."""
        return len(self.prompt) + self.max_new_tokens

    @property
    def recent(self) -> list:
        """The window penalties look back over: the last generated tokens
        (choice_remember_token, src/kipp_server.c:1019-1027)."""
        return self.output[-RECENT_WINDOW:]


@dataclasses.dataclass
class StepPlan:
    entries: list                      # list[StepEntry]
    requests: list                     # list[Request], parallel to entries
    sampled: list                      # indices of entries whose logits are sampled

    @property
    def tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batch_tokens: int, chunk_size: Optional[int] = None,
                 max_running: Optional[int] = None, max_positions: Optional[int] = None,
                 policy: str = "reserve", admit=None, release=None):
        """``admit(rid)`` / ``release(rid)`` take and give back a request's slot
        and pages; they default to the cache manager's own (an engine passes
        its ``add_request`` / ``finish`` so that per-request state is zeroed)."""
        if policy not in ("reserve", "preempt"):
            raise ValueError("policy must be 'reserve' or 'preempt'")
        if max_batch_tokens <= 0:
            raise ValueError("max_batch_tokens must be positive")
        self.cache = cache
        self._admit = admit or cache.admit
        self._release = release or cache.release
        self.max_batch_tokens = max_batch_tokens
        self.chunk_size = chunk_size or max_batch_tokens
        self.max_running = min(max_running or cache.slots.max_requests, cache.slots.max_requests)
        self.max_positions = max_positions
        self.policy = policy
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self._arrivals = 0
        self.stats = {"preemptions": 0, "steps": 0, "admitted": 0}

    # -- intake ----------------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if request.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        request.sampling.validate()
        if self.max_positions is not None and request.total_budget > self.max_positions:
            # the reference rejects prompt + max_tokens > context (src/kipp_server.c:1676-1684)
            raise ValueError(f"request {request.id!r}: prompt + max_new_tokens "
                             f"({request.total_budget}) exceeds the context of {self.max_positions}")
        for g in self.cache.groups:
            if g.peak_pages(request.total_budget, self._step_cap()) > g.pool.n_pages:
                raise ValueError(f"request {request.id!r} can never fit: it needs more pages than "
                                 f"group {g.index} has ({g.pool.n_pages})")
        seed = request.sampling.seed & MASK64
        request.rng_state = seed if seed else 1
        request.arrival = self._arrivals
        self._arrivals += 1
        request.state = RequestState.WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- page arithmetic ---------------------------------------------------------------
    def _step_cap(self) -> int:
        return min(self.chunk_size, self.max_batch_tokens)

    def _outstanding(self, group) -> int:
        """Pages the running requests may still take in ``group``."""
        total = 0
        for r in self.running:
            held = self.cache.pages_held(r.id)[group.index]
            total += max(0, group.peak_pages(r.total_budget, self._step_cap()) - held)
        return total

    def _can_admit(self, request: Request) -> bool:
        if len(self.running) >= self.max_running or self.cache.slots.free_slots == 0:
            return False
        for g in self.cache.groups:
            if self.policy == "reserve":
                need = g.peak_pages(request.total_budget, self._step_cap())
                if g.pool.free_pages < need + self._outstanding(g):
                    return False
            else:
                first = min(request.pending, self._step_cap())
                if g.pool.free_pages < -(-first // g.page_size):
                    return False
        return True

    def _admit_waiting(self) -> None:
        while self.waiting and self._can_admit(self.waiting[0]):   # head-of-line blocking
            r = self.waiting.popleft()
            self._admit(r.id)
            r.state = RequestState.RUNNING
            r.fed = 0
            self.running.append(r)
            self.stats["admitted"] += 1

    # -- planning ------------------------------------------------------------------------
    def _plan(self) -> StepPlan:
        budget = self.max_batch_tokens
        entries, requests, sampled = [], [], []
        # decoding requests first: one token each
        for r in self.running:
            if r.pending == 1 and r.fed >= len(r.prompt) and budget > 0:
                entries.append(StepEntry(r.id, r.tokens_between(r.fed, r.fed + 1), [0]))
                requests.append(r)
                sampled.append(len(entries) - 1)
                budget -= 1
        # then prompt portions (and recomputation after a preemption) in arrival order
        for r in self.running:
            if budget <= 0:
                break
            if r.pending == 1 and r.fed >= len(r.prompt):
                continue
            n = min(r.pending, self.chunk_size, budget)
            if n <= 0:
                continue
            toks = r.tokens_between(r.fed, r.fed + n)
            last = r.fed + n == len(r.prompt) + len(r.output)
            want = [n - 1] if last and len(r.output) < r.max_new_tokens else []
            entries.append(StepEntry(r.id, toks, want))
            requests.append(r)
            if want:
                sampled.append(len(entries) - 1)
            budget -= n
        return StepPlan(entries, requests, sampled)

    def _fits(self, plan: StepPlan) -> bool:
        need = [0] * len(self.cache.groups)
        for e, r in zip(plan.entries, plan.requests):
            for gi, m in enumerate(self.cache.missing_pages(r.id, r.fed + len(e.tokens))):
                need[gi] += m
        return all(n <= g.pool.free_pages for n, g in zip(need, self.cache.groups))

    def _preempt_youngest(self) -> bool:
        if len(self.running) <= 1:
            return False
        victim = max(self.running, key=lambda r: r.arrival)
        self.running.remove(victim)
        self._release(victim.id)
        victim.state = RequestState.WAITING
        victim.fed = 0
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)
        return True

    def schedule(self) -> Optional[StepPlan]:
        """The next step's batch, or None when nothing can run."""
        # finished-at-zero requests (max_new_tokens == 0) still prefill nothing
        self._admit_waiting()
        while True:
            if not self.running:
                return None
            plan = self._plan()
            if not plan.entries:
                return None
            if self._fits(plan):
                self.stats["steps"] += 1
                return plan
            if self.policy == "reserve":
                raise RuntimeError("reservation failed to keep a step within the pool")
            if not self._preempt_youngest():
                # one request alone does not fit: shrink its portion to what does
                r = plan.requests[0]
                g_free = min(g.pool.free_pages * g.page_size for g in self.cache.groups)
                room = g_free + (-r.fed) % self.cache.page_size
                if room <= 0:
                    raise RuntimeError(f"request {r.id!r} cannot grow: the pool is exhausted")
                e = plan.entries[0]
                n = min(len(e.tokens), room)
                last = r.fed + n == len(r.prompt) + len(r.output)
                plan = StepPlan([StepEntry(r.id, e.tokens[:n], [n - 1] if last and e.want else [])],
                                [r], [0] if last and e.want else [])
                if not self._fits(plan):
                    raise RuntimeError(f"request {r.id!r} cannot grow: the pool is exhausted")
                self.stats["steps"] += 1
                return plan

    # -- after the step -------------------------------------------------------------------
    def complete(self, plan: StepPlan, tokens: list) -> list:
        """Record a finished step.  ``tokens[i]`` is the token sampled for
        ``plan.sampled[i]``.  The cache manager's lengths must already have
        advanced (``Engine.step`` does that).  Returns the requests that finished."""
        if len(tokens) != len(plan.sampled):
            raise ValueError("one sampled token per sampled entry")
        for e, r in zip(plan.entries, plan.requests):
            r.fed += len(e.tokens)
        done = []
        for idx, tok in zip(plan.sampled, tokens):
            r = plan.requests[idx]
            tok = int(tok)
            if tok in r.stop_token_ids:
                r.finish_reason = "stop"              # the stop token is not kept
            else:
                r.output.append(tok)
                if len(r.output) >= r.max_new_tokens:
                    r.finish_reason = "length"
                elif self.max_positions is not None and len(r.prompt) + len(r.output) >= self.max_positions:
                    r.finish_reason = "length"
            if r.finish_reason is not None:
                done.append(r)
        for r in list(self.running):
            if r.finish_reason is None and r.max_new_tokens == 0 and r.pending == 0:
                r.finish_reason = "length"
                done.append(r)
        for r in done:
            self._finish(r)
        return done

    def _finish(self, r: Request) -> None:
        r.state = RequestState.FINISHED
        self.running.remove(r)
        self._release(r.id)                            # pages and slot go back at once
        self.finished.append(r)

    def abort(self, request_id) -> None:
        for r in list(self.running):
            if r.id == request_id:
                r.finish_reason = "abort"
                self._finish(r)
                return
        for r in list(self.waiting):
            if r.id == request_id:
                self.waiting.remove(r)
                r.state, r.finish_reason = RequestState.FINISHED, "abort"
                self.finished.append(r)
                return
