"""The scheduler above ``step``: admits requests, cuts prompts into portions
under a token budget, decodes, finishes and frees.  The decisions are the host
core's (csrc/host/scheduler.hpp); this module is their face: requests as Python
objects, plans as lists of ``StepEntry``.

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

import ctypes
import dataclasses
import enum
from collections import deque
from typing import Optional

from .. import native as N
from ..cache import CacheManager
from ..sampling.params import MASK64, RECENT_WINDOW, SamplingParams, to_native
from .batch import StepEntry


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


_REASONS = {0: None, 1: "stop", 2: "length", 3: "abort"}


@dataclasses.dataclass
class Request:
    id: object
    prompt: list
    max_new_tokens: int
    sampling: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    stop_token_ids: tuple = ()
    # -- mirrored from the scheduler -----------------------------------------------
    state: RequestState = RequestState.WAITING
    output: list = dataclasses.field(default_factory=list)
    finish_reason: Optional[str] = None
    fed: int = 0                       # tokens of prompt + output already in the cache
    rng_state: int = 1
    arrival: int = 0
    preemptions: int = 0

    @property
    def all_tokens(self) -> list:
        return self.prompt + self.output

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
                 policy: str = "reserve", engine=None):
        """Over a cache manager (the scheduler takes and gives back slots and pages
        itself), or, with ``engine``, over that engine's own scheduler, which
        ``Engine``/``LLM`` drive through ``kipp_engine_run``."""
        if policy not in ("reserve", "preempt"):
            raise ValueError("policy must be 'reserve' or 'preempt'")
        if max_batch_tokens <= 0:
            raise ValueError("max_batch_tokens must be positive")
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.chunk_size = chunk_size or max_batch_tokens
        self.max_positions = max_positions
        self.policy = policy
        self._lib = N.lib()
        self._engine = engine
        opt = N.SchedulerOptions(max_batch_tokens, int(chunk_size or 0), int(max_running or 0),
                                 int(max_positions or 0), 1 if policy == "preempt" else 0)
        if engine is not None:
            N.check(self._lib.kipp_engine_scheduler_configure(engine._h, ctypes.byref(opt)), engine=engine._h)
            self._h = self._lib.kipp_engine_scheduler(engine._h)
            self._owned = False
        else:
            ng = len(cache.groups)
            pages = (ctypes.c_int * max(ng, 1))(*[g.n_pages for g in cache.groups])
            windows = (ctypes.c_int * max(ng, 1))(*[int(g.window or 0) for g in cache.groups])
            h = ctypes.c_void_p()
            N.check(self._lib.kipp_scheduler_create(cache._h, ng, pages, windows, cache.page_size,
                                                    cache.slots.max_requests, ctypes.byref(opt), ctypes.byref(h)))
            self._h = h
            self._owned = True
        self._owners = cache._owners
        self._requests: dict = {}          # request id -> Request
        self._ints: dict = {}              # the library's number of a request -> its id
        self._numbers: dict = {}           # and back (a finished request's number is forgotten by the cache)
        self._arrivals = 0
        self.finished: list[Request] = []

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "_h", None):
            self._lib.kipp_scheduler_destroy(self._h)
            self._h = None

    def _check(self, rc: int) -> None:
        N.check(rc, scheduler=self._h)

    # -- intake ----------------------------------------------------------------------
    def add(self, request: Request) -> None:
        request.sampling.validate()
        params, keep = to_native([request.sampling])
        prompt = (ctypes.c_int32 * max(len(request.prompt), 1))(*[int(t) for t in request.prompt])
        stops = (ctypes.c_int32 * max(len(request.stop_token_ids), 1))(*[int(t) for t in request.stop_token_ids])
        seed = request.sampling.seed & MASK64
        known = request.id in self._owners
        g = N.GenerationRequest()
        g.id = self._owners.id_of(request.id, create=True)
        g.prompt, g.n_prompt = prompt, len(request.prompt)
        g.max_new_tokens = request.max_new_tokens
        g.sampling = params[0]
        g.seed = seed
        g.stop_tokens, g.n_stop_tokens = stops, len(request.stop_token_ids)
        try:
            self._check(self._lib.kipp_scheduler_submit(self._h, ctypes.byref(g)))
        except Exception:
            if not known:
                self._owners.forget(request.id)
            raise
        del keep
        request.rng_state = seed if seed else 1
        request.arrival = self._arrivals
        self._arrivals += 1
        request.state = RequestState.WAITING
        self._requests[request.id] = request
        self._ints[int(g.id)] = request.id
        self._numbers[request.id] = int(g.id)

    def has_work(self) -> bool:
        return bool(self._lib.kipp_scheduler_has_work(self._h))

    def _ids(self, which: int) -> list:
        n = ctypes.c_int()
        cap = max(len(self._requests), 1)
        buf = (ctypes.c_int64 * cap)()
        self._check(self._lib.kipp_scheduler_list(self._h, which, buf, cap, ctypes.byref(n)))
        return [self._ints[int(buf[i])] for i in range(min(n.value, cap))]

    @property
    def waiting(self) -> deque:
        return deque(self._requests[i] for i in self._ids(0))

    @property
    def running(self) -> list:
        return [self._requests[i] for i in self._ids(1)]

    @property
    def stats(self) -> dict:
        out = (ctypes.c_longlong * 5)()
        self._lib.kipp_scheduler_stats(self._h, out)
        return {"preemptions": int(out[0]), "steps": int(out[1]), "admitted": int(out[2]),
                "tokens_fed": int(out[3]), "tokens_sampled": int(out[4])}

    def _refresh(self, request: Request) -> None:
        i = self._numbers[request.id]
        st = N.GenerationState()
        self._check(self._lib.kipp_scheduler_poll(self._h, i, ctypes.byref(st)))
        if st.n_tokens != len(request.output):
            buf = (ctypes.c_int32 * max(st.n_tokens, 1))()
            n = ctypes.c_int()
            self._check(self._lib.kipp_scheduler_output(self._h, i, buf, st.n_tokens, ctypes.byref(n)))
            request.output = [int(buf[k]) for k in range(st.n_tokens)]
        request.preemptions = st.preemptions
        request.finish_reason = _REASONS.get(st.reason)
        request.rng_state = int(self._lib.kipp_scheduler_rng_state(self._h, i))
        if st.finished:
            request.state = RequestState.FINISHED

    def sync(self) -> list:
        """Bring the Python requests up to date with the scheduler; returns the
        requests that have finished since the last call."""
        waiting, running = set(self._ids(0)), set(self._ids(1))
        done = []
        for rid in self._ids(2):
            r = self._requests[rid]
            if r.state is not RequestState.FINISHED:
                self._refresh(r)
                r.state = RequestState.FINISHED
                self.finished.append(r)
                done.append(r)
                if not self._live_in_cache(rid):
                    self._owners.forget(rid)
        for rid, r in self._requests.items():
            if rid in running:
                r.state = RequestState.RUNNING
                self._refresh(r)
            elif rid in waiting:
                if r.state is RequestState.RUNNING:          # put back by a preemption
                    r.fed = 0
                r.state = RequestState.WAITING
                self._refresh(r)
        return done

    def _live_in_cache(self, rid) -> bool:
        i = self._owners.id_of(rid)
        return bool(i) and self.cache._lib.kipp_cm_slot(self.cache._h, i) >= 0

    # -- planning ------------------------------------------------------------------------
    def schedule(self) -> Optional[StepPlan]:
        """The next step's batch, or None when nothing can run."""
        cap = max(len(self._requests), 1)
        buf = (N.PlanEntry * cap)()
        n = ctypes.c_int()
        self._check(self._lib.kipp_scheduler_schedule(self._h, buf, cap, ctypes.byref(n)))
        self.sync()
        if n.value == 0:
            return None
        entries, requests, sampled = [], [], []
        for k in range(n.value):
            pe = buf[k]
            r = self._requests[self._ints[int(pe.id)]]
            toks = (ctypes.c_int32 * pe.n_tokens)()
            self._check(self._lib.kipp_scheduler_tokens(self._h, pe.id, pe.first, pe.n_tokens, toks))
            r.fed = pe.first
            entries.append(StepEntry(r.id, [int(t) for t in toks], [pe.n_tokens - 1] if pe.want_last else []))
            requests.append(r)
            if pe.want_last:
                sampled.append(k)
        return StepPlan(entries, requests, sampled)

    # -- after the step -------------------------------------------------------------------
    def complete(self, plan: StepPlan, tokens: list) -> list:
        """Record a finished step.  ``tokens[i]`` is the token sampled for
        ``plan.sampled[i]``.  The cache manager's lengths must already have
        advanced (the step does that).  Returns the requests that finished."""
        if len(tokens) != len(plan.sampled):
            raise ValueError("one sampled token per sampled entry")
        buf = (ctypes.c_int32 * max(len(tokens), 1))(*[int(t) for t in tokens])
        self._check(self._lib.kipp_scheduler_complete(self._h, buf, len(tokens)))
        for e, r in zip(plan.entries, plan.requests):
            r.fed += len(e.tokens)
        return self.sync()

    def abort(self, request_id) -> None:
        self._check(self._lib.kipp_scheduler_abort(self._h, self._numbers[request_id]))
        self.sync()
