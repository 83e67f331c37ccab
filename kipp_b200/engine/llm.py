"""The Python entry point: token ids in, token ids out.

The reference has no Python entry to its engine (Python is tooling only,
docs/ARCHITECTURE.md:25-26); this one follows its C API's vocabulary
(src/kipp.h: open a model, evaluate, sample) and its CLI's option names
(src/kipp_cli.c:571-610): ``decode`` = tokens to generate, ``temperature`` 0 =
greedy, ``top_p``, ``top_k``, ``min_p``, ``seed``.  Generation itself (plan a
step, run it, sample, record) is the host core's loop (``kipp_engine_run``,
csrc/host/scheduler.hpp); the command line and the benchmark go through the
same loop.
"""
from __future__ import annotations

import ctypes
import dataclasses
import time
from typing import Optional, Sequence

from ..config.base import ModelConfig
from ..sampling.params import SamplingParams
from .engine import Engine
from .scheduler import Request, Scheduler


@dataclasses.dataclass
class GenerationResult:
    request_id: object
    prompt: list
    tokens: list                       # generated token ids
    finish_reason: str                 # "stop" | "length" | "abort"
    preemptions: int = 0


class LLM:
    """A model on one GPU with a scheduler above it.

    ``model``            folder with config.json + safetensors, or a ModelConfig
                         (random weights from ``seed``)
    ``dtype``            "bfloat16" (serving kernels) or "float32" (true 32-bit)
    ``kv_block_size``    tokens per cache page
    ``kv_blocks``        pages in each cache group (default: what the free device
                         memory holds, at most ``ctx`` tokens of ``max_requests`` requests)
    ``ctx``              most tokens one request may hold (default: the model's
                         max_position_embeddings)
    ``max_batch_tokens`` token budget of one step
    ``chunk``            largest prompt portion of one request in one step
    ``policy``           "reserve" or "preempt": what happens when pages run out
    """

    def __init__(self, model, *, dtype="bfloat16", device="cuda:0", kv_block_size: int = 16,
                 kv_blocks: Optional[int] = None, kv_tokens: Optional[int] = None,
                 ctx: Optional[int] = None, max_requests: int = 64, max_batch_tokens: int = 8192,
                 chunk: Optional[int] = None, policy: str = "reserve", seed: int = 0,
                 stop_token_ids: Sequence[int] = (), sigma: Optional[float] = None, norm_jitter: float = 0.1,
                 **engine_options):
        if kv_blocks is not None:
            cache_tokens = kv_blocks * kv_block_size
        elif kv_tokens is not None:
            cache_tokens = kv_tokens
        else:
            cache_tokens = None                       # sized from the free device memory
        opts = dict(dtype=dtype, device=device, page_size=kv_block_size, max_requests=max_requests,
                    max_batch_tokens=max_batch_tokens, cache_tokens=cache_tokens, **engine_options)
        if isinstance(model, ModelConfig):
            self.engine = Engine.from_config(model, seed, sigma=sigma, norm_jitter=norm_jitter, **opts)
        else:
            self.engine = Engine.from_folder(model, **opts)
        limit = self.engine.info()["max_positions"] or 8192
        self.ctx = min(ctx, limit) if ctx else limit
        self.chunk = chunk
        self.policy = policy
        self.max_batch_tokens = max_batch_tokens
        self.stop_token_ids = tuple(stop_token_ids)
        eos = getattr(self.engine.spec.config, "eos_token_id", None)
        if eos is not None and not self.stop_token_ids:
            self.stop_token_ids = (int(eos),)
        self.metrics: dict = {}
        self.step_log: list = []

    def new_scheduler(self) -> Scheduler:
        """The engine's own scheduler, set up anew with this object's options."""
        e = self.engine
        return Scheduler(e.cache, max_batch_tokens=self.max_batch_tokens, chunk_size=self.chunk,
                         max_positions=self.ctx, policy=self.policy, engine=e)

    def generate(self, prompts: Sequence[Sequence[int]], decode: int = 16, *,
                 temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0,
                 seed: int = 1, sampling: Optional[Sequence[SamplingParams]] = None,
                 stop_token_ids: Optional[Sequence[int]] = None) -> list:
        """Generate up to ``decode`` tokens for every prompt (lists of token ids).
        Request i samples with seed ``seed + i`` (never 0), as the reference
        seeds its choices (src/kipp_server.c:1852-1862)."""
        sched = self.new_scheduler()
        stops = tuple(stop_token_ids) if stop_token_ids is not None else self.stop_token_ids
        requests = []
        for i, prompt in enumerate(prompts):
            sp = sampling[i] if sampling is not None else SamplingParams(
                temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                seed=(seed + i) or 1)
            r = Request(id=i, prompt=[int(t) for t in prompt], max_new_tokens=decode, sampling=sp,
                        stop_token_ids=stops)
            sched.add(r)
            requests.append(r)
        self.run(sched)
        return [GenerationResult(r.id, r.prompt, list(r.output), r.finish_reason or "abort",
                                 r.preemptions) for r in requests]

    def run(self, sched: Scheduler, record_steps: bool = False) -> None:
        """Drive ``sched`` (the engine's scheduler) until no request is left.  With
        ``record_steps`` the loop is run one step at a time and every step's wall
        time (token ids on the host before, sampled ids on the host after) goes to
        ``self.step_log``."""
        engine = self.engine
        lib, h = engine._lib, engine._h
        steps = ctypes.c_int()
        self.step_log = []
        t0 = time.perf_counter()
        total = 0
        if not record_steps:
            engine._check(lib.kipp_engine_run(h, 0, ctypes.byref(steps)))
            total = steps.value
        else:
            before = sched.stats
            while sched.has_work():
                t_step = time.perf_counter()
                engine._check(lib.kipp_engine_run(h, 1, ctypes.byref(steps)))
                engine.synchronize()
                seconds = time.perf_counter() - t_step
                after = sched.stats
                fed = after["tokens_fed"] - before["tokens_fed"]
                sampled = after["tokens_sampled"] - before["tokens_sampled"]
                # a step that feeds more tokens than it samples carries a prompt portion
                self.step_log.append({"seconds": seconds, "tokens": fed, "sampled": sampled,
                                      "prefill": fed > sampled or fed == 0, "decode_only": fed == sampled and fed > 0,
                                      "h2d_bytes": engine.last_h2d_bytes, "d2h_bytes": 4 * sampled})
                before = after
                total += steps.value
        sched.sync()
        engine.synchronize()
        self.metrics = {"steps": total, "seconds": time.perf_counter() - t0, **sched.stats}
