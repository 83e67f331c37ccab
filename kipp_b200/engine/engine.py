"""The engine: a model bound to a device, its cache, and the step function.

``step`` takes a batch of (request, its next tokens) — portions of prompts
beside single decoded tokens, cut anywhere — runs exactly those tokens as one
batch against the cache that earlier steps left, and returns the logits at the
wanted places.  It generalises the reference's ``kipp_eval_batch``
(src/kipp.c:3984-4082): any mixture of items, nothing changes on error, lengths
advance on success.
"""
from __future__ import annotations

import dataclasses
from typing import Iterable, Optional

import torch

from ..cache import CacheManager, OutOfPages
from ..config.base import ModelConfig
from ..config.registry import get_architecture, load_config
from ..models.spec import LayerRun, ModelSpec
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors
from .batch import Staging, StepEntry, StepMeta, pack_step
from .runtime import Runtime


@dataclasses.dataclass
class CacheView:
    k_pages: Optional[torch.Tensor]      # [pages, kv_heads, page_size, head_dim] of one run's cache
    v_pages: Optional[torch.Tensor]
    block_table: torch.Tensor            # int32 [entries, width] for this step
    page_size: int


class StepContext:
    """What a part sees during one step."""

    def __init__(self, engine: "Engine", meta: StepMeta):
        rt = engine.runtime
        self.engine = engine
        self.meta = meta
        self.device = rt.device
        self.dtype = rt.dtype
        self.ops = rt.ops
        self.workspace = rt.workspace
        self.status = rt.status
        self.step_cache: dict = {}       # what parts share within ONE forward pass (e.g. rotary tables)

    def cache_view(self, run: LayerRun) -> CacheView:
        gi, j = self.engine.cache.group_of_cache[run.cache]
        g = self.engine.cache.groups[gi]
        return CacheView(g.k[j], g.v[j], self.meta.block_tables[gi], g.page_size)

    def state_view(self, run: LayerRun) -> torch.Tensor:
        """[max_requests, *shape] state of this run's cache id; index it with
        ``meta.slots``."""
        return self.engine.states[run.cache]


class Engine:
    def __init__(self, spec: ModelSpec, tensors: dict, *, dtype="bfloat16",
                 device: str | torch.device = "cuda:0", page_size: int = 16,
                 cache_tokens: int = 8192, max_requests: int = 64,
                 max_batch_tokens: int = 8192, cuda_graphs: bool = True):
        self.spec = spec
        self.runtime = Runtime(device, dtype)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_batch_tokens = max_batch_tokens
        rt = self.runtime
        self._check_device_memory(cache_tokens)
        with torch.cuda.device(rt.device):
            # -- weights -------------------------------------------------------
            spec.embedding.bind(tensors, spec.embedding_prefix, rt)
            for prefix, block in spec.layers:
                block.bind(tensors, prefix, rt)
            spec.final_norm[1].bind(tensors, spec.final_norm[0], rt)
            spec.head[1].bind(tensors, spec.head[0], rt)
            # -- cache ------------------------------------------------------------
            cache_specs, state_specs = {}, {}
            for run in spec.order:
                mixer = spec.layers[run.layer][1].mixer
                cs, ss = mixer.cache_spec(), mixer.state_spec()
                if cs is not None:
                    if cache_specs.setdefault(run.cache, cs) != cs:
                        raise ValueError(f"runs that share cache {run.cache} need equal cache specs")
                if ss is not None:
                    if state_specs.setdefault(run.cache, ss) != ss:
                        raise ValueError(f"runs that share cache {run.cache} need equal state specs")
            n_pages = max(1, -(-cache_tokens // page_size))
            self.cache = CacheManager(cache_specs, page_size, n_pages, max_requests)
            for g in self.cache.groups:
                shape = (len(g.cache_ids), n_pages, g.spec.kv_heads, page_size, g.spec.head_dim)
                g.k = torch.zeros(shape, dtype=rt.dtype, device=rt.device)
                g.v = torch.zeros(shape, dtype=rt.dtype, device=rt.device)
            self.states = {cid: torch.zeros((max_requests,) + tuple(ss.shape), dtype=ss.dtype,
                                            device=rt.device)
                           for cid, ss in state_specs.items()}
        self._staging = Staging()
        # decode steps replay a captured graph per batch size (bfloat16 path)
        self.cuda_graphs = cuda_graphs and self.runtime.dtype == torch.bfloat16
        self._graphs: dict = {}
        self._shapes_seen: dict = {}
        self._last_decode_graph = None
        self.last_forward_launches = 0
        self.graph_replays = 0
        self.graph_kernel_launches = 0
        self.steps_run = 0
        self.last_h2d_bytes = 0

    def _check_device_memory(self, cache_tokens: int) -> None:
        """Refuse before anything is uploaded when weights and cache cannot fit
        (the reference does the same before its one allocation,
        src/cuda/kipp_cuda.cu:542-561)."""
        rt, spec = self.runtime, self.spec
        es = torch.empty((), dtype=rt.dtype).element_size()
        weights = 0
        for ts in spec.tensor_specs():
            if ts.optional and ts.alias_of is not None:
                continue
            n = 1
            for d in ts.shape:
                n *= d
            weights += n * es
        cache = 0
        seen = set()
        for run in spec.order:
            cs = spec.layers[run.layer][1].mixer.cache_spec()
            if cs is not None and run.cache not in seen:
                seen.add(run.cache)
                pages = max(1, -(-cache_tokens // self.page_size))
                cache += 2 * pages * self.page_size * cs.kv_heads * cs.head_dim * es
        need = weights + cache
        free, _total = torch.cuda.mem_get_info(rt.device)
        if need > free:
            raise MemoryError(f"the model needs about {need:,} device bytes ({weights:,} of weights, {cache:,} of "
                              f"cache for {cache_tokens:,} tokens) but only {free:,} are free on {rt.device}")

    # -- construction ------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str, **options) -> "Engine":
        """Load ``folder/config.json`` and its safetensors; the model class is
        chosen by ``architectures[0]``."""
        config = load_config(folder)
        spec = get_architecture(config.architecture).build(config)
        tensors = load_tensors(folder, spec.tensor_specs())
        return cls(spec, tensors, **options)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int, *, sigma: Optional[float] = None,
                    norm_jitter: float = 0.1, weight_dtype: torch.dtype = torch.bfloat16,
                    **options) -> "Engine":
        """Random weights made on the device (no files): for benchmarks of
        sizes too large to write out."""
        spec = get_architecture(config.architecture).build(config)
        device = options.get("device", "cuda:0")
        if sigma is None:
            sigma = float(getattr(config, "initializer_range", 0.02))
        tensors = _LazyRandom(spec.tensor_specs(), seed, sigma, norm_jitter, weight_dtype, device)
        return cls(spec, tensors, **options)

    # -- requests ------------------------------------------------------------------
    def add_request(self, rid) -> int:
        slot = self.cache.admit(rid)
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def finish(self, rid) -> None:
        """The request is over: its pages and its slot are given back."""
        self.cache.release(rid)

    def truncate(self, rid, new_length: int) -> None:
        """Cut a live request back to its first ``new_length`` tokens; the pages
        beyond go back.  A model whose mixers keep state per request can only be
        cut back to nothing (the state is then cleared): a state cannot be unwound."""
        if self.states and new_length != 0:
            raise ValueError("a model with per-request state can only be reset (truncate to 0)")
        self.cache.truncate(rid, new_length)
        if new_length == 0:
            slot = self.cache.slot(rid)
            for st in self.states.values():
                st[slot].zero_()

    def reset(self, rid) -> None:
        """The request keeps its slot and starts again from an empty context."""
        self.truncate(rid, 0)

    def length(self, rid) -> int:
        return self.cache.length(rid)

    def is_live(self, rid) -> bool:
        return rid in self.cache

    # -- the step ----------------------------------------------------------------------
    def step(self, entries: Iterable[StepEntry], *, check: bool = False) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits ``[wanted, vocab]`` on the
        device in the order of the entries and of their ``want`` lists (None if
        nothing is wanted).  The tensor is workspace memory: read or copy it
        before the next step.  Raises ``OutOfPages`` with no request changed
        when the cache cannot hold the step."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            return None
        vocab = self.spec.vocab_size
        seen = set()
        total = 0
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request!r} brings no tokens")
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                raise ValueError(f"request {e.request!r} has a token id outside [0, {vocab})")
            total += len(e.tokens)
        if total > self.max_batch_tokens:
            raise ValueError(f"step of {total} tokens exceeds max_batch_tokens {self.max_batch_tokens}")
        admitted = []
        try:
            for e in entries:
                if e.request not in self.cache:
                    self.add_request(e.request)
                    admitted.append(e.request)
            starts = [self.cache.length(e.request) for e in entries]
            limit = self.spec.max_positions
            for e, s in zip(entries, starts):
                if limit is not None and s + len(e.tokens) > limit:
                    raise ValueError(f"request {e.request!r} would pass max positions {limit}")
            self.cache.reserve([(e.request, s + len(e.tokens)) for e, s in zip(entries, starts)])
        except Exception:
            for rid in admitted:
                self.cache.release(rid)
            raise
        rids = [e.request for e in entries]
        slots = [self.cache.slot(r) for r in rids]
        rt = self.runtime
        with torch.cuda.device(rt.device):
            if self.cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
                logits = self._graph_step(entries, starts, slots, rids)
            elif self.cuda_graphs and self._shape_repeats(entries):
                # e.g. the 2,048-token chunks of long prompts: the third step of a shape
                # is captured, later ones replayed (the host then launches one graph
                # instead of nine kernels per layer)
                logits = self._graph_step(entries, starts, slots, rids, bucket=512, decode=False)
            else:
                tables = [self.cache.block_table_rows(rids, gi) for gi in range(len(self.cache.groups))]
                meta = pack_step(entries, starts, slots, tables, rt.device, self._staging)
                self.last_h2d_bytes = meta.extra["h2d_bytes"]
                logits = self._forward(StepContext(self, meta))
        for e, s in zip(entries, starts):
            self.cache.advance(e.request, s + len(e.tokens))
        self.steps_run += 1
        if check:
            rt.check_status()
        return logits

    def decode_burst(self, requests: list, tokens: list[int], steps: int) -> torch.Tensor:
        """Greedy decoding of ``steps`` tokens for every request without the host in
        the loop.  ``tokens[i]`` is the next token of ``requests[i]`` (its logits
        give the first new token).  Returns int32 ``[steps, len(requests)]`` on
        the device: row k holds the tokens chosen at step k.  The step is captured
        in a CUDA graph together with its argmax, the hand-over of the chosen
        tokens and the move of every request to its next position, so a burst is
        a run of graph replays with no copy and no other launch in between.  Pages for all steps are
        taken first (``OutOfPages`` leaves every request as it was).  Callers
        that must look at every token (stop tokens, sampling with penalties)
        use :meth:`step`."""
        from ..kernels import sampling as _sampling
        n = len(requests)
        if n == 0 or steps <= 0:
            return torch.empty((0, n), dtype=torch.int32, device=self.runtime.device)
        if len(tokens) != n:
            raise ValueError("one next token per request")
        rt = self.runtime
        for r in requests:
            if r not in self.cache:
                raise ValueError(f"decode_burst: request {r!r} is not live (feed its prompt with step())")
        starts = [self.cache.length(r) for r in requests]
        limit = self.spec.max_positions
        if limit is not None and max(starts) + steps > limit:
            raise ValueError(f"a request would pass max positions {limit}")
        # the pages of all steps are mapped first: all or nothing, and the block tables
        # then stay as they are from step to step
        self.cache.reserve([(r, s + steps) for r, s in zip(requests, starts)])
        ring = torch.empty((steps, n), dtype=torch.int32, device=rt.device)
        if not self.cuda_graphs:
            # no graphs (the 32-bit path): the same tokens, one step at a time
            cur = list(tokens)
            for k in range(steps):
                logits = self.step([StepEntry(r, [t], [0]) for r, t in zip(requests, cur)])
                _sampling.argmax_rows(logits, out=ring[k])
                cur = ring[k].tolist()
            return ring
        # a graph of the step that feeds itself: argmax, token feedback and the move to
        # the next position are captured behind the forward pass
        from .graphs import DecodeGraph
        with torch.cuda.device(rt.device):
            entries = [StepEntry(r, [t], [0]) for r, t in zip(requests, tokens)]
            slots = [self.cache.slot(r) for r in requests]
            widths, tables = self._table_widths(requests, 64)
            key = ("burst", n, tuple(widths))
            graph = self._graphs.pop(key, None)
            if graph is None:
                if len(self._graphs) >= 24:
                    self._graphs.pop(next(iter(self._graphs)))
                graph = DecodeGraph(self, n, widths, feedback=True)
            self._graphs[key] = graph
            ring = graph.run_burst(entries, starts, slots, tables, steps)
            for r, s in zip(requests, starts):
                self.cache.advance(r, s + steps)
            self.steps_run += steps
            self.graph_replays += steps
            self.graph_kernel_launches += steps * graph.launches
            self.last_h2d_bytes = graph.static.n_ints * 4
        return ring

    def _shape_repeats(self, entries) -> bool:
        """Whether steps of this shape (tokens and wanted rows per entry) have been
        run twice before: only shapes that keep coming back are worth a capture."""
        sig = tuple((len(e.tokens), len(e.want)) for e in entries)
        seen = self._shapes_seen
        n = seen.get(sig, 0)
        if n >= 2:
            return True
        if len(seen) >= 512:
            seen.clear()
        seen[sig] = n + 1
        return False

    def _table_widths(self, rids, bucket: int):
        """Block-table width per cache group for a captured step, and the tables: what
        the longest entry needs, rounded up to ``bucket`` pages so that a captured graph
        serves many steps and little is copied for short contexts."""
        limit = self.spec.max_positions
        widths = []
        for gi, g in enumerate(self.cache.groups):
            cap = g.pool.n_pages if limit is None else min(g.pool.n_pages, -(-limit // g.page_size))
            need = max(self.cache.table_len(r, gi) for r in rids)
            widths.append(max(1, min(max(cap, need), -(-(need + 1) // bucket) * bucket)))
        tables = [self.cache.block_table_rows(rids, gi, width=w) for gi, w in enumerate(widths)]
        return widths, tables

    def _graph_step(self, entries, starts, slots, rids, bucket: int = 64, decode: bool = True) -> torch.Tensor:
        from .graphs import DecodeGraph
        widths, tables = self._table_widths(rids, bucket)
        if decode:
            key = (len(entries), tuple(widths))
        else:
            key = (tuple((len(e.tokens), len(e.want)) for e in entries), tuple(widths))
        graph = self._graphs.pop(key, None)               # re-inserted below: the dict is kept in order of use
        if graph is None:
            if len(self._graphs) >= 24:
                self._graphs.pop(next(iter(self._graphs)))   # the least recently used
            if decode:
                graph = DecodeGraph(self, len(entries), widths)
            else:
                graph = DecodeGraph(self, len(entries), widths, [len(e.tokens) for e in entries],
                                    [len(e.want) for e in entries])
        self._graphs[key] = graph
        if decode:
            self._last_decode_graph = graph
        logits = graph.run(entries, starts, slots, tables)
        self.last_h2d_bytes = graph.static.n_ints * 4
        self.graph_replays += 1
        self.graph_kernel_launches += graph.launches
        return logits

    def kernel_launches(self) -> int:
        """Kernels of this package run so far: launched directly or replayed in graphs."""
        from ..kernels import ops as _kops
        return _kops.launch_count() + self.graph_kernel_launches

    def _forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        from ..kernels import ops as _kops
        launches0 = _kops.launch_count()
        try:
            return self._forward_impl(ctx)
        finally:
            self.last_forward_launches = _kops.launch_count() - launches0

    def _forward_impl(self, ctx: StepContext) -> Optional[torch.Tensor]:
        spec = self.spec
        x = spec.embedding.forward(ctx)
        for run in spec.order:
            spec.layers[run.layer][1].forward(ctx, run, x)
        meta = ctx.meta
        if meta.n_logit_rows == 0:
            return None
        h = spec.final_norm[1].forward(ctx, x, rows=meta.logit_rows, n_rows=meta.n_logit_rows,
                                       key="final_normed")
        return spec.head[1].forward(ctx, h, meta.n_logit_rows)

    # -- accounting -----------------------------------------------------------------
    def info(self) -> dict:
        """What is loaded and what it may hold (the reference's kipp_model_info and
        kipp_session_info in one, src/kipp.h:109-145, 172-200)."""
        cfg = self.spec.config
        groups = [{"caches": len(g.cache_ids), "kv_heads": g.spec.kv_heads, "head_dim": g.spec.head_dim,
                   "window": g.spec.window, "pages": g.pool.n_pages, "free_pages": g.pool.free_pages}
                  for g in self.cache.groups]
        return {"architecture": getattr(cfg, "architecture", None), "dtype": str(self.runtime.dtype),
                "device": str(self.runtime.device), "layers": len(self.spec.layers),
                "runs": len(self.spec.order), "hidden_size": self.spec.hidden_size,
                "vocab_size": self.spec.vocab_size, "max_positions": self.spec.max_positions,
                "weight_bytes": self.weight_bytes(), "cache_bytes_per_token": self.cache_bytes_per_token(),
                "page_size": self.page_size, "cache_groups": groups, "max_requests": self.max_requests,
                "max_batch_tokens": self.max_batch_tokens,
                "live_requests": {r: self.cache.length(r) for r in self.cache.live_requests()}}

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads (each weight once)."""
        spec = self.spec
        n = sum(spec.layers[run.layer][1].weight_bytes() for run in spec.order)
        n += spec.final_norm[1].weight_bytes() + spec.head[1].weight_bytes()
        return n

    def cache_bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.runtime.dtype).element_size()
        return sum(2 * len(g.cache_ids) * g.spec.kv_heads * g.spec.head_dim * es
                   for g in self.cache.groups)


class _LazyRandom(dict):
    """Mapping name -> random tensor made on first access and not kept, so that
    a large model never exists twice."""

    def __init__(self, specs, seed, sigma, norm_jitter, dtype, device):
        super().__init__()
        self._specs = {s.name: s for s in specs}
        self._args = (seed, sigma, norm_jitter, dtype, device)

    def __contains__(self, name) -> bool:
        s = self._specs.get(name)
        return s is not None and not (s.optional and s.alias_of is not None)

    def __getitem__(self, name):
        seed, sigma, jitter, dtype, device = self._args
        s = self._specs[name]
        for _, t in random_tensors([s], seed, sigma=sigma, norm_jitter=jitter, dtype=dtype,
                                   device=device, skip_aliased=False):
            return t
        raise KeyError(name)
