"""CUDA graphs for decode steps.

A step in which every entry brings one token has the same kernels, grids and
buffers whenever the number of entries is the same: only the contents of the
metadata buffer differ.  Such a step is captured once per batch size and
replayed; the host then pays for one copy of the metadata and one graph launch
instead of some three hundred kernel launches.  (The reference launches 18
kernels per layer and token from the host, src/cuda/kipp_cuda.cu:358-462.)
"""
from __future__ import annotations

import gc

from typing import Optional

import torch

from ..kernels import attention_bf16
from .batch import ATTENTION_TILE, StaticStep, StepMeta, pack_decode, pack_step, step_ints


class DecodeGraph:
    """The captured forward pass of steps of one shape: the same number of tokens
    and wanted rows per entry and the same block-table widths.  Built for decode
    steps (every entry one token); prompt portions of a repeating shape (the
    chunks of long prompts) use it too."""

    def __init__(self, engine, batch: int, table_widths: list[int], q_lens: Optional[list[int]] = None,
                 wants: Optional[list[int]] = None):
        self.engine = engine
        self.batch = batch
        self.table_widths = table_widths
        n = batch
        q_lens = [1] * n if q_lens is None else list(q_lens)
        wants = [1] * n if wants is None else list(wants)
        self.decode_only = all(q == 1 for q in q_lens) and all(w == 1 for w in wants)
        tile = ATTENTION_TILE
        ints = step_ints(n, sum(q_lens), sum(wants), sum(1 for q in q_lens if q == 1),
                         sum(-(-q // tile) for q in q_lens if q > 1), sum(-(-q // tile) for q in q_lens),
                         [n * w for w in table_widths],
                         sum(-(-q // (2 * tile)) for q in q_lens if q > 1))
        self.static = StaticStep(ints, engine.runtime.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.generation = None

    def _generation(self):
        return (self.engine.runtime.workspace.generation, attention_bf16.scratch_generation())

    def run(self, entries, starts, slots, tables) -> torch.Tensor:
        from .engine import StepContext
        engine = self.engine
        if self.static.meta is None or not self.decode_only:
            meta = pack_step(entries, starts, slots, tables, engine.runtime.device, static=self.static)
        else:
            meta = pack_decode(self.static, [e.tokens[0] for e in entries], starts, slots, tables)
        if self.graph is not None and self.generation != self._generation():
            self.graph = None                       # a buffer moved since the capture
        if self.graph is None:
            engine._forward(StepContext(engine, meta))      # eager once: buffers, attributes, tensor maps
            torch.cuda.synchronize(engine.runtime.device)
            graph = torch.cuda.CUDAGraph()
            # No garbage collection inside the capture: collecting an engine that is
            # no longer used destroys its graphs, which CUDA forbids while any stream
            # captures and which would invalidate this capture.
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    # a fresh context: what a forward pass computes once per step must be in the graph
                    self.logits = engine._forward(StepContext(engine, meta))
            finally:
                if gc_was_on:
                    gc.enable()
            self.graph = graph
            self.generation = self._generation()
            self.launches = engine.last_forward_launches
        self.graph.replay()
        return self.logits
