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
from ..kernels import sampling as _sampling
from .batch import (ATTENTION_TILE, DECODE_CTA_FIXED_TILES, DECODE_MAX_SPLITS, DECODE_MIN_SPLIT,
                    DECODE_RESIDENT_CTAS, StaticStep, StepMeta, pack_decode, pack_step, step_ints)

BURST_RING_ROWS = 1024      # steps a feedback graph can run before its ring of tokens is read out


class DecodeGraph:
    """The captured forward pass of steps of one shape: the same number of tokens
    and wanted rows per entry and the same block-table widths.  Built for decode
    steps (every entry one token); prompt portions of a repeating shape (the
    chunks of long prompts) use it too."""

    def __init__(self, engine, batch: int, table_widths: list[int], q_lens: Optional[list[int]] = None,
                 wants: Optional[list[int]] = None, feedback: bool = False):
        """``feedback``: a graph of greedy decode steps that feeds itself: after the
        forward pass it takes the argmax of every row, makes it the next step's token
        and moves the step's metadata on by one position, all on the device, so that a
        run of steps is a run of replays with nothing in between."""
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
        self.feedback = feedback
        if feedback:
            if not self.decode_only:
                raise ValueError("a feedback graph is a graph of decode steps")
            dev = engine.runtime.device
            self.next_tokens = torch.zeros(n, dtype=torch.int32, device=dev)
            self.ring = torch.zeros((BURST_RING_ROWS, n), dtype=torch.int32, device=dev)
            self.counter = torch.zeros(1, dtype=torch.int32, device=dev)

    def _feedback_tail(self) -> None:
        """argmax of the step's logits -> next tokens, ring row, positions + 1 (captured)."""
        o, dev, n = self.static.offsets, self.static.device, self.batch
        _sampling.argmax_rows(self.logits, out=self.next_tokens)
        # sections of the packed metadata: 0 keys per split, 1 token ids, 2 positions, 5 cached lengths
        _sampling.burst_advance(dev[o[1]:o[1] + n], dev[o[2]:o[2] + n], dev[o[5]:o[5] + n], dev[o[0]:o[0] + 1],
                                self.next_tokens, self.ring, self.counter, 8, DECODE_RESIDENT_CTAS,
                                DECODE_CTA_FIXED_TILES, DECODE_MIN_SPLIT, DECODE_MAX_SPLITS)

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
                    if self.feedback:
                        self._feedback_tail()
            finally:
                if gc_was_on:
                    gc.enable()
            self.graph = graph
            self.generation = self._generation()
            self.launches = engine.last_forward_launches + (2 if self.feedback else 0)
            if self.feedback:
                # the capture ran nothing, the eager pass before it did: the metadata is
                # as packed (the tail was not part of the eager pass)
                self.counter.zero_()
        self.graph.replay()
        return self.logits

    def run_burst(self, entries, starts, slots, tables, steps: int) -> torch.Tensor:
        """``steps`` greedy steps from the given tokens; returns int32 [steps, batch]
        (a copy).  The first replay runs the packed step, each later one the step the
        tail of the one before prepared."""
        out = torch.empty((steps, self.batch), dtype=torch.int32, device=self.engine.runtime.device)
        done = 0
        first = True
        while done < steps:
            chunk = min(steps - done, BURST_RING_ROWS)
            self.counter.zero_()
            if first:
                self.run(entries, starts, slots, tables)          # packs, captures if need be, replays once
                first = False
                for _ in range(chunk - 1):
                    self.graph.replay()
            else:
                for _ in range(chunk):
                    self.graph.replay()
            out[done:done + chunk].copy_(self.ring[:chunk])
            done += chunk
        return out
