"""Turns the logits of a step into one token per wanted row, on the device.

The host keeps each request's generator state and draws the uniform number;
the kernels do everything that touches the vocabulary (penalties, maximum,
candidate cut, top-k, min-p, nucleus, the draw).
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..kernels import sampling as _k
from .params import RECENT_WINDOW, SamplingParams, next_uniform


class Sampler:
    def __init__(self, device: torch.device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               rng_states: list[int], recent: Sequence[Sequence[int]] | None = None) -> torch.Tensor:
        """``logits`` float32 [rows, vocab] on the device (modified in place when a
        row has penalties or a bias).  ``rng_states[i]`` is advanced for rows
        with temperature > 0 only, as the reference leaves the generator
        untouched on the greedy path.  Returns int32 [rows] on the device."""
        rows = logits.shape[0]
        if len(params) != rows or len(rng_states) != rows:
            raise ValueError("one SamplingParams and one generator state per row")
        self._penalties(logits, params, recent)
        if all(p.temperature <= 0.0 for p in params):
            return _k.argmax_rows(logits)
        f32 = np.zeros((3, rows), dtype=np.float32)
        topk = np.zeros(rows, dtype=np.int32)
        uni = np.zeros(rows, dtype=np.float64)
        for i, p in enumerate(params):
            f32[0, i], f32[1, i], f32[2, i] = p.temperature, p.top_p, p.min_p
            topk[i] = p.top_k
            if p.temperature > 0.0:
                rng_states[i], uni[i] = next_uniform(rng_states[i])
        dev = self.device
        f32_d = torch.from_numpy(f32).to(dev)
        return _k.sample_rows(logits, f32_d[0], torch.from_numpy(topk).to(dev), f32_d[1], f32_d[2],
                              torch.from_numpy(uni).to(dev))

    def _penalties(self, logits, params, recent) -> None:
        rows = logits.shape[0]
        need_pen = recent is not None and any(p.has_penalties and len(r) for p, r in zip(params, recent))
        need_bias = any(p.logit_bias for p in params)
        if not (need_pen or need_bias):
            return
        dev = self.device
        rec = cnt = rep = pres = freq = bt = bv = bc = None
        if need_pen:
            rec_h = np.full((rows, RECENT_WINDOW), -1, dtype=np.int32)
            cnt_h = np.zeros(rows, dtype=np.int32)
            pen_h = np.zeros((3, rows), dtype=np.float32)
            for i, (p, r) in enumerate(zip(params, recent)):
                r = list(r)[-RECENT_WINDOW:]
                if p.has_penalties:
                    rec_h[i, :len(r)] = r
                    cnt_h[i] = len(r)
                pen_h[:, i] = (p.repetition_penalty, p.presence_penalty, p.frequency_penalty)
            rec, cnt = torch.from_numpy(rec_h).to(dev), torch.from_numpy(cnt_h).to(dev)
            pen = torch.from_numpy(pen_h).to(dev)
            rep, pres, freq = pen[0], pen[1], pen[2]
        if need_bias:
            width = max(len(p.logit_bias) for p in params)
            bt_h = np.zeros((rows, width), dtype=np.int32)
            bv_h = np.zeros((rows, width), dtype=np.float32)
            bc_h = np.zeros(rows, dtype=np.int32)
            for i, p in enumerate(params):
                for j, (tok, val) in enumerate(p.logit_bias.items()):
                    bt_h[i, j], bv_h[i, j] = int(tok), float(val)
                bc_h[i] = len(p.logit_bias)
            bt, bv, bc = (torch.from_numpy(a).to(dev) for a in (bt_h, bv_h, bc_h))
        _k.apply_penalties(logits, rec, cnt, rep, pres, freq, bt, bv, bc)
