"""The flattened description of one step that the kernels read.

All tokens of all entries lie in one list; each entry (one request's portion)
is a run of consecutive tokens.  The reference's nearest shape is the Metal
bridge's round (a flat token workspace with per-part offsets, start positions
and block tables, src/metal/kipp_metal.m:1182-1190).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import numpy as np
import torch


ATTENTION_TILE = 64       # tokens per work item of the prefill attention kernel


@dataclasses.dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and the indices among
    them (``want``) whose logits are asked for."""
    request: object
    tokens: list
    want: list = dataclasses.field(default_factory=list)


@dataclasses.dataclass
class StepMeta:
    tokens: int                       # T, total tokens of the step
    entries: int
    token_ids: torch.Tensor           # int32 [T]
    positions: torch.Tensor           # int32 [T] absolute position of each token
    entry_of_token: torch.Tensor      # int32 [T]
    q_start: torch.Tensor             # int32 [entries + 1] first token of each entry
    context_len: torch.Tensor         # int32 [entries] tokens cached before the step
    slots: torch.Tensor               # int32 [entries] state slot of each entry
    logit_rows: Optional[torch.Tensor]  # int32 [R] token rows whose logits are wanted
    n_logit_rows: int
    block_tables: list                # per cache group: int32 [entries, width]
    decode_rows: Optional[torch.Tensor] = None    # int32 [n]: entries that bring one token
    n_decode: int = 0
    prefill_work: Optional[torch.Tensor] = None   # int32 [items, 2]: (entry, first token) per 64-token tile
    n_prefill_items: int = 0
    all_work: Optional[torch.Tensor] = None       # the same over every entry (for kernels without a decode path)
    n_all_items: int = 0
    # host copies for kernel choice
    q_lens: list = dataclasses.field(default_factory=list)
    kv_lens: list = dataclasses.field(default_factory=list)
    extra: dict = dataclasses.field(default_factory=dict)    # work lists of attention kernels

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_kv_len(self) -> int:
        return max(self.kv_lens) if self.kv_lens else 0


class Staging:
    """A ring of pinned host buffers for the step metadata.  A buffer is reused
    only after the copy that read it has finished."""

    def __init__(self, depth: int = 4):
        self._bufs: list = [None] * depth
        self._events: list = [None] * depth
        self._next = 0

    def get(self, n_ints: int) -> tuple[torch.Tensor, int]:
        i = self._next
        self._next = (i + 1) % len(self._bufs)
        if self._events[i] is not None:
            self._events[i].synchronize()
        buf = self._bufs[i]
        if buf is None or buf.numel() < n_ints:
            buf = torch.empty(max(n_ints, 1024) * 2, dtype=torch.int32, pin_memory=True)
            self._bufs[i] = buf
        return buf, i

    def sent(self, i: int) -> None:
        ev = self._events[i]
        if ev is None:
            ev = self._events[i] = torch.cuda.Event()
        ev.record()


def pack_step(entries: list, starts: list[int], slots: list[int], tables: list[np.ndarray],
              device: torch.device, staging: Optional[Staging] = None) -> StepMeta:
    """Build the device metadata from host lists with one host-to-device copy.

    ``starts[i]`` is the number of tokens entry i has cached; ``tables[g]`` is
    the int32 [entries, width_g] block table of cache group g."""
    n = len(entries)
    q_lens = [len(e.tokens) for e in entries]
    T = sum(q_lens)
    q_start = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(q_lens, out=q_start[1:])
    token_ids = np.empty(T, dtype=np.int32)
    positions = np.empty(T, dtype=np.int32)
    entry_of_token = np.empty(T, dtype=np.int32)
    rows: list[int] = []
    for i, e in enumerate(entries):
        a, b = int(q_start[i]), int(q_start[i + 1])
        token_ids[a:b] = e.tokens
        positions[a:b] = np.arange(starts[i], starts[i] + q_lens[i], dtype=np.int32)
        entry_of_token[a:b] = i
        for w in e.want:
            if not 0 <= w < q_lens[i]:
                raise ValueError(f"want index {w} is outside the entry's {q_lens[i]} tokens")
            rows.append(a + w)
    decode_rows = [i for i, q in enumerate(q_lens) if q == 1]
    prefill_work = [(i, t) for i, q in enumerate(q_lens) if q > 1 for t in range(0, q, ATTENTION_TILE)]
    all_work = [(i, t) for i, q in enumerate(q_lens) for t in range(0, q, ATTENTION_TILE)]
    fixed = [token_ids, positions, entry_of_token, q_start,
             np.asarray(starts, dtype=np.int32), np.asarray(slots, dtype=np.int32),
             np.asarray(rows, dtype=np.int32), np.asarray(decode_rows, dtype=np.int32),
             np.asarray(prefill_work, dtype=np.int32).reshape(-1),
             np.asarray(all_work, dtype=np.int32).reshape(-1)]
    parts = fixed + [t.reshape(-1) for t in tables]
    # 4-int alignment of every section keeps 16-byte alignment for vector loads.
    offsets, total = [], 0
    for p in parts:
        offsets.append(total)
        total += (p.size + 3) // 4 * 4
    total = max(total, 4)
    if staging is None:
        host, ring = torch.empty(total, dtype=torch.int32, pin_memory=True), None
    else:
        host, ring = staging.get(total)
    hv = host.numpy()
    for p, o in zip(parts, offsets):
        hv[o:o + p.size] = p
    dev = host[:total].to(device, non_blocking=True)
    if ring is not None:
        staging.sent(ring)

    def sec(i):
        return dev[offsets[i]:offsets[i] + parts[i].size]

    block_tables = [sec(len(fixed) + g).view(tables[g].shape) for g in range(len(tables))]
    return StepMeta(tokens=T, entries=n, token_ids=sec(0), positions=sec(1), entry_of_token=sec(2),
                    q_start=sec(3), context_len=sec(4), slots=sec(5),
                    logit_rows=sec(6) if rows else None, n_logit_rows=len(rows),
                    block_tables=block_tables,
                    decode_rows=sec(7) if decode_rows else None, n_decode=len(decode_rows),
                    prefill_work=sec(8).view(-1, 2) if prefill_work else None,
                    n_prefill_items=len(prefill_work),
                    all_work=sec(9).view(-1, 2), n_all_items=len(all_work), q_lens=q_lens,
                    kv_lens=[s + q for s, q in zip(starts, q_lens)],
                    extra={"h2d_bytes": total * 4})
