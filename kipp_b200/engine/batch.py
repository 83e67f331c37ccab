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
DECODE_RESIDENT_CTAS = 444  # decode-attention CTAs resident at once: 3 per SM on 148 SMs
DECODE_MAX_SPLITS = 32
DECODE_MIN_SPLIT = 128


DECODE_CTA_FIXED_TILES = 5   # what a decode-attention CTA costs beside its key tiles, in tiles of 64 keys


def decode_split_length(kv_lens: list, kv_heads_hint: int = 8) -> int:
    """Keys per split for the decoded tokens of a step.  The number of splits is
    the one with the best (share of the resident CTA slots that the waves fill)
    x (share of a CTA's time spent on keys rather than on its set-up, its merge
    of four warps and its partial results): many short splits fill the GPU when
    there are few (token, kv head) pairs, few long ones are better once the
    pairs alone fill it (measured on B200: batch 64 at 2,048 keys is 9 % faster
    with 3 splits than with 6, batch 8 at 8,192 keys fastest with 6)."""
    if not kv_lens:
        return DECODE_MIN_SPLIT
    pairs = len(kv_lens) * kv_heads_hint
    longest = max(kv_lens)
    best, best_score = 1, -1.0
    for splits in range(1, DECODE_MAX_SPLITS + 1):
        if splits > 1 and longest // splits < DECODE_MIN_SPLIT:
            break
        ctas = pairs * splits
        waves = -(-ctas // DECODE_RESIDENT_CTAS)
        tiles = -(-(-(-longest // splits)) // 64)
        score = ctas / (waves * DECODE_RESIDENT_CTAS) * tiles / (tiles + DECODE_CTA_FIXED_TILES)
        if score > best_score + 1e-9:
            best, best_score = splits, score
    keys = -(-longest // best)
    return max(DECODE_MIN_SPLIT, -(-keys // 64) * 64)


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
    prefill_work128: Optional[torch.Tensor] = None   # (entry, first token) per 128-token tile, entries of > 1 token
    n_prefill_items128: int = 0
    decode_split_keys: Optional[torch.Tensor] = None   # int32 [4]: keys per split of decoded tokens
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


class StaticStep:
    """Fixed host and device buffers for steps of one shape (a CUDA graph reads
    the device buffer at the same addresses on every replay)."""

    def __init__(self, n_ints: int, device: torch.device):
        self.n_ints = n_ints
        self.host = torch.zeros(n_ints, dtype=torch.int32, pin_memory=True)
        self.device = torch.zeros(n_ints, dtype=torch.int32, device=device)
        self.meta: Optional[StepMeta] = None
        self.offsets: list[int] = []          # of the sections of the packed buffer, once packed


def pack_step(entries: list, starts: list[int], slots: list[int], tables: list[np.ndarray],
              device: torch.device, staging: Optional[Staging] = None,
              static: Optional[StaticStep] = None) -> StepMeta:
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
    work128 = [(i, t) for i, q in enumerate(q_lens) if q > 1 for t in range(0, q, 2 * ATTENTION_TILE)]
    split = np.zeros(4, dtype=np.int32)
    split[0] = decode_split_length([starts[i] + 1 for i in decode_rows])
    fixed = [split, token_ids, positions, entry_of_token, q_start,
             np.asarray(starts, dtype=np.int32), np.asarray(slots, dtype=np.int32),
             np.asarray(rows, dtype=np.int32), np.asarray(decode_rows, dtype=np.int32),
             np.asarray(prefill_work, dtype=np.int32).reshape(-1),
             np.asarray(all_work, dtype=np.int32).reshape(-1),
             np.asarray(work128, dtype=np.int32).reshape(-1)]
    parts = fixed + [t.reshape(-1) for t in tables]
    # 4-int alignment of every section keeps 16-byte alignment for vector loads.
    offsets, total = [], 0
    for p in parts:
        offsets.append(total)
        total += (p.size + 3) // 4 * 4
    total = max(total, 4)
    if static is not None:
        if static.n_ints != total:
            raise ValueError("a static step must keep its shape")
        hv = static.host.numpy()
        for p, o in zip(parts, offsets):
            hv[o:o + p.size] = p
        static.device.copy_(static.host, non_blocking=True)
        static.offsets = offsets
        if static.meta is not None:            # same layout: the views stay valid
            static.meta.q_lens = q_lens
            static.meta.kv_lens = [s + q for s, q in zip(starts, q_lens)]
            return static.meta
        dev = static.device
    else:
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
    meta = StepMeta(tokens=T, entries=n, decode_split_keys=sec(0), token_ids=sec(1), positions=sec(2),
                    entry_of_token=sec(3), q_start=sec(4), context_len=sec(5), slots=sec(6),
                    logit_rows=sec(7) if rows else None, n_logit_rows=len(rows),
                    block_tables=block_tables,
                    decode_rows=sec(8) if decode_rows else None, n_decode=len(decode_rows),
                    prefill_work=sec(9).view(-1, 2) if prefill_work else None,
                    n_prefill_items=len(prefill_work),
                    all_work=sec(10).view(-1, 2), n_all_items=len(all_work),
                    prefill_work128=sec(11).view(-1, 2) if work128 else None, n_prefill_items128=len(work128),
                    q_lens=q_lens,
                    kv_lens=[s + q for s, q in zip(starts, q_lens)],
                    extra={"h2d_bytes": total * 4})
    if static is not None:
        static.meta = meta
    return meta


def pack_decode(static: StaticStep, tokens: list[int], starts: list[int], slots: list[int],
                tables: list[np.ndarray]) -> StepMeta:
    """The same as :func:`pack_step` for a step in which every entry brings one
    token and wants its logits, into a static step that :func:`pack_step` has
    filled once for that many entries: the sections that depend only on the
    number of entries (token-to-entry map, row lists, work lists) are left as
    they are; token ids, positions, context lengths, slots, the split length
    and the block tables are written."""
    meta, o = static.meta, static.offsets
    n = len(tokens)
    if meta is None or meta.entries != n or meta.tokens != n or meta.n_decode != n:
        raise ValueError("pack_decode needs a static step packed for as many one-token entries")
    hv = static.host.numpy()
    kv_lens = [s + 1 for s in starts]
    hv[o[0]] = decode_split_length(kv_lens)
    hv[o[1]:o[1] + n] = tokens
    hv[o[2]:o[2] + n] = starts
    hv[o[5]:o[5] + n] = starts
    hv[o[6]:o[6] + n] = slots
    for g, t in enumerate(tables):
        at = o[12 + g]
        hv[at:at + t.size] = t.reshape(-1)
    static.device.copy_(static.host, non_blocking=True)
    meta.kv_lens = kv_lens
    return meta


def step_ints(n_entries: int, n_tokens: int, n_rows: int, n_decode: int, n_prefill_items: int,
              n_all_items: int, table_ints: list[int], n_prefill_items128: int = 0) -> int:
    """Size in int32 of the packed buffer of a step of this shape."""
    sizes = [4, n_tokens, n_tokens, n_tokens, n_entries + 1, n_entries, n_entries, n_rows, n_decode,
             2 * n_prefill_items, 2 * n_all_items, 2 * n_prefill_items128] + list(table_ints)
    return max(sum((s + 3) // 4 * 4 for s in sizes), 4)
