"""Helpers of the GPU tests: model folders, plain logits, trace replay, bounds."""
from __future__ import annotations

import functools
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

import plain_qwen3 as P
from tiny import CONFIGS, make_model_folder, nmse, read_config, read_weights

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Error bounds, fixed before the kernels were written.  float32: the engine
# against the float64 plain model.  bfloat16: against the plain model with the
# same bfloat16 weights and with activations rounded where the engine stores
# 16-bit values (the reference's bound for its GPU path against its CPU oracle
# is NMSE <= 1e-4, tests/kipp_test.c:2945-3083).
BOUND = {"float32": 1e-10, "bfloat16": 1e-4}

_tmp = tempfile.TemporaryDirectory(prefix="kipp_b200_tests_")


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    return make_model_folder(os.path.join(_tmp.name, name), name)


@functools.lru_cache(maxsize=None)
def plain_weights(name: str, dtype: str):
    w = read_weights(model_folder(name))
    if dtype == "bfloat16":
        # matrices are rounded to bfloat16 for the tensor cores; 1-D scales stay float32
        w = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in w.items()}
    return read_config(model_folder(name)), w


_plain_cache: dict = {}


def plain_logits(name: str, dtype: str, tokens: list) -> torch.Tensor:
    """[len(tokens), vocab] logits of the plain model for one whole sequence."""
    key = (name, dtype, tuple(tokens))
    if key not in _plain_cache:
        cfg, w = plain_weights(name, dtype)
        rounding = P.bf16_round if dtype == "bfloat16" else P.no_round
        with torch.no_grad():
            _plain_cache[key] = P.plain_forward(cfg, w, list(tokens), rounding=rounding)
    return _plain_cache[key]


def random_tokens(name: str, n: int, seed: int) -> list:
    vocab = CONFIGS[name][0]["vocab_size"]
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def replay(name: str, dtype: str, steps: list, max_tokens: int, page_size: int = 16) -> dict:
    """Run ``steps`` (dicts as bin/trace_run reads them) through the program;
    returns {step: float32 array [wanted, vocab]}."""
    vocab = CONFIGS[name][0]["vocab_size"]
    with tempfile.TemporaryDirectory(prefix="trace_") as out:
        proc = subprocess.run(
            [sys.executable, TRACE_RUN, "--model", model_folder(name), "--dtype", dtype, "--out", out,
             "--max-tokens", str(max_tokens), "--page-size", str(page_size)],
            input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
            timeout=600)
        assert proc.returncode == 0, proc.stderr[-4000:]
        done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
        assert done == [f"done {s['step']}" for s in steps], proc.stdout[-2000:]
        result = {}
        for s in steps:
            wanted = sum(len(e.get("want", [])) for e in s["entries"])
            path = os.path.join(out, f"{s['step']}.f32")
            if wanted:
                result[s["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
            else:
                assert not os.path.exists(path)
        return result


class Trace:
    """Builds replay steps and remembers which sequence position each wanted
    logits row belongs to."""

    def __init__(self):
        self.steps: list = []
        self.rows: dict = {}          # step -> [(request, position)]
        self.fed: dict = {}

    def step(self, entries: list, end: list = ()) -> None:
        """entries: (request id, tokens, want indices)."""
        n = len(self.steps)
        rows, out = [], []
        for rid, tokens, want in entries:
            start = self.fed.get(rid, 0)
            out.append({"id": rid, "tokens": list(tokens), "want": list(want)})
            rows += [(rid, start + w) for w in want]
            self.fed[rid] = start + len(tokens)
        self.steps.append({"step": n, "entries": out, "end": list(end)})
        self.rows[n] = rows
        for rid in end:
            self.fed.pop(rid, None)

    def collect(self, result: dict) -> dict:
        """{(request, position): logits row}"""
        out = {}
        for step, rows in self.rows.items():
            for i, key in enumerate(rows):
                assert key not in out
                out[key] = torch.from_numpy(result[step][i].copy())
        return out


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    e = nmse(got, want)
    assert e <= BOUND[dtype], f"{what}: NMSE {e:.3e} above {BOUND[dtype]:.0e}"
    assert torch.isfinite(got).all(), what


# ---------------------------------------------------------------------------
class StepMetaForTests:
    """The flattened description of a step as the kernels read it, for the tests of
    single kernels (the engine's own packing is the library's, csrc/host/engine.hpp)."""


def split_length(decoded: int, longest: int, kv_heads: int = 8, sm_count: int = 148, own: bool = False) -> int:
    """Keys per decode-attention split as the library's planner chooses them."""
    from kipp_b200 import native as N
    return N.lib().kipp_attention_split_length(decoded, longest, kv_heads, sm_count, 1 if own else 0)


def pack_meta(entries: list, starts: list, slots: list, tables: list, device) -> StepMetaForTests:
    """``entries``: (request, tokens, want) or objects with ``.tokens`` / ``.want``;
    ``starts[i]`` tokens entry i has cached; ``tables[g]`` int32 [entries, width_g]."""
    toks = [list(e.tokens) if hasattr(e, "tokens") else list(e[1]) for e in entries]
    wants = [list(e.want) if hasattr(e, "want") else list(e[2]) for e in entries]
    q_lens = [len(t) for t in toks]
    T = sum(q_lens)
    q_start = np.zeros(len(entries) + 1, dtype=np.int32)
    np.cumsum(q_lens, out=q_start[1:])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(np.asarray(a, dtype=np.int32))).to(device)   # noqa: E731
    m = StepMetaForTests()
    m.tokens, m.entries = T, len(entries)
    m.q_lens, m.kv_lens = q_lens, [s + q for s, q in zip(starts, q_lens)]
    m.token_ids = dev([t for ts in toks for t in ts])
    m.positions = dev([s + i for s, q in zip(starts, q_lens) for i in range(q)])
    m.entry_of_token = dev([i for i, q in enumerate(q_lens) for _ in range(q)])
    m.q_start, m.context_len, m.slots = dev(q_start), dev(starts), dev(slots)
    rows = [int(q_start[i]) + w for i, ws in enumerate(wants) for w in ws]
    m.logit_rows, m.n_logit_rows = (dev(rows) if rows else None), len(rows)
    m.block_tables = [dev(t) for t in tables]
    decode_rows = [i for i, q in enumerate(q_lens) if q == 1]
    m.decode_rows, m.n_decode = (dev(decode_rows) if decode_rows else None), len(decode_rows)
    tile = 64
    work = [(i, t) for i, q in enumerate(q_lens) if q > 1 for t in range(0, q, tile)]
    every = [(i, t) for i, q in enumerate(q_lens) for t in range(0, q, tile)]
    work128 = [(i, t) for i, q in enumerate(q_lens) if q > 1 for t in range(0, q, 2 * tile)]
    m.prefill_work, m.n_prefill_items = (dev(work).view(-1, 2) if work else None), len(work)
    m.all_work, m.n_all_items = dev(every).view(-1, 2), len(every)
    m.prefill_work128, m.n_prefill_items128 = (dev(work128).view(-1, 2) if work128 else None), len(work128)
    longest = max([starts[i] + 1 for i in decode_rows], default=0)
    m.decode_split_keys = dev([split_length(len(decode_rows), longest)] * max(len(decode_rows), 4))
    m.extra = {}
    return m


# ---------------------------------------------------------------------------
class PartHarness:
    """Runs single parts the way the engine does: a runtime, a cache manager
    and the step context a part sees, without a model around them."""

    def __init__(self, dtype: str, cache_specs: dict, page_size: int = 8, n_pages: int = 64,
                 state_specs: dict | None = None, max_requests: int = 4):
        from kipp_b200.cache import CacheManager
        from kipp_b200.engine.runtime import Runtime
        self.runtime = Runtime("cuda:0", dtype)
        self.cache = CacheManager(cache_specs, page_size, n_pages, max_requests)
        rt = self.runtime
        for g in self.cache.groups:
            shape = (len(g.cache_ids), n_pages, g.spec.kv_heads, page_size, g.spec.head_dim)
            g.k = torch.zeros(shape, dtype=rt.dtype, device=rt.device)
            g.v = torch.zeros(shape, dtype=rt.dtype, device=rt.device)
        self.states = {cid: torch.zeros((max_requests,) + tuple(s.shape), dtype=s.dtype, device=rt.device)
                       for cid, s in (state_specs or {}).items()}

    def context(self, layout: list):
        """layout: [(request id, number of new tokens)].  Reserves pages; call
        ``commit`` after the parts ran."""
        from kipp_b200.engine.batch import StepEntry, pack_step
        from kipp_b200.engine.engine import CacheView
        for rid, _ in layout:
            if rid not in self.cache:
                self.cache.admit(rid)
        starts = [self.cache.length(rid) for rid, _ in layout]
        self.cache.reserve([(rid, s + n) for (rid, n), s in zip(layout, starts)])
        rids = [rid for rid, _ in layout]
        tables = [self.cache.block_table_rows(rids, gi) for gi in range(len(self.cache.groups))]
        entries = [StepEntry(rid, [0] * n, []) for rid, n in layout]
        meta = pack_step(entries, starts, [self.cache.slot(r) for r in rids], tables, self.runtime.device)
        harness, rt = self, self.runtime
        self._pending = [(rid, s + n) for (rid, n), s in zip(layout, starts)]

        class Ctx:
            pass
        ctx = Ctx()
        ctx.meta, ctx.device, ctx.dtype, ctx.ops = meta, rt.device, rt.dtype, rt.ops
        ctx.workspace, ctx.status = rt.workspace, rt.status
        ctx.step_cache = {}

        def cache_view(run):
            gi, j = harness.cache.group_of_cache[run.cache]
            g = harness.cache.groups[gi]
            return CacheView(g.k[j], g.v[j], meta.block_tables[gi], g.page_size)
        ctx.cache_view = cache_view
        ctx.state_view = lambda run: harness.states[run.cache]
        return ctx

    def commit(self) -> None:
        for rid, n in self._pending:
            self.cache.advance(rid, n)
        self.runtime.check_status()


def part_tol(dtype: str) -> dict:
    return dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
