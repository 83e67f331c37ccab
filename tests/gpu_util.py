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
        path = P.BF16_PATH if dtype == "bfloat16" else P.F32_PATH
        with torch.no_grad():
            _plain_cache[key] = P.plain_forward(cfg, w, list(tokens), **path)
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
def part_engine(dtype: str, hidden: int, *, block=None, final_norm=None, head=None, embedding=None, vocab: int = 32,
                page_size: int = 8, n_pages: int = 64, max_requests: int = 4, seed: int = 0, sigma: float = 0.1,
                norm_jitter: float = 0.2, **options):
    """An engine around the parts under test (the rest of the model is filler):
    returns (engine, the tensors it was bound with as float32/bfloat16-rounded CPU
    tensors).  ``Engine.run_part`` then runs one part alone the way a step does."""
    from kipp_b200.engine import Engine
    from kipp_b200.models.spec import LayerRun, ModelSpec
    from kipp_b200.parts import (AttentionMixer, NoPositionEncoding, OutputHead, PreNormBlock, RMSNorm,
                                 SwiGLUFeedForward, TokenEmbedding)
    from kipp_b200.weights import random_tensors
    if block is None:
        block = PreNormBlock(RMSNorm(hidden, 1e-5), AttentionMixer(hidden, 1, 1, 16, NoPositionEncoding()),
                             RMSNorm(hidden, 1e-5), SwiGLUFeedForward(hidden, 16))
    emb = embedding or TokenEmbedding(vocab, hidden)
    spec = ModelSpec(config=None, hidden_size=hidden, vocab_size=vocab, embedding=emb,
                     layers=[("model.layers.0.", block)], order=[LayerRun(0, 0)],
                     final_norm=("model.norm.", final_norm or RMSNorm(hidden, 1e-5)),
                     head=("lm_head.", head or OutputHead(vocab, hidden, tied_to="model.embed_tokens.weight")),
                     embedding_prefix="model.embed_tokens.", max_positions=4096)
    t = dict(random_tensors(spec.tensor_specs(), seed, sigma=sigma, norm_jitter=norm_jitter))
    if dtype == "bfloat16":
        # matrices are rounded to bfloat16 for the tensor cores; 1-D scales stay float32
        t = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in t.items()}
    eng = Engine(spec, t, dtype=dtype, page_size=page_size, cache_tokens=n_pages * page_size,
                 max_requests=max_requests, max_batch_tokens=512, **options)
    return eng, t


def part_tol(dtype: str) -> dict:
    return dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
