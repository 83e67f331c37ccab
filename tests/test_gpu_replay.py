"""Trace replay through bin/trace_run against the plain implementation, in
32-bit and in bfloat16: whole requests; the last 32 tokens one by one; portions
of changing size down to two tokens; and up to four live requests mixed, with
so few pages that they are used again."""
import pytest
import torch

from gpu_util import Trace, assert_close, plain_logits, random_tokens, replay
from tiny import nmse

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 97], "B": [1, 64, 100, 200], "C": [9, 70, 130, 41], "D": [3, 129, 260, 66],
           "E": [3, 200, 330, 70]}
PORTIONS = [7, 2, 19, 2, 48, 3, 2, 31, 64, 2, 5]


def build_trace(name: str):
    """One trace holding every way of cutting; request ids say which."""
    seqs = {f"r{i}": random_tokens(name, n, seed=10 + i) for i, n in enumerate(LENGTHS[name])}
    tr = Trace()
    # 1. each request alone and whole, every position wanted
    for rid, toks in seqs.items():
        tr.step([("whole-" + rid, toks, list(range(len(toks))))], end=["whole-" + rid])
    # 2. most of it in one step, the last 32 tokens one by one
    for rid, toks in seqs.items():
        k = max(len(toks) - 32, 0)
        if k:
            tr.step([("tail-" + rid, toks[:k], [k - 1])])
        for j in range(k, len(toks)):
            tr.step([("tail-" + rid, [toks[j]], [0])], end=["tail-" + rid] if j == len(toks) - 1 else [])
    # 3. portions of changing size, down to two tokens
    for rid, toks in seqs.items():
        at, i = 0, 0
        while at < len(toks):
            n = min(PORTIONS[i % len(PORTIONS)], len(toks) - at)
            last = at + n == len(toks)
            tr.step([("cut-" + rid, toks[at:at + n], list(range(n)))], end=["cut-" + rid] if last else [])
            at, i = at + n, i + 1
    # 4. mixed: up to four live requests, portions of some beside decoded tokens
    #    of others; requests come and go so that their pages are used again
    order = list(seqs) + list(seqs)[::-1]              # every sequence twice: 8 requests
    plan = {f"mix{j}-{rid}": seqs[rid] for j, rid in enumerate(order)}
    waiting = list(plan)
    live: dict = {}
    tick = 0
    peak = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        peak = max(peak, sum(-(-len(plan[r]) // 64) * 64 for r in live))
        entries, ended = [], []
        for j, (rid, at) in enumerate(list(live.items())):
            toks = plan[rid]
            rest = len(toks) - at
            if at == 0 and rest > 3 and (tick + j) % 3 == 0:
                continue                                 # a request may be left out of a step
            head = max(len(toks) - 12, 1)                # the last 12 tokens go one by one
            if at >= head:
                n = 1
            else:
                n = min(max(2, PORTIONS[(tick + j) % len(PORTIONS)]), head - at)
            want = list(range(n)) if n <= 3 else [0, n // 2, n - 1]
            entries.append((rid, toks[at:at + n], want))
            live[rid] = at + n
            if live[rid] == len(toks):
                ended.append(rid)
        if entries:
            tr.step(entries, end=ended)
        for rid in ended:
            del live[rid]
        tick += 1
    tr.peak_tokens = max(peak, max(-(-len(t) // 64) * 64 for t in seqs.values()))
    return seqs, tr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_every_way_of_cutting_matches_the_plain_model(name, dtype):
    seqs, tr = build_trace(name)
    page = {"A": 16, "B": 8, "C": 16, "D": 32, "E": 16}[name]
    got = tr.collect(replay(name, dtype, tr.steps, max_tokens=tr.peak_tokens, page_size=page))
    total_pages_needed = sum(-(-len(t) // page) for t in seqs.values()) * 5
    assert total_pages_needed > 2 * tr.peak_tokens // page           # pages had to be used again
    modes = {"whole": 0, "tail": 0, "cut": 0, "mix": 0}
    worst = {}
    for (rid, pos), row in got.items():
        mode, base = rid.split("-", 1)
        mode = "mix" if mode.startswith("mix") else mode
        want = plain_logits(name, dtype, seqs[base])[pos]
        assert_close(row, want, dtype, f"{name} {dtype} {rid} position {pos}")
        modes[mode] += 1
        worst[mode] = max(worst.get(mode, 0.0), nmse(row, want))
    assert all(n > 0 for n in modes.values()), modes
    assert modes["whole"] == sum(LENGTHS[name]) and modes["cut"] == sum(LENGTHS[name])
    # the 32-bit kernels sum in an order that does not depend on the cut, the batch
    # or the pages: every way of cutting gives the same bits
    if dtype == "float32":
        for (rid, pos), row in got.items():
            mode, base = rid.split("-", 1)
            if mode != "whole":
                assert torch.equal(row, got[("whole-" + base, pos)]), (rid, pos)
