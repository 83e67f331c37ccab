"""The engine in process: long decoding, the first tokens of a sequence,
generation through the entry point (greedy and sampled), what happens when
pages run out, graphs against plain launches."""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
from gpu_util import (BOUND, assert_close, model_folder, plain_logits, plain_weights, random_tokens)
from tiny import nmse

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def engine(name, dtype, **kw):
    from kipp_b200.engine import Engine
    opts = dict(dtype=dtype, page_size=16, cache_tokens=1024, max_requests=8, max_batch_tokens=512)
    opts.update(kw)
    return Engine.from_folder(model_folder(name), **opts)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_long_decoding(name, dtype):
    """A short prompt and then 300 tokens one by one (given, not sampled), across
    many pages and, in D, far past the window."""
    from kipp_b200.engine import StepEntry
    toks = random_tokens(name, 330, seed=3)
    want = plain_logits(name, dtype, toks)
    eng = engine(name, dtype, page_size=8)
    rows = [eng.step([StepEntry("r", toks[:30], [29])], check=True).cpu().clone()]
    for t in toks[30:]:
        rows.append(eng.step([StepEntry("r", [t], [0])]).cpu().clone())
    eng.runtime.check_status()
    got = torch.cat(rows)
    assert_close(got, want[29:], dtype, f"{name} long decode")
    worst = max(nmse(got[i], want[29 + i]) for i in range(0, 301, 25))
    assert worst <= BOUND[dtype]
    # the decode steps ran as captured graphs (a graph's first step runs directly and is then captured)
    assert eng.graph_replays >= 290


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    """Positions 0, 1, 2: one key, no history, each as a step of its own and
    together."""
    from kipp_b200.engine import StepEntry
    toks = random_tokens("A", 3, seed=9)
    want = plain_logits("A", dtype, toks)
    eng = engine("A", dtype)
    one = [eng.step([StepEntry("x", [t], [0])]).cpu().clone() for t in toks]
    assert_close(torch.cat(one), want, dtype, "one by one")
    both = eng.step([StepEntry("y", toks, [0, 1, 2])]).cpu()
    assert_close(both, want, dtype, "together")
    single = eng.step([StepEntry("z", toks[:1], [0])]).cpu()
    assert_close(single, want[:1], dtype, "a prompt of one token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_steps_equal_plain_launches(dtype):
    from kipp_b200.engine import StepEntry
    seqs = [random_tokens("D", n, seed=n) for n in (70, 9, 140)]
    outs = []
    for graphs in (True, False):
        eng = engine("D", dtype, cuda_graphs=graphs)
        eng.step([StepEntry(i, s[:-6], []) for i, s in enumerate(seqs)])
        rows = []
        for j in range(6, 0, -1):
            rows.append(eng.step([StepEntry(i, [s[-j]], [0]) for i, s in enumerate(seqs)]).cpu().clone())
        outs.append(torch.stack(rows))
    assert torch.equal(outs[0], outs[1])             # same kernels, same order: bitwise


def test_out_of_pages_leaves_every_request_unchanged():
    from kipp_b200.cache import OutOfPages
    from kipp_b200.engine import StepEntry
    eng = engine("A", "float32", cache_tokens=64, page_size=16)       # 4 pages
    a = random_tokens("A", 40, seed=1)
    b = random_tokens("A", 30, seed=2)
    la = eng.step([StepEntry("a", a[:20], [19])]).cpu().clone()
    eng.step([StepEntry("b", b[:17], [])])
    assert eng.cache.free_pages() == [0]
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", a[20:33], [0]), StepEntry("c", [1, 2, 3], [2])])
    assert eng.length("a") == 20 and eng.length("b") == 17 and not eng.is_live("c")
    eng.cache.check()
    eng.finish("b")                                                    # pages come back and are used again
    lb = eng.step([StepEntry("a", a[20:40], [19])]).cpu()
    want = plain_logits("A", "float32", a)
    assert_close(la, want[19:20], "float32")
    assert_close(lb, want[39:40], "float32")
    with pytest.raises(ValueError, match="twice"):
        eng.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    with pytest.raises(ValueError, match="outside"):
        eng.step([StepEntry("q", [256], [0])])
    with pytest.raises(ValueError, match="max positions"):
        eng.step([StepEntry("q", [1] * 129, [])])
    assert not eng.is_live("q")


def greedy_plain(name, dtype, prompt, steps):
    cfg, w = plain_weights(name, dtype)
    path = P.BF16_PATH if dtype == "bfloat16" else P.F32_PATH
    seq, gaps = list(prompt), []
    for _ in range(steps):
        logits = P.plain_forward(cfg, w, seq, **path)[-1]
        top = torch.topk(logits, 2).values
        gaps.append(float(top[0] - top[1]))
        seq.append(int(logits.argmax()))
    return seq[len(prompt):], gaps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(name, dtype):
    """The tiny benchmark workloads: A = prompts of 5/17/33 tokens, 8 greedy steps,
    page 16; B = prompts of 1/64/100/200, portions of 48 mixed with decoding,
    page 8."""
    from kipp_b200.engine.llm import LLM
    lengths = {"A": [5, 17, 33], "B": [1, 64, 100, 200]}[name]
    prompts = [random_tokens(name, n, seed=20 + n) for n in lengths]
    llm = LLM(model_folder(name), dtype=dtype, kv_block_size={"A": 16, "B": 8}[name], kv_tokens=640,
              max_requests=4, max_batch_tokens=64, chunk=48)
    out = llm.generate(prompts, decode=8)
    assert llm.metrics["tokens_sampled"] == 8 * len(prompts)
    for prompt, res in zip(prompts, out):
        want, gaps = greedy_plain(name, dtype, prompt, 8)
        assert res.finish_reason == "length" and len(res.tokens) == 8
        for i, (g, w_) in enumerate(zip(res.tokens, want)):
            if g != w_:
                # only a near-tie may go the other way; the sequences part there
                assert gaps[i] < (1e-4 if dtype == "float32" else 5e-2), (i, g, w_, gaps[i])
                break
    assert llm.engine.cache.free_pages() == [llm.engine.cache.groups[0].pool.n_pages]


def test_sampled_generation_follows_the_plain_sampler():
    """Temperature 0.8, seeded per request: with the engine's own float32 logits
    the device sampler must draw what the plain sampler draws from them."""
    from kipp_b200.engine import Request, StepEntry
    from kipp_b200.engine.llm import LLM
    from kipp_b200.sampling import SamplingParams
    prompts = [random_tokens("B", n, seed=40 + n) for n in (1, 64, 100)]
    llm = LLM(model_folder("B"), dtype="float32", kv_block_size=8, kv_tokens=1024, max_requests=4,
              max_batch_tokens=64, chunk=48)
    params = [SamplingParams(temperature=0.8, seed=5 + i, top_k=[0, 50, 0][i], top_p=[1.0, 1.0, 0.9][i])
              for i in range(3)]
    out = llm.generate(prompts, decode=10, sampling=params)
    again = llm.generate(prompts, decode=10, sampling=params)
    assert [r.tokens for r in out] == [r.tokens for r in again]            # seeded: reproducible
    other = llm.generate(prompts, decode=10, sampling=[SamplingParams(temperature=0.8, seed=99 + i)
                                                       for i in range(3)])
    assert [r.tokens for r in out] != [r.tokens for r in other]
    from kipp_b200.engine import Engine
    eng = Engine.from_folder(model_folder("B"), dtype="float32", page_size=8, cache_tokens=512)
    for i, (prompt, res, sp) in enumerate(zip(prompts, out, params)):
        seq, state = list(prompt), sp.seed
        logits = eng.step([StepEntry(("s", i), seq, [len(seq) - 1])]).cpu()[0]
        for tok in res.tokens:
            want, state = P.plain_sample(logits.numpy(), sp.temperature, state, top_k=sp.top_k, top_p=sp.top_p)
            assert tok == want
            logits = eng.step([StepEntry(("s", i), [tok], [0])]).cpu()[0]


def test_preemption_recomputes_the_same_tokens():
    """With too few pages for all requests the youngest is put back and
    recomputed; greedy output must not change."""
    from kipp_b200.engine.llm import LLM
    prompts = [random_tokens("A", n, seed=60 + n) for n in (30, 28, 26)]
    roomy = LLM(model_folder("A"), dtype="float32", kv_block_size=16, kv_tokens=512, max_requests=4,
                max_batch_tokens=64)
    want = [r.tokens for r in roomy.generate(prompts, decode=20)]
    tight = LLM(model_folder("A"), dtype="float32", kv_block_size=16, kv_tokens=112, max_requests=4,
                max_batch_tokens=64, policy="preempt")              # 7 pages; 3 x 50 tokens need 12
    res = tight.generate(prompts, decode=20)
    assert [r.tokens for r in res] == want
    assert tight.metrics["preemptions"] >= 1 and sum(r.preemptions for r in res) >= 1
    waits = LLM(model_folder("A"), dtype="float32", kv_block_size=16, kv_tokens=112, max_requests=4,
                max_batch_tokens=64, policy="reserve")
    assert [r.tokens for r in waits.generate(prompts, decode=20)] == want
    assert waits.metrics["preemptions"] == 0


def test_command_line(tmp_path):
    import subprocess
    import sys
    import os
    from gpu_util import ROOT
    ids = random_tokens("A", 12, seed=5)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--model", model_folder("A"),
                           "--prompt-ids", ",".join(map(str, ids)), "--decode", "6", "--dtype", "float32",
                           "--top", "3"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = proc.stdout.strip().splitlines()
    assert lines[0].startswith("generated\t")
    generated = [int(t) for t in lines[0].split("\t")[1].split()]
    want, _ = greedy_plain("A", "float32", ids, 6)
    assert generated == want
    assert len(lines) == 4 and lines[1].startswith("1\t")
    full = plain_logits("A", "float32", ids + generated)
    assert int(lines[1].split("\t")[1]) == int(full[-1].argmax())
    assert "KIPP_METRIC backend=cuda prefill_tokens=12" in proc.stderr and "decode_tokens=6" in proc.stderr
    # two prompts of different lengths run beside one another through the same scheduler
    other = random_tokens("A", 31, seed=6)
    both = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--model", model_folder("A"),
                           "--prompt-ids", ",".join(map(str, ids)), "--prompt-ids", ",".join(map(str, other)),
                           "--decode", "5", "--dtype", "float32", "--chunk", "16", "--top", "0"],
                          capture_output=True, text=True, timeout=300)
    assert both.returncode == 0, both.stderr[-2000:]
    got = [[int(t) for t in line.split("\t")[1].split()] for line in both.stdout.strip().splitlines()]
    assert got == [greedy_plain("A", "float32", ids, 5)[0], greedy_plain("A", "float32", other, 5)[0]]
    assert "prefill_tokens=43" in both.stderr and "decode_tokens=10" in both.stderr
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--model", model_folder("A"),
                          "--prompt-ids", "1,2", "--decode", "2", "--temperature", "0.5", "--top-p", "0"],
                         capture_output=True, text=True, timeout=300)
    assert bad.returncode == 2 and "top_p" in bad.stderr


def test_refuses_a_model_that_cannot_fit_before_uploading_anything():
    """Weights plus cache are checked against the free device memory first."""
    from kipp_b200.config import config_from_dict, load_preset
    from kipp_b200.engine import Engine
    cfg_dict, init = load_preset("qwen3-32b")
    import time
    t0 = time.perf_counter()
    with pytest.raises(MemoryError, match="device bytes"):
        Engine.from_config(config_from_dict(cfg_dict), init["seed"], dtype="bfloat16", page_size=16,
                           cache_tokens=4_000_000, max_requests=4)
    assert time.perf_counter() - t0 < 5.0            # refused at once: 64 GB of weights were neither made nor uploaded


def test_repeating_prompt_shapes_replay_a_graph_with_the_eager_results():
    """Portions of a shape seen before are captured and then replayed; the logits
    must be exactly those of an engine without graphs, at other contexts, other
    tokens and other pages than the capture saw."""
    from kipp_b200.engine import Engine, StepEntry
    folder = model_folder("D")
    opts = dict(dtype="bfloat16", page_size=16, cache_tokens=1024, max_requests=4, max_batch_tokens=256)
    with_graphs = Engine.from_folder(folder, **opts)
    eager = Engine.from_folder(folder, cuda_graphs=False, **opts)
    seqs = {r: random_tokens("D", 70 * 3 + 5, seed=60 + i) for i, r in enumerate("abc")}
    replays0 = with_graphs.graph_replays
    for r, seq in seqs.items():                          # the same cuts for every request
        at = 0
        for n in (70, 70, 70, 5):
            entry = [StepEntry(r, seq[at:at + n], [0, n - 1])]
            got = with_graphs.step(entry, check=True).clone()
            want = eager.step(entry, check=True)
            assert torch.equal(got, want), (r, at)
            at += n
    # two requests beside each other, shapes repeating from step to step
    for eng in (with_graphs, eager):
        for r in "abc":
            eng.finish(r)
    outs = []
    for eng in (with_graphs, eager):
        rows = []
        for k in range(3):
            rows.append(eng.step([StepEntry("x", seqs["a"][40 * k:40 * k + 40], [39]),
                                  StepEntry("y", seqs["b"][33 * k:33 * k + 33], [])], check=True).clone())
        outs.append(torch.cat(rows))
    assert torch.equal(outs[0], outs[1])
    assert with_graphs.graph_replays - replays0 >= 4 and eager.graph_replays == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_burst_gives_the_tokens_of_greedy_steps(dtype):
    """Several greedy steps with the tokens fed back on the device: the same
    tokens as step() + argmax with the host in between, pages for all steps
    taken first, lengths advanced; a burst that cannot get its pages changes
    nothing."""
    from kipp_b200.cache import OutOfPages
    from kipp_b200.engine import Engine, StepEntry
    from kipp_b200.kernels import argmax_rows
    folder = model_folder("B")
    opts = dict(dtype=dtype, page_size=8, cache_tokens=400, max_requests=4, max_batch_tokens=128)
    a, b = Engine.from_folder(folder, **opts), Engine.from_folder(folder, **opts)
    prompts = {r: random_tokens("B", n, seed=70 + n) for r, n in (("x", 37), ("y", 9), ("z", 64))}
    firsts = {}
    for eng in (a, b):
        for r, p in prompts.items():
            firsts[r] = int(argmax_rows(eng.step([StepEntry(r, p, [len(p) - 1])], check=True))[0])
    rids = list(prompts)
    steps = 21
    ring = a.decode_burst(rids, [firsts[r] for r in rids], steps).cpu()
    cur = [firsts[r] for r in rids]
    for k in range(steps):
        cur = argmax_rows(b.step([StepEntry(r, [t], [0]) for r, t in zip(rids, cur)], check=True)).tolist()
        assert ring[k].tolist() == cur, k
    a.runtime.check_status()
    assert [a.length(r) for r in rids] == [b.length(r) for r in rids]
    a.cache.check()
    # a second burst goes on from there, and one that cannot fit leaves everything as it was
    ring2 = a.decode_burst(rids, ring[-1].tolist(), 3).cpu()
    for k in range(3):
        cur = argmax_rows(b.step([StepEntry(r, [t], [0]) for r, t in zip(rids, cur)], check=True)).tolist()
        assert ring2[k].tolist() == cur
    lengths, free = [a.length(r) for r in rids], a.cache.free_pages()
    with pytest.raises(OutOfPages):
        a.decode_burst(rids, ring2[-1].tolist(), 200)
    assert [a.length(r) for r in rids] == lengths and a.cache.free_pages() == free
    a.cache.check()


def test_decode_burst_longer_than_its_ring(monkeypatch):
    """The tokens of a burst collect in a ring on the device that is read out when
    it is full: with a ring of 8 rows, 21 steps give the tokens of 21 single steps."""
    from kipp_b200.engine import Engine, StepEntry
    from kipp_b200.kernels import argmax_rows
    monkeypatch.setenv("KIPP_B200_BURST_RING_ROWS", "8")
    folder = model_folder("A")
    opts = dict(dtype="bfloat16", page_size=16, cache_tokens=512, max_requests=4, max_batch_tokens=128)
    a, b = Engine.from_folder(folder, **opts), Engine.from_folder(folder, **opts)
    prompts = {r: random_tokens("A", n, seed=90 + n) for r, n in (("p", 30), ("q", 17))}
    cur = []
    for eng in (a, b):
        cur = [int(argmax_rows(eng.step([StepEntry(r, p, [len(p) - 1])], check=True))[0]) for r, p in prompts.items()]
    rids = list(prompts)
    ring = a.decode_burst(rids, cur, 21).cpu()
    for k in range(21):
        cur = argmax_rows(b.step([StepEntry(r, [t], [0]) for r, t in zip(rids, cur)], check=True)).tolist()
        assert ring[k].tolist() == cur, k
    a.runtime.check_status()
    a.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_truncate_and_reset_continue_like_a_fresh_request(dtype):
    """A request cut back to 23 tokens and fed other tokens gives what a new
    request with those tokens gives; the pages beyond the cut are free again."""
    from kipp_b200.engine import Engine, StepEntry
    folder = model_folder("B")
    eng = Engine.from_folder(folder, dtype=dtype, page_size=8, cache_tokens=256, max_requests=3,
                             max_batch_tokens=128)
    first, other = random_tokens("B", 50, seed=81), random_tokens("B", 30, seed=82)
    eng.step([StepEntry("s", first, [])], check=True)
    held = eng.cache.pages_held("s")[0]
    eng.truncate("s", 23)
    assert eng.length("s") == 23 and eng.cache.pages_held("s")[0] == 3 < held
    got = eng.step([StepEntry("s", other, [0, 29])], check=True).clone()
    want = eng.step([StepEntry("fresh", first[:23] + other, [23, 52])], check=True)
    assert nmse(got, want) < (1e-12 if dtype == "float32" else 1e-5)
    info = eng.info()
    assert info["live_requests"] == {"s": 53, "fresh": 53} and info["cache_groups"][0]["pages"] == 32
    assert info["layers"] == 3 and info["vocab_size"] == 1000 and info["weight_bytes"] > 0
    eng.reset("s")
    assert eng.length("s") == 0 and eng.cache.pages_held("s") == [0]
    again = eng.step([StepEntry("s", first[:23] + other, [23, 52])], check=True)
    assert nmse(again, want) < 1e-12                        # the same kernels on the same tokens
    eng.cache.check()


def test_equal_prompt_portions_without_a_wait_in_between():
    """Six and more equal portions of one prompt, nothing wanted and nothing waited
    for between them: from the third on they replay one captured graph, and the host
    runs ahead of the device.  Each step's metadata must be the one it was packed
    with (the host buffer of a graph is rewritten only after its copy was read)."""
    from kipp_b200.engine import Engine, StepEntry
    folder = model_folder("E")
    opts = dict(dtype="bfloat16", page_size=16, cache_tokens=2048, max_requests=2, max_batch_tokens=256)
    toks = random_tokens("E", 8 * 128 + 3, seed=77)
    outs = []
    for graphs in (True, False):
        eng = Engine.from_folder(folder, cuda_graphs=graphs, **opts)
        for k in range(8):
            eng.step([StepEntry("p", toks[128 * k:128 * (k + 1)], [])])       # no sync, no check
        outs.append(eng.step([StepEntry("p", toks[1024:], [0, 2])], check=True).cpu().clone())
        if graphs:
            assert eng.graph_replays >= 5
    assert torch.equal(outs[0], outs[1])
    assert_close(outs[0], plain_logits("E", "bfloat16", toks)[[1024, 1026]], "bfloat16", "after eight portions")


def test_the_serving_kernels_ran_at_the_benchmark_head_size():
    """Configuration E (128-wide heads): a portion of 64 tokens and more takes the
    tcgen05 attention, decoded tokens the split-K kernel with the fused norm, rotation
    and cache write, the norms of a decode step but its first and last run inside the
    products around them, and decode steps replay a graph."""
    from kipp_b200.engine import Engine, StepEntry
    eng = Engine.from_folder(model_folder("E"), dtype="bfloat16", page_size=16, cache_tokens=1024, max_requests=4,
                             max_batch_tokens=512)
    toks = random_tokens("E", 210, seed=5)
    eng.step([StepEntry("a", toks[:200], []), StepEntry("b", toks[:3], [])], check=True)
    for t in toks[200:]:
        eng.step([StepEntry("a", [t], [0]), StepEntry("b", [t], [0])])
    eng.synchronize()
    c = eng.info()["counters"]
    assert c["tc_prefill_launches"] >= 2 and c["fused_decode_launches"] >= 2 and c["graph_replays"] >= 8
    assert c["folded_norms"] >= 4 and c["folded_norms"] % 4 == 0       # 2 layers: 4 of a step's 5 norms


def test_a_long_portion_norms_rotates_and_writes_the_cache_in_its_projection():
    """Configuration E (128-wide heads): a portion of 1,024 tokens and more, beside a second
    request in the same step, leaves q, k and v through the projection's own epilogue; fed
    in shorter portions the same tokens take the separate kernel.  Either way the end of the
    prompt, the tokens decoded after it and the request beside it match the plain model."""
    from kipp_b200.engine import Engine, StepEntry
    folder = model_folder("E")
    opts = dict(dtype="bfloat16", page_size=16, cache_tokens=4096, max_requests=2, max_batch_tokens=1280)
    toks = random_tokens("E", 1150, seed=12)
    other = random_tokens("E", 40, seed=13)
    ref = plain_logits("E", "bfloat16", toks[:1104])
    ref_other = plain_logits("E", "bfloat16", other)
    for cut in (1100, 400):
        eng = Engine.from_folder(folder, **opts)
        for lo in range(0, 1100, cut):
            hi = min(1100, lo + cut)
            batch = [StepEntry("a", toks[lo:hi], [hi - lo - 1] if hi == 1100 else [])]
            if lo == 0:
                batch.append(StepEntry("b", other, [39]))
            out = eng.step(batch, check=True)
            out = out.cpu() if out is not None else out
            if hi == 1100:
                assert_close(out[:1], ref[[1099]], "bfloat16", f"end of the prompt, portions of {cut}")
            if lo == 0:
                assert_close(out[-1:], ref_other[[39]], "bfloat16", f"the request beside it, portions of {cut}")
        rows = [eng.step([StepEntry("a", [t], [0])], check=True).cpu().clone() for t in toks[1100:1104]]
        assert_close(torch.cat(rows), ref[[1100, 1101, 1102, 1103]], "bfloat16", f"decoded after portions of {cut}")
        assert (eng.info()["counters"]["projections_to_heads"] > 0) == (cut == 1100)
    # the same shape again and again is captured in a graph: four prompts of 1,024 tokens, no sync
    # in between, each against the plain model
    eng = Engine.from_folder(folder, **opts)
    prompts = [random_tokens("E", 1024, seed=20 + i) for i in range(4)]
    outs = []
    for i, pr in enumerate(prompts):
        outs.append(eng.step([StepEntry(("g", i), pr, [1023])]).clone())
        eng.finish(("g", i))
    eng.synchronize()
    assert eng.graph_replays >= 1 and eng.info()["counters"]["projections_to_heads"] > 0
    for i, pr in enumerate(prompts):
        assert_close(outs[i].cpu(), plain_logits("E", "bfloat16", pr)[[1023]], "bfloat16", f"prompt {i} of a repeated shape")


def test_logit_rows_are_limited():
    from kipp_b200.engine import Engine, StepEntry
    eng = Engine.from_folder(model_folder("A"), dtype="float32", page_size=16, cache_tokens=256, max_requests=2,
                             max_batch_tokens=128, max_logit_rows=4)
    assert eng.info()["max_logit_rows"] == 4
    with pytest.raises(ValueError, match="max_logit_rows"):
        eng.step([StepEntry("a", [1, 2, 3, 4, 5, 6], [0, 1, 2, 3, 4])])
    assert not eng.is_live("a")
    assert eng.step([StepEntry("a", [1, 2, 3, 4, 5, 6], [0, 1, 2, 5])]).shape == (4, 256)


def test_a_decoded_token_does_not_depend_on_its_neighbours_with_own_length_splits():
    """With own_length_splits the keys per split of a decoded token come from its
    own context alone: decoded alone or beside seven others of other lengths, its
    bfloat16 logits are the same bits."""
    from kipp_b200.engine import Engine, StepEntry
    folder = model_folder("E")
    opts = dict(dtype="bfloat16", page_size=16, cache_tokens=8192, max_requests=8, max_batch_tokens=4096,
                own_length_splits=True)
    lengths = [700, 30, 1500, 129, 64, 1023, 300, 5]
    seqs = [random_tokens("E", n + 4, seed=200 + n) for n in lengths]
    alone = Engine.from_folder(folder, **opts)
    alone.step([StepEntry("x", seqs[0][:-4], [])])
    rows_alone = [alone.step([StepEntry("x", [t], [0])], check=True).clone() for t in seqs[0][-4:]]
    beside = Engine.from_folder(folder, **opts)
    beside.step([StepEntry(i, s[:-4], []) for i, s in enumerate(seqs)])
    for k in range(4):
        out = beside.step([StepEntry(i, [s[len(s) - 4 + k]], [0]) for i, s in enumerate(seqs)], check=True)
        assert torch.equal(out[0], rows_alone[k][0]), k
    assert_close(rows_alone[-1][0].cpu(), plain_logits("E", "bfloat16", seqs[0])[-1], "bfloat16")


def test_status_words_are_all_read():
    """A kernel that refused an access or gave up a bounded wait leaves a word in the
    engine's status buffer; every word is read and turned into an error."""
    import json
    from kipp_b200.engine import Engine, StepEntry
    from kipp_b200.native import KernelError
    eng = Engine.from_folder(model_folder("A"), dtype="bfloat16", page_size=16, cache_tokens=256, max_requests=2,
                             max_batch_tokens=128)
    eng.step([StepEntry("a", [1, 2, 3], [2])], check=True)
    for word, needle in ((0, "refused"), (1, "bounded wait"), (2, "bounded wait")):
        eng._debug_set_status(word, 2 if word == 0 else 1)
        with pytest.raises(KernelError, match=needle):
            eng.synchronize()
        eng.synchronize()                                  # the words were cleared


def test_engine_in_32_bit_against_the_reference_oracle_with_rounded_keys_and_values():
    """The engine's own float32 logits (not only the plain model's) against the
    reference's CPU oracle at the smallest shape its registry takes, on the same
    random weights: with kv_round_bf16 the 32-bit cache keeps keys and values
    rounded to bfloat16, the reference's storage contract (src/kipp.c:2806-2811).
    The prompt goes in as a portion and then token by token."""
    import importlib.util
    import json
    import os
    from kipp_b200.config import config_from_dict
    from kipp_b200.engine import Engine, StepEntry
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(golden, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    with open(os.path.join(golden, "model_06b.json")) as f:
        gold = json.load(f)
    m = gold["shape"]
    cfg = config_from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=m["L"], hidden_size=m["H"],
        num_attention_heads=m["NH"], num_key_value_heads=m["KV"], head_dim=m["HD"], intermediate_size=m["F"],
        vocab_size=m["V"], rope_theta=m["theta"], rms_norm_eps=m["eps"], tie_word_embeddings=True,
        max_position_embeddings=256))
    names = {name: (i, shape) for i, (name, shape) in enumerate(mg.model_tensors())}

    class Weights:                                     # one tensor at a time: the model is 2.4 GB in float32
        def get(self, name, default=None):
            if name not in names:
                return default
            i, shape = names[name]
            return mg.model_tensor(i, shape)

    from kipp_b200.models.spec import ModelSpec
    eng = Engine(ModelSpec.from_library(cfg), Weights(), dtype="float32", page_size=16, cache_tokens=64,
                 max_requests=1, max_batch_tokens=64, kv_round_bf16=True)
    toks = gold["tokens"]
    head = len(toks) // 2
    rows = [eng.step([StepEntry("g", toks[:head], list(range(head)))], check=True).cpu().clone()]
    for t in toks[head:]:
        rows.append(eng.step([StepEntry("g", [t], [0])], check=True).cpu().clone())
    logits = torch.cat(rows).double()
    idx = torch.tensor(gold["indices"])
    for pos, row in enumerate(gold["positions"]):
        assert int(logits[pos].argmax()) == row["argmax"], pos
        got, want = logits[pos][idx], torch.tensor(row["sample"], dtype=torch.float64)
        assert float(((got - want) ** 2).sum() / (want ** 2).sum()) < 5e-5, pos     # the reference's own bound
    # without the rounding the cache holds more bits than the reference's: the logits move
    plain = Engine(ModelSpec.from_library(cfg), Weights(), dtype="float32", page_size=16, cache_tokens=64,
                   max_requests=1, max_batch_tokens=64)
    other = plain.step([StepEntry("g", toks, [len(toks) - 1])], check=True).cpu().double()
    assert 0 < nmse(other[0], logits[-1]) < 1e-3


def test_profile_gives_the_kernels_of_a_step():
    """Between profile_start and profile_stop steps run without graphs and an event follows
    every launch: the kernels of a decode step with the time between the events."""
    from kipp_b200.engine import Engine, StepEntry
    eng = Engine.from_folder(model_folder("E"), dtype="bfloat16", page_size=16, cache_tokens=512, max_requests=2,
                             max_batch_tokens=128)
    toks = random_tokens("E", 40, seed=3)
    eng.step([StepEntry("a", toks[:30], [])], check=True)
    replays = eng.graph_replays
    eng.profile_start()
    for t in toks[30:34]:
        eng.step([StepEntry("a", [t], [0])])
    spent = eng.profile_stop()
    assert eng.graph_replays == replays
    assert {"attn_decode_mma_fused", "embed_gather"} <= set(spent) and all(v >= 0 for v in spent.values())
    assert sum(k.startswith("gemm_tc ") for k in spent) >= 4                 # the products by shape
    assert 0 < sum(spent.values()) < 1000
    eng.step([StepEntry("a", [toks[34]], [0])], check=True)          # and on with graphs


def test_many_decoded_tokens_are_dealt_out_as_a_stream():
    """230 requests with 1,000 cached tokens each decode together: 460 (token, kv head) pairs
    on 444 places would need several waves of splits, so the planner deals the key tiles out
    as a stream.  Every request holds the same tokens: each row of logits against the plain
    model."""
    from kipp_b200.engine import Engine, StepEntry
    n, length = 230, 1000
    eng = Engine.from_folder(model_folder("E"), dtype="bfloat16", page_size=16, cache_tokens=n * (length + 32),
                             max_requests=n, max_batch_tokens=2048)
    toks = random_tokens("E", length + 2, seed=21)
    rids = [("s", i) for i in range(n)]
    for i in range(0, n, 2):
        eng.step([StepEntry(r, toks[:length], []) for r in rids[i:i + 2]])
    before = eng.info()["counters"]["stream_decode_launches"]
    for k in range(2):
        out = eng.step([StepEntry(r, [toks[length + k]], [0]) for r in rids], check=True).double().cpu()
        want = plain_logits("E", "bfloat16", toks[:length + k + 1])[-1]
        for row in (0, 1, n // 2, n - 1):
            assert_close(out[row], want, "bfloat16", f"row {row} of step {k}")
        assert float((out - out[0]).abs().max()) <= 2e-2 * float(out[0].abs().max())
    assert eng.info()["counters"]["stream_decode_launches"] > before
    eng.cache.check()
