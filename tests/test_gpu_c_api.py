"""The C interface from a C program: tests/c_api/replay.c is compiled here
against kipp_b200.h and libkipp_engine.so and run as a process of its own (no
Python in it).  It opens tiny models from their folders, replays a trace with
mixed steps through kipp_engine_step and generates greedy tokens with the
scheduler; its logits must be the very bits that bin/trace_run (the Python face
of the same library) writes for the same trace, and its tokens the plain
model's greedy continuation."""
import os
import shutil
import struct
import subprocess
import tempfile

import numpy as np
import pytest
import torch

from gpu_util import ROOT, Trace, model_folder, random_tokens, replay
from test_gpu_engine import greedy_plain
from tiny import CONFIGS

pytestmark = pytest.mark.gpu
HOST = os.path.join(ROOT, "kipp_b200", "csrc", "host")


@pytest.fixture(scope="module")
def program(tmp_path_factory):
    from kipp_b200.csrc import build
    build.build_all(verbose=False)                       # the C program has no resolver that builds on demand
    lib_dir = os.path.dirname(build.compile_host_library())
    exe = str(tmp_path_factory.mktemp("c_api") / "replay")
    cc = shutil.which("gcc") or shutil.which("cc")
    assert cc, "no C compiler"
    proc = subprocess.run([cc, "-std=c11", "-O1", "-Wall", "-Werror", "-I", HOST,
                           os.path.join(ROOT, "tests", "c_api", "replay.c"), "-o", exe,
                           "-L", lib_dir, "-lkipp_engine", f"-Wl,-rpath,{lib_dir}"],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return exe


def mixed_trace(name: str):
    """Three requests: whole, in portions beside decoded tokens, pages reused."""
    a, b, c = (random_tokens(name, n, seed=300 + n) for n in (70, 41, 23))
    tr = Trace()
    tr.step([(1, a[:50], [49]), (2, b[:2], [0, 1])])
    tr.step([(1, a[50:51], [0]), (2, b[2:30], [27]), (3, c[:9], [])])
    tr.step([(1, a[51:52], [0]), (2, b[30:31], [0]), (3, c[9:], [0, 13])], end=[3])
    for k in range(52, 60):
        tr.step([(1, a[k:k + 1], [0]), (2, b[k - 21:k - 20], [0])])
    tr.step([(1, a[60:], list(range(10))), (2, b[39:], [0, 1])], end=[1, 2])
    tr.step([(4, c, [len(c) - 1])], end=[4])
    return tr


def write_binary(tr: Trace, path: str, prompt: list, decode: int) -> None:
    ints = [len(tr.steps)]
    for s in tr.steps:
        ints += [s["step"], len(s["entries"])]
        for e in s["entries"]:
            ints += [int(e["id"]), len(e["tokens"])] + list(e["tokens"]) + [len(e["want"])] + list(e["want"])
        ints += [len(s["end"])] + [int(r) for r in s["end"]]
    ints += [len(prompt)] + list(prompt) + [decode]
    with open(path, "wb") as f:
        f.write(struct.pack(f"<{len(ints)}i", *ints))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_c_program_matches_trace_run_bit_for_bit(program, name, dtype):
    tr = mixed_trace(name)
    vocab = CONFIGS[name][0]["vocab_size"]
    prompt = random_tokens(name, 19, seed=77)
    max_tokens, page = 256, 16
    python_side = replay(name, dtype, tr.steps, max_tokens=max_tokens, page_size=page)
    with tempfile.TemporaryDirectory(prefix="c_api_") as tmp:
        trace_path = os.path.join(tmp, "trace.bin")
        write_binary(tr, trace_path, prompt, 8)
        env = dict(os.environ, HOME=tmp)
        proc = subprocess.run([program, model_folder(name), dtype, str(max_tokens), str(page), trace_path, tmp],
                              capture_output=True, text=True, timeout=300, env=env)
        assert proc.returncode == 0, proc.stderr[-3000:]
        lines = proc.stdout.strip().splitlines()
        assert lines[:len(tr.steps)] == [f"done {s['step']}" for s in tr.steps]
        for s in tr.steps:
            wanted = sum(len(e["want"]) for e in s["entries"])
            path = os.path.join(tmp, f"{s['step']}.f32")
            if not wanted:
                assert not os.path.exists(path)
                continue
            got = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
            assert np.array_equal(got, python_side[s["step"]]), (name, dtype, s["step"])
        generated = [int(t) for t in lines[len(tr.steps)].split()[1:]]
        want, gaps = greedy_plain(name, dtype, prompt, 8)
        assert len(generated) == 8 and lines[-1].startswith("finished 1 reason 2")
        for i, (g, w) in enumerate(zip(generated, want)):
            if g != w:                                   # only a near-tie may go the other way
                assert gaps[i] < (1e-4 if dtype == "float32" else 5e-2), (i, g, w, gaps[i])
                break
