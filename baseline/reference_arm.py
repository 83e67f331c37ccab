"""The reference arm of bench.py: the UNMODIFIED reference, built by baseline/build_reference.py
into baseline/_ref/libkipp_ref.so, driven through its own public API (src/kipp.h:
kipp_model_open_backend with the CUDA backend, kipp_session_create, kipp_session_eval,
kipp_eval_batch) on random weights of the benchmark's shape.  None of this repository's
models, kernels or engine is on that path.

The reference opens only GGUF files of the checkpoints in its registry
(src/kipp_checkpoints.h:25-79), so the random weights are written as a throw-away GGUF file
that carries the identity strings of the registry row with the benchmark's sizes (the file
format as src/kipp.c:506-593 reads it: metadata keys, reversed dimensions, 32-byte alignment).

What it can and cannot run in a benchmark's time: its CUDA backend evaluates one token at a
time with scalar kernels (18 launches per layer and token, src/cuda/kipp_cuda.cu:358-462; the
attention kernel walks the context serially, cuda/kipp_kernels.cu:160), and a batch is a loop
over its items (src/cuda/kipp_cuda.cu:660-740).  A context of 8,192 tokens for 8 requests would
take it hours to fill, so the decode figure is taken after short prompts (the record's
``config.seq_len`` says how long) -- the easiest case for the reference -- and the prompt is fed
until 2,048 tokens or a time budget, whichever comes first.
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libkipp_ref.so")

# registry rows of the reference by (layers, hidden, feed-forward, heads): repository, revision, tied
REGISTRY = {
    (28, 1024, 3072, 16): ("Qwen/Qwen3-0.6B-Base", "da87bfb608c14b7cf20ba1ce41287e8de496c0cd", True),
    (36, 2560, 9728, 32): ("Qwen/Qwen3-4B-Base", "906bfd4b4dc7f14ee4320094d8b41684abff8539", True),
    (36, 4096, 12288, 32): ("Qwen/Qwen3-8B-Base", "49e3418fbbbca6ecbdf9608b4d22e5a407081db4", False),
}


class Err(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int), ("message", ctypes.c_char * 256)]


class BatchItem(ctypes.Structure):
    _fields_ = [("session", ctypes.c_void_p), ("tokens", ctypes.POINTER(ctypes.c_uint32)),
                ("token_count", ctypes.c_size_t), ("logits", ctypes.POINTER(ctypes.c_float))]


def tensor_list(c: dict, tied: bool) -> list:
    H, F, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    q, kv = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    t = [("model.embed_tokens.weight", (V, H)), ("model.norm.weight", (H,))]
    if not tied:
        t.append(("lm_head.weight", (V, H)))
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t += [(p + "input_layernorm.weight", (H,)), (p + "self_attn.q_proj.weight", (q, H)),
              (p + "self_attn.k_proj.weight", (kv, H)), (p + "self_attn.v_proj.weight", (kv, H)),
              (p + "self_attn.o_proj.weight", (H, q)), (p + "self_attn.q_norm.weight", (c["head_dim"],)),
              (p + "self_attn.k_norm.weight", (c["head_dim"],)), (p + "post_attention_layernorm.weight", (H,)),
              (p + "mlp.gate_proj.weight", (F, H)), (p + "mlp.up_proj.weight", (F, H)),
              (p + "mlp.down_proj.weight", (H, F))]
    return t


def write_gguf(path: str, c: dict, seed: int, repository: str, revision: str, tied: bool) -> int:
    """Random bfloat16 weights N(0, 0.02) (norm scales near 1), made on the GPU tensor by tensor."""
    import numpy as np
    import torch

    def s(b):
        b = b.encode() if isinstance(b, str) else b
        return struct.pack("<Q", len(b)) + b

    def kv(k, t, payload):
        return s(k) + struct.pack("<I", t) + payload
    V = c["vocab_size"]
    md = [kv("general.architecture", 8, s("qwen3")), kv("general.alignment", 4, struct.pack("<I", 32)),
          kv("kipp.source.repository", 8, s(repository)), kv("kipp.source.revision", 8, s(revision)),
          kv("kipp.quant.scheme", 8, s("bf16")),
          kv("qwen3.block_count", 4, struct.pack("<I", c["num_hidden_layers"])),
          kv("qwen3.embedding_length", 4, struct.pack("<I", c["hidden_size"])),
          kv("qwen3.feed_forward_length", 4, struct.pack("<I", c["intermediate_size"])),
          kv("qwen3.attention.head_count", 4, struct.pack("<I", c["num_attention_heads"])),
          kv("qwen3.attention.head_count_kv", 4, struct.pack("<I", c["num_key_value_heads"])),
          kv("qwen3.attention.key_length", 4, struct.pack("<I", c["head_dim"])),
          kv("qwen3.context_length", 4, struct.pack("<I", 32768)),
          kv("qwen3.vocab_size", 4, struct.pack("<I", V)),
          kv("qwen3.rope.freq_base", 6, struct.pack("<f", float(c["rope_theta"]))),
          kv("qwen3.attention.layer_norm_rms_epsilon", 6, struct.pack("<f", float(c["rms_norm_eps"]))),
          kv("qwen3.tie_word_embeddings", 7, struct.pack("<B", 1 if tied else 0)),
          kv("tokenizer.ggml.model", 8, s("gpt2")), kv("tokenizer.ggml.pre", 8, s("qwen2")),
          kv("tokenizer.ggml.add_bos_token", 7, struct.pack("<B", 0)),
          kv("tokenizer.ggml.eos_token_id", 4, struct.pack("<I", 151643)),
          kv("kipp.tokenizer.tokens", 9, struct.pack("<IQ", 8, V) + s("") * V),
          kv("kipp.tokenizer.special", 9, struct.pack("<IQ", 0, V) + bytes(V)),
          kv("kipp.tokenizer.merge_left", 9, struct.pack("<IQ", 4, 0)),
          kv("kipp.tokenizer.merge_right", 9, struct.pack("<IQ", 4, 0)),
          kv("kipp.tokenizer.merge_result", 9, struct.pack("<IQ", 4, 0))]
    tens = tensor_list(c, tied)
    off, ents, offs = 0, [], []
    for name, shape in tens:
        off = (off + 31) & ~31
        offs.append(off)
        dims = tuple(reversed(shape))
        ents.append(s(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims) +
                    struct.pack("<IQ", 30, off))
        off += int(np.prod(shape)) * 2
    hdr = b"GGUF" + struct.pack("<IQQ", 3, len(tens), len(md)) + b"".join(md) + b"".join(ents)
    ds = (len(hdr) + 31) & ~31
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev).manual_seed(seed)
    with open(path, "wb") as f:
        f.write(hdr)
        f.write(b"\0" * (ds - len(hdr)))
        for (name, shape), o in zip(tens, offs):
            f.write(b"\0" * (ds + o - f.tell()))
            if len(shape) == 1:
                t = 1 + (torch.rand(shape, generator=g, device=dev) * 0.2 - 0.1)
            else:
                t = torch.randn(shape, generator=g, device=dev) * 0.02
            f.write(t.to(torch.bfloat16).cpu().view(torch.int16).numpy().tobytes())
    return ds + off


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main(args, config: dict, seed: int, point_prompt: int, prefill_tokens: int) -> int:
    if not os.path.isfile(LIB):
        return unavailable("baseline/_ref/libkipp_ref.so is absent: python baseline/build_reference.py builds the "
                           "reference (a C project that pip cannot install: it has no setup.py or pyproject.toml)")
    key = (config["num_hidden_layers"], config["hidden_size"], config["intermediate_size"],
           config["num_attention_heads"])
    if key not in REGISTRY or config["num_key_value_heads"] != 8 or config["head_dim"] != 128 \
            or config["vocab_size"] != 151936:
        return unavailable("the reference opens only the shapes of its compiled registry (src/kipp_checkpoints.h)")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        lib = ctypes.CDLL(LIB)
    except OSError as e:
        return unavailable(f"the reference library cannot be loaded: {e}")
    sys.path.insert(0, os.path.dirname(HERE))
    from bench import ClockSampler, median_mad

    repository, revision, tied = REGISTRY[key]
    K, W, B = args.steps, max(args.warmup, 3), args.batch
    V = config["vocab_size"]
    budget_s = float(os.environ.get("KIPP_REFERENCE_BUDGET_S", "45"))
    vp, u32p, fpp = ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_float)
    lib.kipp_model_open_backend.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(vp), ctypes.POINTER(Err)]
    lib.kipp_session_create.argtypes = [vp, ctypes.c_uint32, ctypes.POINTER(vp), ctypes.POINTER(Err)]
    lib.kipp_session_eval.argtypes = [vp, u32p, ctypes.c_size_t, fpp, ctypes.c_size_t, ctypes.POINTER(Err)]
    lib.kipp_eval_batch.argtypes = [vp, ctypes.POINTER(BatchItem), ctypes.c_size_t, ctypes.POINTER(Err)]
    lib.kipp_session_destroy.argtypes = [vp]
    lib.kipp_model_close.argtypes = [vp, ctypes.POINTER(Err)]
    err = Err()
    g = torch.Generator().manual_seed(1234)

    def prompt(n):
        return torch.randint(0, V, (n,), generator=g).tolist()

    with tempfile.TemporaryDirectory(prefix="kipp_ref_") as tmp:
        path = os.path.join(tmp, "random.gguf")
        t0 = time.perf_counter()
        size = write_gguf(path, config, seed, repository, revision, tied)
        print(f"reference arm: wrote {size / 1e9:.2f} GB of random weights in {time.perf_counter() - t0:.1f} s",
              file=sys.stderr, flush=True)
        model = vp()
        if lib.kipp_model_open_backend(path.encode(), 2, ctypes.byref(model), ctypes.byref(err)) != 0:
            return unavailable(f"kipp_model_open_backend(cuda) refused the file: {err.message.decode()}")
        os.remove(path)

        def session(capacity):
            s = vp()
            if lib.kipp_session_create(model, capacity, ctypes.byref(s), ctypes.byref(err)) != 0:
                raise RuntimeError(err.message.decode())
            return s

        logits = (ctypes.c_float * V)()

        def feed(s, tokens):
            arr = (ctypes.c_uint32 * len(tokens))(*tokens)
            if lib.kipp_session_eval(s, arr, len(tokens), logits, V, ctypes.byref(err)) != 0:
                raise RuntimeError(err.message.decode())

        # ---- one request: the prompt (until 2,048 tokens or the time budget), then decode at batch 1
        s1 = session(prefill_tokens + W + K + 8)
        toks = prompt(prefill_tokens)
        feed(s1, toks[:8])                                        # warm-up: first launches, module load
        fed, t0 = 8, time.perf_counter()
        while fed < prefill_tokens and time.perf_counter() - t0 < budget_s:
            n = min(32, prefill_tokens - fed)
            feed(s1, toks[fed:fed + n])
            fed += n
        prefill_s = time.perf_counter() - t0
        prefill = {"value": round((fed - 8) / prefill_s, 1), "tokens": fed, "ms": round(prefill_s * 1e3, 1),
                   "complete": fed == prefill_tokens}
        for _ in range(W):
            feed(s1, prompt(1))
        times = []
        for _ in range(K):
            tok = prompt(1)
            t = time.perf_counter()
            feed(s1, tok)
            times.append((time.perf_counter() - t) * 1e3)
        b1_ms, b1_mad = median_mad(times)
        b1_context = fed + W + K // 2
        lib.kipp_session_destroy(s1)

        # ---- batch B: short prompts, then K steps of kipp_eval_batch with one token per request
        short = 32
        sessions = [session(short + W + K + 8) for _ in range(B)]
        for s in sessions:
            feed(s, prompt(short))
        rows = [(ctypes.c_float * V)() for _ in range(B)]

        def batch_step():
            items = (BatchItem * B)()
            keep = []
            for i, s in enumerate(sessions):
                one = (ctypes.c_uint32 * 1)(prompt(1)[0])
                keep.append(one)
                items[i] = BatchItem(s, one, 1, rows[i])
            if lib.kipp_eval_batch(model, items, B, ctypes.byref(err)) != 0:
                raise RuntimeError(err.message.decode())
        sampler = ClockSampler()
        for _ in range(W):
            batch_step()
        sampler.mark_start()
        times = []
        for _ in range(K):
            t = time.perf_counter()
            batch_step()
            times.append((time.perf_counter() - t) * 1e3)
        sampler.mark_end()
        clocks = sampler.stop()
        ms, mad = median_mad(times)
        for s in sessions:
            lib.kipp_session_destroy(s)
        lib.kipp_model_close(model, ctypes.byref(err))

    print(json.dumps({
        "impl": "reference",
        "metric": f"decode tokens/s, Qwen3-4B-shaped bf16, batch {B} (the reference's CUDA backend through its own API)",
        "value": round(B / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 3), "ms_per_step_mad": round(mad, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 weights and cache, float32 activations (the reference's arithmetic)",
        "data": f"synthetic: random weights N(0,0.02) seed {seed} as a throw-away GGUF file, seeded random token ids",
        "config": {"model": "Qwen3-4B-shaped", "layers": config["num_hidden_layers"], "hidden": config["hidden_size"],
                   "heads": config["num_attention_heads"], "kv_heads": 8, "head_dim": 128,
                   "intermediate": config["intermediate_size"], "vocab": V, "global_batch": B,
                   "seq_len": short + W + K, "parallelism": "none (1 GPU)",
                   "note": "context of the decode figure is short on purpose: the reference fills a context one "
                           "token at a time and would need hours for 8 x 8,192 tokens; its easiest case is timed",
                   "timing": "wall clock around the reference's own blocking calls (logits are on the host when "
                             "they return)"},
        "clocks": clocks, "prefill": prefill,
        "points": {"decode_b1": round(1e3 / b1_ms, 1), "decode_b1_ms": round(b1_ms, 3),
                   "decode_b1_ms_mad": round(b1_mad, 3), "decode_b1_context": b1_context},
        "e2e": {"value": round(B / (ms / 1e3), 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * V * B, "steps": K},
    }))
    return 0
