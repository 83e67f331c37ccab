#!/usr/bin/env python3
"""Makes the golden outputs in this folder from the reference's own C code.

    python tests/golden/make_golden.py /path/to/Kipp [--model]

It compiles ``src/kipp.c`` + ``src/kipp_kv_pool.c`` of the reference with
``-DKIPP_TESTING`` into a shared library in a temporary folder (CPU only, no
GPU code) and calls, through ctypes:

* the scalar operators the reference exposes for its own tests
  (``kipp_test_rms_norm``, ``kipp_test_matvec_bf16``, ``kipp_test_rope``,
  ``kipp_test_softmax``, ``kipp_test_silu``, ``kipp_test_float_to_bf16``,
  ``kipp_test_causal_gqa``; src/kipp.h:299-325) and the sampler
  (``kipp_sample_ex``, src/kipp.h:278-295) -> ``operators.json`` (inputs and
  outputs, a few KB);
* with ``--model``: the whole CPU oracle (``kipp_session_eval``) on random
  bfloat16 weights at the smallest shape its registry accepts (Qwen3-0.6B: 28
  layers, hidden 1024, 16 heads, 8 KV heads, head_dim 128, vocab 151,936,
  tied), written as a throw-away GGUF file -> ``model_06b.json`` (argmax and
  256 sampled logits per position).  The reference's model code pins head_dim,
  KV heads and vocabulary (src/kipp.h:19-21), so the tiny test sizes cannot go
  through it.

tests/test_plain.py compares tests/plain_qwen3.py with these files.
"""
import ctypes
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
FP = ctypes.POINTER(ctypes.c_float)


def build(ref: str, out_dir: str) -> ctypes.CDLL:
    so = os.path.join(out_dir, "libkipp_ref.so")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O2", "-std=c11", "-DKIPP_TESTING",
                           f"-I{ref}/src", f"{ref}/src/kipp.c", f"{ref}/src/kipp_kv_pool.c",
                           "-lm", "-o", so])
    return ctypes.CDLL(so)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def fp(a):
    return a.ctypes.data_as(FP)


def to_bf16_bits(a):
    u = f32(a).view(np.uint32)
    return ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


class SampleParams(ctypes.Structure):
    _fields_ = [("temperature", ctypes.c_float), ("top_p", ctypes.c_float),
                ("top_k", ctypes.c_uint32), ("min_p", ctypes.c_float),
                ("frequency_penalty", ctypes.c_float), ("presence_penalty", ctypes.c_float),
                ("repetition_penalty", ctypes.c_float),
                ("recent_tokens", ctypes.POINTER(ctypes.c_uint32)), ("recent_count", ctypes.c_size_t),
                ("logit_bias_tokens", ctypes.POINTER(ctypes.c_uint32)),
                ("logit_bias_values", FP), ("logit_bias_count", ctypes.c_size_t)]


class Err(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int), ("message", ctypes.c_char * 256)]


def operators(lib) -> dict:
    rng = np.random.default_rng(20240)
    out = {}
    u16p = ctypes.POINTER(ctypes.c_uint16)
    # bf16 narrowing
    lib.kipp_test_float_to_bf16.restype = ctypes.c_uint16
    lib.kipp_test_float_to_bf16.argtypes = [ctypes.c_float]
    vals = f32(np.concatenate([rng.normal(0, 3, 24), [0.0, 1.0, -1.0, 1.00390625, 1.01171875, 3.0e38]]))
    out["bf16"] = {"x": vals.tolist(), "bits": [int(lib.kipp_test_float_to_bf16(float(v))) for v in vals]}
    # rms_norm at two sizes / eps
    out["rms_norm"] = []
    for n, eps in ((64, 1e-6), (96, 3e-6), (128, 1e-5)):
        x = f32(rng.normal(0, 2, n)); wb = to_bf16_bits(1 + rng.uniform(-0.2, 0.2, n)); y = np.zeros(n, np.float32)
        lib.kipp_test_rms_norm(fp(x), wb.ctypes.data_as(u16p), fp(y), ctypes.c_size_t(n), ctypes.c_float(eps))
        out["rms_norm"].append({"eps": eps, "x": x.tolist(), "w": from_bf16_bits(wb).tolist(), "y": y.tolist()})
    # matvec
    rows, cols = 7, 48
    W = to_bf16_bits(rng.normal(0, 0.5, (rows, cols))); x = f32(rng.normal(0, 1, cols)); y = np.zeros(rows, np.float32)
    lib.kipp_test_matvec_bf16(W.ctypes.data_as(u16p), fp(x), fp(y), ctypes.c_size_t(rows), ctypes.c_size_t(cols))
    out["matvec"] = {"w": from_bf16_bits(W).tolist(), "x": x.tolist(), "y": y.tolist()}
    # rope
    out["rope"] = []
    for D, theta, pos in ((16, 1e4, 1), (16, 1e4, 77), (32, 1e6, 300), (48, 5e4, 511), (128, 1e6, 8191)):
        h = f32(rng.normal(0, 1, D)); r = h.copy()
        lib.kipp_test_rope(fp(r), ctypes.c_size_t(D), ctypes.c_uint32(pos), ctypes.c_float(theta))
        out["rope"].append({"head_dim": D, "theta": theta, "position": pos, "x": h.tolist(), "y": r.tolist()})
    # softmax, silu
    s = f32(rng.normal(0, 4, 37)); p = s.copy()
    lib.kipp_test_softmax(fp(p), ctypes.c_size_t(len(p)))
    out["softmax"] = {"x": s.tolist(), "y": p.tolist()}
    lib.kipp_test_silu.restype = ctypes.c_float
    lib.kipp_test_silu.argtypes = [ctypes.c_float]
    xs = f32(rng.normal(0, 3, 16))
    out["silu"] = {"x": xs.tolist(), "y": [float(lib.kipp_test_silu(float(v))) for v in xs]}
    # causal GQA: pinned to head_dim 128 and 8 KV heads; 16 query heads (group 2), 9 tokens
    T, nq, nkv, D = 9, 16, 8, 128
    q = f32(rng.normal(0, 1, (T, nq, D))); k = f32(rng.normal(0, 1, (T, nkv, D))); v = f32(rng.normal(0, 1, (T, nkv, D)))
    o = np.zeros((T, nq, D), np.float32); scores = np.zeros(T, np.float32)
    lib.kipp_test_causal_gqa(fp(q), fp(k), fp(v), fp(o), fp(scores), ctypes.c_size_t(T), ctypes.c_size_t(nq))
    out["causal_gqa"] = {"seed": 77, "tokens": T, "q_heads": nq, "kv_heads": nkv, "head_dim": D,
                         "out_sample": o[:, ::5, ::16].tolist()}
    gen = np.random.default_rng(77)       # the test regenerates q, k, v from this seed
    q2 = f32(gen.normal(0, 1, (T, nq, D))); k2 = f32(gen.normal(0, 1, (T, nkv, D))); v2 = f32(gen.normal(0, 1, (T, nkv, D)))
    o2 = np.zeros((T, nq, D), np.float32)
    lib.kipp_test_causal_gqa(fp(q2), fp(k2), fp(v2), fp(o2), fp(scores), ctypes.c_size_t(T), ctypes.c_size_t(nq))
    out["causal_gqa"]["out_sample"] = o2[:, ::5, ::16].tolist()
    out["causal_gqa"]["checksum"] = float(np.abs(o2).sum())
    # sampler: sequences of draws
    lib.kipp_sample_ex.argtypes = [FP, ctypes.c_size_t, ctypes.POINTER(SampleParams),
                                   ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint32),
                                   ctypes.POINTER(Err)]
    out["sampler"] = []
    logits = f32(rng.normal(0, 2.5, 300))
    logits[17] = logits[200] = logits.max() - 0.25            # a tie inside the candidates
    cases = [dict(temperature=0.0), dict(temperature=0.8), dict(temperature=1.3, top_k=5),
             dict(temperature=0.7, top_p=0.6), dict(temperature=1.0, min_p=0.2),
             dict(temperature=0.9, top_k=40, top_p=0.9, min_p=0.02),
             dict(temperature=0.25), dict(temperature=5.0, top_p=0.95)]
    for case in cases:
        sp = SampleParams(temperature=case.get("temperature", 0.0), top_p=case.get("top_p", 1.0),
                          top_k=case.get("top_k", 0), min_p=case.get("min_p", 0.0), repetition_penalty=1.0)
        state = ctypes.c_uint64(12345 + len(out["sampler"]))
        seed = int(state.value)
        toks, err = [], Err()
        for _ in range(24):
            tok = ctypes.c_uint32()
            rc = lib.kipp_sample_ex(fp(logits), ctypes.c_size_t(len(logits)), ctypes.byref(sp),
                                    ctypes.byref(state), ctypes.byref(tok), ctypes.byref(err))
            assert rc == 0, err.message
            toks.append(int(tok.value))
        out["sampler"].append({"params": case, "seed": seed, "tokens": toks, "final_state": int(state.value)})
    out["sampler_logits"] = logits.tolist()
    # penalties + bias on the greedy path
    recent = (ctypes.c_uint32 * 6)(3, 9, 3, 250, 9, 3)
    bt = (ctypes.c_uint32 * 2)(11, 9); bvals = (ctypes.c_float * 2)(1.5, -0.75)
    sp = SampleParams(temperature=0.0, top_p=1.0, repetition_penalty=1.3, presence_penalty=0.4,
                      frequency_penalty=0.2, recent_tokens=recent, recent_count=6,
                      logit_bias_tokens=bt, logit_bias_values=bvals, logit_bias_count=2)
    pl = f32(rng.normal(0, 1, 300)); pl[3] = 6.0; pl[9] = 5.9; pl[11] = 4.6; pl[250] = -2.0
    tok = ctypes.c_uint32(); state = ctypes.c_uint64(1); err = Err()
    assert lib.kipp_sample_ex(fp(pl), ctypes.c_size_t(300), ctypes.byref(sp), ctypes.byref(state),
                              ctypes.byref(tok), ctypes.byref(err)) == 0
    out["penalties"] = {"logits": pl.tolist(), "recent": [3, 9, 3, 250, 9, 3], "bias": {"11": 1.5, "9": -0.75},
                        "repetition": 1.3, "presence": 0.4, "frequency": 0.2, "token": int(tok.value)}
    return out


# ---------------------------------------------------------------------------
MODEL = dict(V=151936, L=28, H=1024, F=3072, NH=16, HD=128, KV=8, theta=1e6, eps=1e-6)


def model_tensors():
    """(name, shape) in GGUF order; values come from model_tensor()."""
    m = MODEL
    t = [("model.embed_tokens.weight", (m["V"], m["H"])), ("model.norm.weight", (m["H"],))]
    for l in range(m["L"]):
        p = f"model.layers.{l}."
        t += [(p + "input_layernorm.weight", (m["H"],)),
              (p + "self_attn.q_proj.weight", (m["NH"] * m["HD"], m["H"])),
              (p + "self_attn.k_proj.weight", (m["KV"] * m["HD"], m["H"])),
              (p + "self_attn.v_proj.weight", (m["KV"] * m["HD"], m["H"])),
              (p + "self_attn.o_proj.weight", (m["H"], m["NH"] * m["HD"])),
              (p + "self_attn.q_norm.weight", (m["HD"],)), (p + "self_attn.k_norm.weight", (m["HD"],)),
              (p + "post_attention_layernorm.weight", (m["H"],)),
              (p + "mlp.gate_proj.weight", (m["F"], m["H"])), (p + "mlp.up_proj.weight", (m["F"], m["H"])),
              (p + "mlp.down_proj.weight", (m["H"], m["F"]))]
    return t


def model_tensor(index: int, shape) -> torch.Tensor:
    """bfloat16 values of tensor number ``index``: N(0, 0.03) matrices (large
    enough that layers matter), 1 + U(-0.2, 0.2) norm scales."""
    g = torch.Generator().manual_seed(1000 + index)
    if len(shape) == 1:
        return (1 + (torch.rand(shape, generator=g) * 0.4 - 0.2)).to(torch.bfloat16)
    return (torch.randn(shape, generator=g) * 0.03).to(torch.bfloat16)


MODEL_TOKENS = [13048, 220, 99489, 5, 151000, 77777, 1234, 42, 90001, 7, 150000, 31337]


def write_gguf(path: str) -> None:
    m = MODEL

    def s(b):
        b = b.encode() if isinstance(b, str) else b
        return struct.pack("<Q", len(b)) + b
    kv = lambda k, t, payload: s(k) + struct.pack("<I", t) + payload
    md = [kv("general.architecture", 8, s("qwen3")), kv("general.alignment", 4, struct.pack("<I", 32)),
          kv("kipp.source.repository", 8, s("Qwen/Qwen3-0.6B-Base")),
          kv("kipp.source.revision", 8, s("da87bfb608c14b7cf20ba1ce41287e8de496c0cd")),
          kv("kipp.quant.scheme", 8, s("bf16")),
          kv("qwen3.block_count", 4, struct.pack("<I", m["L"])),
          kv("qwen3.embedding_length", 4, struct.pack("<I", m["H"])),
          kv("qwen3.feed_forward_length", 4, struct.pack("<I", m["F"])),
          kv("qwen3.attention.head_count", 4, struct.pack("<I", m["NH"])),
          kv("qwen3.attention.head_count_kv", 4, struct.pack("<I", m["KV"])),
          kv("qwen3.attention.key_length", 4, struct.pack("<I", m["HD"])),
          kv("qwen3.context_length", 4, struct.pack("<I", 32768)),
          kv("qwen3.vocab_size", 4, struct.pack("<I", m["V"])),
          kv("qwen3.rope.freq_base", 6, struct.pack("<f", m["theta"])),
          kv("qwen3.attention.layer_norm_rms_epsilon", 6, struct.pack("<f", m["eps"])),
          kv("qwen3.tie_word_embeddings", 7, struct.pack("<B", 1)),
          kv("tokenizer.ggml.model", 8, s("gpt2")), kv("tokenizer.ggml.pre", 8, s("qwen2")),
          kv("tokenizer.ggml.add_bos_token", 7, struct.pack("<B", 0)),
          kv("tokenizer.ggml.eos_token_id", 4, struct.pack("<I", 151643)),
          kv("kipp.tokenizer.tokens", 9, struct.pack("<IQ", 8, m["V"]) + s("") * m["V"]),
          kv("kipp.tokenizer.special", 9, struct.pack("<IQ", 0, m["V"]) + bytes(m["V"])),
          kv("kipp.tokenizer.merge_left", 9, struct.pack("<IQ", 4, 0)),
          kv("kipp.tokenizer.merge_right", 9, struct.pack("<IQ", 4, 0)),
          kv("kipp.tokenizer.merge_result", 9, struct.pack("<IQ", 4, 0))]
    tens = model_tensors()
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
    with open(path, "wb") as f:
        f.write(hdr)
        f.write(b"\0" * (ds - len(hdr)))
        for i, ((name, shape), o) in enumerate(zip(tens, offs)):
            f.write(b"\0" * (ds + o - f.tell()))
            f.write(model_tensor(i, shape).view(torch.int16).numpy().tobytes())


def whole_model(lib, tmp: str) -> dict:
    path = os.path.join(tmp, "rand06b.gguf")
    write_gguf(path)
    V = MODEL["V"]
    model, err = ctypes.c_void_p(), Err()
    assert lib.kipp_model_open(path.encode(), ctypes.byref(model), ctypes.byref(err)) == 0, err.message
    sess = ctypes.c_void_p()
    assert lib.kipp_session_create(model, ctypes.c_uint32(64), ctypes.byref(sess), ctypes.byref(err)) == 0
    lib.kipp_session_eval.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint32), ctypes.c_size_t,
                                      FP, ctypes.c_size_t, ctypes.POINTER(Err)]
    idx = np.random.default_rng(5).choice(V, 256, replace=False)
    idx.sort()
    rows = []
    logits = np.zeros(V, np.float32)
    for tok in MODEL_TOKENS:                         # token by token: logits at every position
        one = (ctypes.c_uint32 * 1)(tok)
        assert lib.kipp_session_eval(sess, one, 1, fp(logits), V, ctypes.byref(err)) == 0, err.message
        rows.append({"argmax": int(logits.argmax()), "sample": logits[idx].tolist(),
                     "norm": float(np.sqrt((logits.astype(np.float64) ** 2).sum()))})
    os.remove(path)
    return {"shape": MODEL, "tokens": MODEL_TOKENS, "indices": idx.tolist(), "positions": rows}


def main() -> None:
    ref = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        lib = build(ref, tmp)
        with open(os.path.join(HERE, "operators.json"), "w") as f:
            json.dump(operators(lib), f)
        if "--model" in sys.argv:
            with open(os.path.join(HERE, "model_06b.json"), "w") as f:
                json.dump(whole_model(lib, tmp), f)


if __name__ == "__main__":
    main()
