"""A plain, slow implementation of the Qwen3 dense decoder for tests.

Whole sequences, no cache, one function for each part, written from the
reference's formulas (each function cites them) and sharing no code with
``kipp_b200``.  Arithmetic is float64 by default so that it can serve as the
truth for both the 32-bit and the bfloat16 engine paths; ``rounding`` emulates
the places where the bfloat16 path stores 16-bit activations.

The whole-model code of the reference cannot run the tiny test sizes (it pins
head_dim 128, 8 KV heads and a vocabulary of 151,936 in src/kipp.h:19-21), so
this file rests on the formulas; its operators are compared once with the
reference's own scalar functions in tests/golden/.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """Round to nearest even at bfloat16 and widen back
    (float_to_bf16 / bf16_to_float, src/kipp.c:2174-2186)."""
    return x.to(torch.float32).to(torch.bfloat16).to(x.dtype)


def no_round(x: torch.Tensor) -> torch.Tensor:
    return x


def plain_embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """x_t = float(E[id_t, :]), no scaling (src/kipp.c:2579-2585)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)].to(F64)


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, stored=None) -> torch.Tensor:
    """y_i = x_i / sqrt(mean(x^2) + eps) * w_i over the last dim
    (rms_norm, src/kipp.c:2221-2231).  ``stored`` emulates a 16-bit path that
    keeps x_i * w_i in 16 bits and applies the row's factor afterwards in 32-bit."""
    x = x.to(F64)
    scale = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    if stored is not None:
        return stored(x * weight.to(F64)) * scale
    return x * scale * weight.to(F64)


def plain_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y_r = sum_c W[r, c] x_c, weight row-major [out, in], no bias
    (matvec_bf16, src/kipp.c:2233-2243)."""
    return x.to(F64) @ weight.to(F64).t()


def plain_head_norm(h: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm of each head vector over head_dim with one weight for all heads
    (normalize_heads, src/kipp.c:2480-2500).  h is [T, heads, D]."""
    return plain_rmsnorm(h, weight, eps)


def plain_rope(h: torch.Tensor, positions, theta: float) -> torch.Tensor:
    """Half-split rotation (rope_head, src/kipp.c:2368-2382): for i < D/2,
    f = theta^(-2i/D) and a = pos*f are evaluated in float32 as the reference
    does; (h_i, h_{i+D/2}) <- (h_i cos a - h_{i+D/2} sin a, h_{i+D/2} cos a + h_i sin a)."""
    T, _, D = h.shape
    half = D // 2
    # powf(theta, -(2.0f * i) / D): the exponent is a float32 quotient; the power
    # is taken in double and rounded to float32 once, which is what a correctly
    # rounded powf returns.
    exponent = (-(2.0 * torch.arange(half, dtype=torch.float32)) / float(D)).to(F64)
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float32).to(F64), exponent).to(torch.float32)
    pos = torch.as_tensor(positions, dtype=torch.float32).reshape(T, 1)
    angle = (pos * freq).to(F64)                      # float32 product, then exact widening
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    first, second = h[..., :half].to(F64), h[..., half:].to(F64)
    return torch.cat([first * cos - second * sin, second * cos + first * sin], dim=-1)


def plain_softmax(s: torch.Tensor) -> torch.Tensor:
    """exp(s - max) / sum (softmax, src/kipp.c:2384-2400)."""
    e = torch.exp(s - s.max())
    return e / e.sum()


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window=None) -> torch.Tensor:
    """Causal grouped-query attention (causal_gqa, src/kipp.c:2520-2562):
    kv head g = h // (Nq / Nkv); s_j = (q_h . k_{j,g}) / sqrt(D) for the keys
    j <= t the token may see; p = softmax(s); o_h = sum_j p_j v_{j,g}.
    A window of w limits the keys to t - w < j <= t.  q [T, Nq, D]; k, v [T, Nkv, D]."""
    T, n_q, D = q.shape
    n_kv = k.shape[1]
    per_kv = n_q // n_kv
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros(T, n_q, D, dtype=F64)
    q, k, v = q.to(F64), k.to(F64), v.to(F64)
    for t in range(T):
        first = 0 if window is None else max(0, t - window + 1)
        for h in range(n_q):
            g = h // per_kv
            s = (k[first:t + 1, g, :] @ q[t, h, :]) * scale
            p = plain_softmax(s)
            out[t, h, :] = p @ v[first:t + 1, g, :]
    return out


def plain_silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)) (silu, src/kipp.c:2402-2404)."""
    return x / (1.0 + torch.exp(-x))


def plain_feed_forward(n: torch.Tensor, gate_w, up_w, down_w, rounding=no_round) -> torch.Tensor:
    """W_down (silu(W_gate n) * (W_up n)) (src/kipp.c:2996-3010)."""
    act = plain_silu(plain_linear(n, gate_w)) * plain_linear(n, up_w)
    return plain_linear(rounding(act), down_w)


def layer_window(config: dict, layer: int):
    """Window of a layer from the checkpoint's config keys, None = full."""
    types = config.get("layer_types")
    if types is not None:
        return config.get("sliding_window") if types[layer] == "sliding_attention" else None
    if config.get("use_sliding_window") and config.get("sliding_window"):
        return config["sliding_window"] if layer >= config.get("max_window_layers", 0) else None
    return None


def plain_block(x, config: dict, w: dict, prefix: str, layer: int, rounding=no_round,
                positions=None, kv_rounding=None, norm_stored=None) -> torch.Tensor:
    """One layer in the reference's order (cpu_forward, src/kipp.c:2587-2652):
    norm -> q,k,v -> per-head norm of q and k -> rotation of q and k ->
    attention -> output projection -> add -> norm -> SwiGLU -> add.
    ``norm_stored``: the two norms of the layer keep x * w in 16 bits and apply the
    row's factor afterwards (see plain_rmsnorm) instead of rounding the norm's result."""
    T = x.shape[0]
    n_q, n_kv = config["num_attention_heads"], config["num_key_value_heads"]
    D = config.get("head_dim") or config["hidden_size"] // n_q
    eps, theta = config["rms_norm_eps"], config["rope_theta"]
    if positions is None:
        positions = list(range(T))
    if kv_rounding is None:
        kv_rounding = rounding
    def block_norm(x, weight):
        if norm_stored is not None:
            return plain_rmsnorm(x, weight, eps, stored=norm_stored)
        return rounding(plain_rmsnorm(x, weight, eps))
    n = block_norm(x, w[prefix + "input_layernorm.weight"])
    q = rounding(plain_linear(n, w[prefix + "self_attn.q_proj.weight"])).reshape(T, n_q, D)
    k = rounding(plain_linear(n, w[prefix + "self_attn.k_proj.weight"])).reshape(T, n_kv, D)
    v = rounding(plain_linear(n, w[prefix + "self_attn.v_proj.weight"])).reshape(T, n_kv, D)
    q = plain_head_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = plain_head_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q = rounding(plain_rope(q, positions, theta))
    # keys are stored after norm and rotation; the reference rounds stored keys
    # and values to bfloat16 (round_trip_bf16, src/kipp.c:2614-2615)
    k = kv_rounding(plain_rope(k, positions, theta))
    v = kv_rounding(v)
    a = rounding(plain_attention(q, k, v, layer_window(config, layer))).reshape(T, n_q * D)
    x = x + plain_linear(a, w[prefix + "self_attn.o_proj.weight"])
    n = block_norm(x, w[prefix + "post_attention_layernorm.weight"])
    x = x + plain_feed_forward(n, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                               w[prefix + "mlp.down_proj.weight"], rounding)
    return x


# How the engine's bfloat16 path stores activations: 16-bit between kernels, and the norms inside
# a layer as x * w with the row's factor applied by the product that follows.
BF16_PATH = dict(rounding=bf16_round, norm_stored=bf16_round)
F32_PATH = dict(rounding=no_round)


def plain_forward(config: dict, w: dict, tokens, rounding=no_round, kv_rounding=None, norm_stored=None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of every position of one whole sequence
    (cpu_forward, src/kipp.c:2564-2664, which returns the last row only)."""
    x = plain_embedding(w["model.embed_tokens.weight"], tokens)
    for layer in range(config["num_hidden_layers"]):
        x = plain_block(x, config, w, f"model.layers.{layer}.", layer, rounding, kv_rounding=kv_rounding,
                        norm_stored=norm_stored)
    n = rounding(plain_rmsnorm(x, w["model.norm.weight"], config["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else w["lm_head.weight"]
    return plain_linear(n, head)


# ---------------------------------------------------------------------------
# Sampling (kipp_sample_ex, src/kipp.c:3433-3559; RNG src/kipp.c:3322-3333)
# ---------------------------------------------------------------------------
MASK64 = (1 << 64) - 1


def xorshift64_star(state: int) -> tuple[int, int]:
    x = state & MASK64
    x ^= x >> 12
    x ^= (x << 25) & MASK64
    x ^= x >> 27
    return x, (x * 2685821657736338717) & MASK64


def uniform_unit(state: int) -> tuple[int, float]:
    state, r = xorshift64_star(state)
    return state, (r >> 11) / 9007199254740992.0


def plain_sample(logits, temperature: float, rng_state: int, top_k: int = 0, top_p: float = 1.0,
                 min_p: float = 0.0) -> tuple[int, int]:
    """Returns (token, new rng state).  Greedy when temperature <= 0 (first
    maximum wins, RNG untouched); else candidates with logit/T >= max/T - 20,
    sorted by scaled logit descending and token ascending, top-k, weights
    expf(scaled - max) in float32, sums in double, min-p, nucleus, one draw."""
    import numpy as np
    values = np.asarray(logits, dtype=np.float32)
    best = int(np.argmax(values))                      # first maximum
    if temperature <= 0.0:
        return best, rng_state
    inv_t = np.float32(1.0) / np.float32(temperature)
    scaled = (values * inv_t).astype(np.float32)
    scaled_max = np.float32(values[best] * inv_t)
    cutoff = np.float32(scaled_max - np.float32(20.0))
    idx = np.nonzero(scaled >= cutoff)[0]
    order = np.lexsort((idx, -scaled[idx].astype(np.float64)))
    idx = idx[order]
    if top_k and top_k < len(idx):
        idx = idx[:top_k]
    weights = np.exp((scaled[idx] - scaled_max).astype(np.float32)).astype(np.float32)
    if min_p > 0.0 and len(idx):
        threshold = float(np.float32(min_p)) * float(weights[0])
        below = np.nonzero(weights[1:].astype(np.float64) < threshold)[0]
        if len(below):
            idx, weights = idx[:below[0] + 1], weights[:below[0] + 1]
    total = 0.0
    for wv in weights:
        total += float(wv)
    target = float(np.float32(top_p)) * total
    kept, count = 0.0, 0
    while count < len(idx) and kept < target:
        kept += float(weights[count])
        count += 1
    if count == 0:
        count, kept = 1, float(weights[0])
    rng_state, u = uniform_unit(rng_state)
    draw = u * kept
    token, cumulative = int(idx[count - 1]), 0.0
    for i in range(count):
        cumulative += float(weights[i])
        if draw < cumulative:
            token = int(idx[i])
            break
    return token, rng_state
