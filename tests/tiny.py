"""Tiny Qwen3 configurations for tests and helpers to build them.

A and B differ in every size and option (layers, hidden, heads, KV heads and
group size, head_dim, q width equal / unequal to hidden, feed-forward width,
vocabulary power of two / not, theta, eps, tied / untied head, positions).
C adds layers with a window beside full layers (two cache groups).
"""
from __future__ import annotations

import os

import torch

TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
    intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, hidden_act="silu", attention_bias=False, initializer_range=0.02,
    torch_dtype="float32")
TINY_A_INIT = dict(seed=0, sigma=0.02, norm_jitter=0.1)

TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=128,
    intermediate_size=352, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
    head_dim=32, max_position_embeddings=512, rope_theta=1000000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, hidden_act="silu", attention_bias=False, initializer_range=0.05,
    torch_dtype="float32")
TINY_B_INIT = dict(seed=1, sigma=0.05, norm_jitter=0.2)

TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=515, hidden_size=96,
    intermediate_size=208, num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3,
    head_dim=48, max_position_embeddings=512, rope_theta=50000.0, rms_norm_eps=3e-6,
    tie_word_embeddings=True, hidden_act="silu", attention_bias=False, initializer_range=0.04,
    sliding_window=40, layer_types=["full_attention", "sliding_attention", "sliding_attention",
                                    "full_attention"],
    torch_dtype="float32")
TINY_C_INIT = dict(seed=7, sigma=0.04, norm_jitter=0.15)

# D has a head size the tensor-core attention kernels take (64), a group of 3
# and one windowed layer.
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=777, hidden_size=192,
    intermediate_size=320, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
    head_dim=64, max_position_embeddings=1024, rope_theta=200000.0, rms_norm_eps=2e-6,
    tie_word_embeddings=False, hidden_act="silu", attention_bias=False, initializer_range=0.05,
    sliding_window=50, layer_types=["sliding_attention", "full_attention"], torch_dtype="float32")
TINY_D_INIT = dict(seed=11, sigma=0.05, norm_jitter=0.1)

# E has the head size of the shipped Qwen3 models (128): prompt portions of 64
# tokens and more run on the tcgen05 attention kernel, shorter ones on mma.sync,
# decoded tokens on the split-K kernel with the fused norm/rotation/cache write.
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=640, hidden_size=256,
    intermediate_size=416, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
    head_dim=128, max_position_embeddings=2048, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, hidden_act="silu", attention_bias=False, initializer_range=0.03,
    torch_dtype="float32")
TINY_E_INIT = dict(seed=13, sigma=0.03, norm_jitter=0.1)

CONFIGS = {"A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "C": (TINY_C, TINY_C_INIT),
           "D": (TINY_D, TINY_D_INIT), "E": (TINY_E, TINY_E_INIT)}


def make_model_folder(folder: str, name: str, dtype=torch.float32) -> str:
    """Write config.json and model.safetensors of tiny configuration ``name``."""
    from kipp_b200.config import config_from_dict
    from kipp_b200.weights import write_random_model
    cfg, init = CONFIGS[name]
    config = config_from_dict(cfg)
    return write_random_model(folder, config, init["seed"], sigma=init["sigma"],
                              norm_jitter=init["norm_jitter"], dtype=dtype)


def read_weights(folder: str) -> dict:
    """All tensors of a model folder as CPU tensors (through the safetensors
    package, not through the engine's loader)."""
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k)
    return out


def read_config(folder: str) -> dict:
    import json
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def nmse(a: torch.Tensor, b: torch.Tensor) -> float:
    """sum((a-b)^2) / sum(b^2), the reference's logit error measure
    (logit_nmse, tests/kipp_test.c:1117-1127)."""
    a, b = a.double(), b.double()
    return float(((a - b) ** 2).sum() / (b ** 2).sum())
