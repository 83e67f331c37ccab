"""Causal grouped-query attention over the paged cache, with optional per-head
q/k RMSNorm and a position encoding applied to q and k.

Order of operations as the reference's block (docs/ARCHITECTURE.md:77-92,
src/kipp.c:2950-2993): q/k/v projections (no bias) -> per-head norm of q and k
-> rotation -> keys and values into the cache -> attention -> output
projection added to the residual stream.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..weights.spec import INIT_NEAR_ONE, TensorSpec
from .base import Mixer, PagedKVSpec, PositionEncoding


class AttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PositionEncoding, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_dim = num_heads * head_dim
        self.kv_dim = num_kv_heads * head_dim
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # -- declarations -------------------------------------------------------
    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        specs = [
            TensorSpec(prefix + "q_proj.weight", (self.q_dim, self.hidden_size)),
            TensorSpec(prefix + "k_proj.weight", (self.kv_dim, self.hidden_size)),
            TensorSpec(prefix + "v_proj.weight", (self.kv_dim, self.hidden_size)),
            TensorSpec(prefix + "o_proj.weight", (self.hidden_size, self.q_dim)),
        ]
        if self.qk_norm_eps is not None:
            specs += [TensorSpec(prefix + "q_norm.weight", (self.head_dim,), INIT_NEAR_ONE),
                      TensorSpec(prefix + "k_norm.weight", (self.head_dim,), INIT_NEAR_ONE)]
        return specs

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def bind(self, tensors, prefix, runtime) -> None:
        dev, dt = runtime.device, runtime.dtype
        # One matrix for q, k and v so that one product makes all three.
        self.w_qkv = torch.cat([tensors[prefix + n].to(dev).to(dt) for n in
                                ("q_proj.weight", "k_proj.weight", "v_proj.weight")], 0).contiguous()
        self.w_o = tensors[prefix + "o_proj.weight"].to(dev).to(dt).contiguous()
        if self.qk_norm_eps is not None:
            qn = tensors[prefix + "q_norm.weight"].to(dev)
            kn = tensors[prefix + "k_norm.weight"].to(dev)
            if qn.dtype != kn.dtype:
                qn, kn = qn.float(), kn.float()
            self.q_norm, self.k_norm = qn.contiguous(), kn.contiguous()

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        if self.q_norm is not None:
            n += 2 * self.q_norm.numel() * self.q_norm.element_size()
        return n

    # -- one step -------------------------------------------------------------
    def forward(self, ctx, run, h, residual) -> None:
        T = ctx.meta.tokens
        ws, ops = ctx.workspace, ctx.ops
        qkv = ws.buffer("qkv", (T, self.q_dim + 2 * self.kv_dim), ctx.dtype)
        ops.gemm(qkv, h, self.w_qkv, "store", m=T)
        cache = ctx.cache_view(run)                      # pages of this run's cache id
        q = ws.buffer("q", (T, self.num_heads, self.head_dim), ctx.dtype)
        inv_freq = self.position.inv_freq(ctx.device)
        cos_sin = None
        if inv_freq is not None:
            # the step's (cos, sin) table: the same for every layer that rotates alike
            tables = ctx.step_cache.setdefault("rope_tables", {})
            key = (self.position.table_key(), T)
            cos_sin = tables.get(key)
            if cos_sin is None:
                cos_sin = ws.buffer(f"rope_table_{len(tables)}", (T, inv_freq.numel(), 2), torch.float32)
                ops.rope_table(ctx.meta.positions, inv_freq, T, out=cos_sin)
                tables[key] = cos_sin
        attn = ws.buffer("attn_out", (T, self.q_dim), ctx.dtype)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        fused_ok = getattr(ops, "attention_decode_fused_ok", None)
        if fused_ok is not None and fused_ok(ctx.meta, ctx.dtype, self.num_heads, self.num_kv_heads,
                                             self.head_dim, self.position.rotary_dim):
            # decoded tokens only: norm, rotation and the cache write happen inside the
            # attention kernel, straight from the projection's output
            ops.attention_decode_fused(
                attn.view(T, self.num_heads, self.head_dim), qkv, cache.k_pages, cache.v_pages,
                self.q_norm, self.k_norm, eps, cos_sin, run.writes_cache, ctx.meta, cache.block_table,
                cache.page_size, self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window,
                ctx.status)
        else:
            ops.qk_norm_rope_write(
                qkv, q, cache.k_pages, cache.v_pages, self.q_norm, self.k_norm, eps,
                inv_freq, self.position.rotary_dim,
                ctx.meta.positions, ctx.meta.entry_of_token, cache.block_table, cache.page_size, T,
                self.num_heads, self.num_kv_heads, self.head_dim, run.writes_cache, ctx.status,
                cos_sin=cos_sin)
            ops.attention(attn.view(T, self.num_heads, self.head_dim), q, cache.k_pages, cache.v_pages,
                          ctx.meta, cache.block_table, cache.page_size, self.num_heads,
                          self.num_kv_heads, self.head_dim, self.scale, self.window, ctx.status)
        ops.gemm(residual, attn, self.w_o, "add", m=T)
