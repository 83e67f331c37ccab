"""Dense SwiGLU feed-forward: x += W_down (silu(W_gate n) * (W_up n))
(src/kipp.c:2994-3010, silu src/kipp.c:2402-2404)."""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import FeedForward


class SwiGLUFeedForward(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.w_gate_up = self.w_down = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [
            TensorSpec(prefix + "gate_proj.weight", (self.intermediate_size, self.hidden_size)),
            TensorSpec(prefix + "up_proj.weight", (self.intermediate_size, self.hidden_size)),
            TensorSpec(prefix + "down_proj.weight", (self.hidden_size, self.intermediate_size)),
        ]

    def bind(self, tensors, prefix, runtime) -> None:
        dev, dt = runtime.device, runtime.dtype
        gate = tensors[prefix + "gate_proj.weight"].to(dev).to(dt)
        up = tensors[prefix + "up_proj.weight"].to(dev).to(dt)
        # Rows interleaved (gate_0, up_0, gate_1, up_1, ...): one product makes
        # both, and a gate sits beside its up value in the epilogue.
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(
            2 * self.intermediate_size, self.hidden_size).contiguous()
        self.w_down = tensors[prefix + "down_proj.weight"].to(dev).to(dt).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, ctx, h, residual) -> None:
        T = ctx.meta.tokens
        act = ctx.workspace.buffer("ffn_act", (T, self.intermediate_size), ctx.dtype)
        ctx.ops.gemm(act, h, self.w_gate_up, "swiglu", m=T)
        ctx.ops.gemm(residual, act, self.w_down, "add", m=T)
