"""Launchers of the sampling kernels."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .ops import KernelError, _check, _fn, _ptr, _stream, c_float, c_int, c_void_p

c_ll = ctypes.c_longlong


def _rows(logits: torch.Tensor) -> tuple[int, int]:
    if logits.dim() != 2 or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] with unit inner stride")
    return logits.shape[0], logits.shape[1]


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, n = _rows(logits)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    need = _fn("sampling", "kipp_argmax_scratch_bytes", [c_int, c_int], restype=c_ll)(rows, n)
    scratch = torch.empty(max(1, need // 8), dtype=torch.int64, device=logits.device)   # long rows: shares of blocks
    f = _fn("sampling", "kipp_argmax_rows_split", [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_ll, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), rows, n, _ptr(out), _ptr(scratch), need, _stream()), "argmax_rows")
    return out


def burst_advance(tokens: torch.Tensor, positions: torch.Tensor, context_len: torch.Tensor,
                  next_tokens: torch.Tensor, ring: torch.Tensor, counter: torch.Tensor) -> None:
    """Between two greedy decode steps on the device: ``next_tokens`` become the
    step's tokens and row ``counter`` of ``ring``, positions and cached lengths move
    on by one."""
    n = next_tokens.numel()
    for t in (tokens, positions, context_len, next_tokens, ring, counter):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("burst_advance takes contiguous int32 tensors")
    if min(tokens.numel(), positions.numel(), context_len.numel()) < n or ring.shape[1] != n:
        raise KernelError("burst_advance: sections shorter than the batch")
    f = _fn("sampling", "kipp_burst_advance",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(tokens), _ptr(positions), _ptr(context_len), _ptr(next_tokens), _ptr(ring), _ptr(counter), n,
             ring.shape[0], _stream()), "burst_advance")


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                top_p: torch.Tensor, min_p: torch.Tensor, uniform: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row.  Per-row parameters: float32 temperature (<= 0 means
    greedy), int32 top_k (0 = off), float32 top_p in (0, 1], float32 min_p in
    [0, 1], float64 uniform draw in [0, 1)."""
    rows, n = _rows(logits)
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"),
                        (top_p, torch.float32, "top_p"), (min_p, torch.float32, "min_p"),
                        (uniform, torch.float64, "uniform")):
        if t.dtype != dt or t.numel() < rows or not t.is_contiguous():
            raise KernelError(f"sample_rows: {name} must be contiguous {dt} with one value per row")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "kipp_sample_rows",
            [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p])
    _check(f(_ptr(logits), logits.stride(0), rows, n, _ptr(temperature), _ptr(top_k), _ptr(top_p),
             _ptr(min_p), _ptr(uniform), _ptr(out), _stream()), "sample_rows")
    return out


def apply_penalties(logits: torch.Tensor, recent: Optional[torch.Tensor],
                    recent_count: Optional[torch.Tensor], repetition: Optional[torch.Tensor],
                    presence: Optional[torch.Tensor], frequency: Optional[torch.Tensor],
                    bias_tokens: Optional[torch.Tensor] = None,
                    bias_values: Optional[torch.Tensor] = None,
                    bias_count: Optional[torch.Tensor] = None) -> None:
    """In place: logit bias, then repetition / presence / frequency penalties
    over each row's recent tokens (int32 [rows, width], counts int32 [rows])."""
    rows, n = _rows(logits)
    f = _fn("sampling", "kipp_apply_penalties",
            [c_void_p, c_ll, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), rows, n, _ptr(recent),
             recent.shape[1] if recent is not None else 0, _ptr(recent_count), _ptr(repetition),
             _ptr(presence), _ptr(frequency), _ptr(bias_tokens), _ptr(bias_values),
             bias_tokens.shape[1] if bias_tokens is not None else 0, _ptr(bias_count), _stream()),
           "apply_penalties")
