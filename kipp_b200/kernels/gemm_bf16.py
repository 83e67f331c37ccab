"""Choice among the bfloat16 matrix-product kernels."""
from __future__ import annotations

import ctypes

import torch

from .ops import EPILOGUES, KernelError, _check, _fn, _ptr, _stream, c_int, c_void_p, dtype_code

c_ll = ctypes.c_longlong

def plan(tokens: int, features: int, K: int, splits: int = 0, tile: int = 0, tile_f: int = 0):
    """(token tile, feature tile, K splits) the tensor-core kernel uses for a shape."""
    f = _fn("gemm_tc", "kipp_gemm_tc_plan",
            [c_int, c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int),
             ctypes.POINTER(c_int)])
    t, tf, sp = c_int(), c_int(), c_int()
    f(tokens, features, K, splits, tile, tile_f, ctypes.byref(t), ctypes.byref(tf), ctypes.byref(sp))
    return t.value, tf.value, sp.value


def tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands (TMA needs 16-byte
    aligned bases and row pitches)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def choose(M, N, K, a, w, out, epilogue) -> str:
    return "tc" if tc_ok(a, w) else "simt"


class NormFold(ctypes.Structure):
    """kipp_gemm_norm_fold of the kernel library: what folds an RMSNorm into the
    products around it (few-token kernel only)."""
    _fields_ = [("norm_w", c_void_p), ("norm_w_dtype", c_int), ("xn", c_void_p), ("ldn", c_ll),
                ("ssq_out", c_void_p), ("ssq_in", c_void_p), ("ssq_in_slots", c_int),
                ("inv_n", ctypes.c_float), ("eps", ctypes.c_float)]


def fold_emit(norm_w: torch.Tensor, xn: torch.Tensor, ssq: torch.Tensor) -> NormFold:
    """For a residual add: also write xn = bf16(new residual * norm_w) and
    ssq[t, f // 32] = sums of squares of the new residual."""
    return NormFold(_ptr(norm_w), dtype_code(norm_w.dtype), _ptr(xn), xn.stride(0), _ptr(ssq), None, 0, 0.0, 0.0)


def fold_scale(ssq: torch.Tensor, n: int, eps: float) -> NormFold:
    """For a store or SwiGLU product: scale row t by 1 / sqrt(sum(ssq[t]) / n + eps)."""
    return NormFold(None, 0, None, 0, None, _ptr(ssq), ssq.shape[1], 1.0 / n, eps)


class HeadSink(ctypes.Structure):
    """kipp_gemm_head_sink of the kernel library: where the rows of a fused q/k/v
    projection go when they skip the stored product."""
    _fields_ = [("q_out", c_void_p), ("k_pages", c_void_p), ("v_pages", c_void_p),
                ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("norm_dtype", c_int), ("eps", ctypes.c_float),
                ("cos_sin", c_void_p), ("positions", c_void_p), ("entry_of_token", c_void_p),
                ("block_table", c_void_p), ("table_width", c_int), ("page_size", c_int),
                ("n_q", c_int), ("n_kv", c_int), ("write_cache", c_int)]


def heads_ok(tokens: int, head_dim: int, rotary_dim: int) -> bool:
    """Whether `run_heads` takes a step of this many tokens."""
    return bool(_fn("gemm_tc", "kipp_gemm_tc_heads_ok", [c_int, c_int, c_int])(tokens, head_dim, rotary_dim))


def run_heads(a, w, q_out, k_pages, v_pages, q_norm_w, k_norm_w, eps, cos_sin, positions, entry_of_token,
              block_table, n_q, n_kv, write_cache=True, status=None, fold: NormFold | None = None) -> None:
    """The fused q/k/v projection a @ w.T of a prompt-sized step with per-head norm,
    rotation and the cache write in its epilogue (head_dim 128): what
    `run` followed by `ops.qk_norm_rope_write` gives, bit for bit.  ``cos_sin`` is
    ``ops.rope_table(..., by_pair=True)`` or None."""
    if cos_sin is not None and tuple(cos_sin.shape) != (64, a.shape[0], 2):
        raise KernelError("gemm_tc_heads: cos_sin must be the step's table laid out by pair, [64, tokens, 2]")
    if not tc_ok(a, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned bases and row pitches")
    N, K = w.shape
    if status is None:
        status = _status(a.device)
    sink = HeadSink(_ptr(q_out), _ptr(k_pages), _ptr(v_pages),
                    _ptr(q_norm_w) if q_norm_w is not None else None,
                    _ptr(k_norm_w) if k_norm_w is not None else None,
                    dtype_code(q_norm_w.dtype) if q_norm_w is not None else 0, eps,
                    _ptr(cos_sin) if cos_sin is not None else None, _ptr(positions), _ptr(entry_of_token),
                    _ptr(block_table), block_table.shape[1], k_pages.shape[2], n_q, n_kv, int(write_cache))
    f = _fn("gemm_tc", "kipp_gemm_tc_heads",
            [c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, ctypes.POINTER(NormFold),
             ctypes.POINTER(HeadSink), c_void_p, c_void_p])
    _check(f(_ptr(a), _ptr(w), a.shape[0], N, K, a.stride(0), w.stride(0),
             ctypes.byref(fold) if fold is not None else None, ctypes.byref(sink), _ptr(status), _stream()),
           "gemm_tc_heads")


def run(impl, out, a, w, epilogue, M, splits: int = 0, status=None, tile: int = 0, tile_f: int = 0,
        fold: NormFold | None = None) -> None:
    if impl != "tc":
        raise KernelError(f"unknown gemm implementation {impl!r}")
    if not tc_ok(a, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned bases and row pitches")
    N, K = w.shape
    if status is None:
        status = _status(a.device)
    f = _fn("gemm_tc", "kipp_gemm_tc_fold",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int, c_int,
             c_int, c_int, ctypes.POINTER(NormFold), c_void_p, c_void_p])
    _check(f(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0),
             out.stride(0), EPILOGUES[epilogue], splits, tile, tile_f,
             ctypes.byref(fold) if fold is not None else None, _ptr(status), _stream()), "gemm_tc")


_status_words: dict = {}


def _status(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _status_words:
        _status_words[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status_words[key]


def status_word(device: torch.device) -> torch.Tensor:
    """int32[4]; element 1 is set when a tensor-core kernel gave up a wait."""
    return _status(device)
