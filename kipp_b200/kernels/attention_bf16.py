"""Launchers of the tensor-core attention kernels (bfloat16) and the choice
between them and the CUDA-core kernel."""
from __future__ import annotations

import ctypes

import torch

from .ops import KernelError, _check, _fn, _ptr, _stream, c_float, c_int, c_void_p

MAX_SPLITS = 32           # key splits of one decoded token

_scratch: dict = {}
_generation = 0


def scratch_generation() -> int:
    """Changes whenever the decode scratch moved (captured graphs go stale)."""
    return _generation


def supported(head_dim: int, n_q: int, n_kv: int) -> bool:
    f = _fn("attention_mma", "kipp_attn_mma_supported", [c_int, c_int, c_int])
    return bool(f(head_dim, n_q, n_kv))


def decode_supported(head_dim: int, n_q: int, n_kv: int) -> bool:
    f = _fn("attention_mma", "kipp_attn_decode_supported", [c_int, c_int, c_int])
    return bool(f(head_dim, n_q, n_kv))


def prefill_tc_supported(head_dim: int, n_q: int, n_kv: int, page_size: int = 0) -> bool:
    """Whether the tcgen05 portion kernel takes these sizes (with a page size:
    also whether its TMA boxes fit the pages)."""
    f = _fn("attention_tc", "kipp_attn_prefill_tc_supported", [c_int, c_int, c_int])
    if not f(head_dim, n_q, n_kv):
        return False
    if page_size:
        return bool(_fn("attention_tc", "kipp_attn_prefill_tc_page_ok", [c_int])(page_size))
    return True


PREFILL_TC = True           # prompt portions on tcgen05 where the sizes allow
PREFILL_TC_MIN_TOKENS = 64  # shorter portions waste a 128-row tile: they stay on mma.sync


def prefill_tc(out, q, k_pages, v_pages, meta, block_table, page_size, n_q, n_kv, head_dim, scale,
               window, status) -> None:
    """Portions of more than one token through the tcgen05 kernel (128-token tiles)."""
    if not (k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape == v_pages.shape
            and tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)):
        raise KernelError("attn_prefill_tc: pages must be contiguous [pages, n_kv, page_size, head_dim]")
    if not q.is_contiguous() or tuple(q.shape[1:]) != (n_q, head_dim):
        raise KernelError("attn_prefill_tc: q must be contiguous [tokens, n_q, head_dim]")
    if not out.is_contiguous() or out.shape != q.shape:
        raise KernelError("attn_prefill_tc: out must be contiguous and of q's shape")
    f = _fn("attention_tc", "kipp_attn_prefill_tc",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(out), _ptr(q), q.shape[0], _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(meta.q_start),
             _ptr(meta.context_len), _ptr(block_table), block_table.shape[1], page_size,
             _ptr(meta.prefill_work128), meta.n_prefill_items128, n_q, n_kv, head_dim, float(scale),
             int(window or 0), _ptr(status), _stream()), "attn_prefill_tc")


def choose(meta, n_q, n_kv, head_dim, page_size) -> str:
    return "mma" if supported(head_dim, n_q, n_kv) else "simt"


def decode_scratch(device: torch.device, n: int, n_q: int, head_dim: int) -> torch.Tensor:
    """float32 scratch of the split-K decode kernel: partial outputs and
    (max, sum) pairs of every split, kept per device and grown on demand."""
    floats = n * n_q * MAX_SPLITS * (head_dim + 2) + n * n_q
    key = (device.type, device.index)
    cur = _scratch.get(key)
    if cur is None or cur.numel() < floats:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("attention scratch must exist before a CUDA graph is captured")
        global _generation
        cur = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _scratch[key] = cur
        _generation += 1
    return cur


def stream_ctas(device: torch.device) -> int:
    """The grid of the stream cut of the decode attention: one wave, three CTAs per SM."""
    return 3 * torch.cuda.get_device_properties(device).multi_processor_count


def stream_ok(n_decode: int) -> bool:
    f = _fn("attention_mma", "kipp_attn_decode_stream_ok", [c_int, c_int])
    return bool(f(n_decode, MAX_SPLITS))


def run(impl, out, q, k_pages, v_pages, meta, block_table, page_size, n_q, n_kv, head_dim, scale,
        window, status, stream: bool = True) -> None:
    """``stream``: the decoded tokens' key tiles are dealt out in equal runs to one wave of
    CTAs; False: every token is cut into splits of ``meta.decode_split_keys`` keys."""
    if impl != "mma":
        raise KernelError(f"unknown attention implementation {impl!r}")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_mma takes bfloat16")
    use_decode = meta.n_decode > 0 and decode_supported(head_dim, n_q, n_kv)
    work, items = (meta.prefill_work, meta.n_prefill_items) if use_decode else (meta.all_work, meta.n_all_items)
    longest = max((n for n in meta.q_lens if n > 1), default=0)
    if (PREFILL_TC and meta.n_prefill_items128 and longest >= PREFILL_TC_MIN_TOKENS
            and (use_decode or meta.n_decode == 0) and prefill_tc_supported(head_dim, n_q, n_kv, page_size)
            and all(t.data_ptr() % 16 == 0 for t in (out, q, k_pages, v_pages))):
        prefill_tc(out, q, k_pages, v_pages, meta, block_table, page_size, n_q, n_kv, head_dim, scale, window,
                   status)
    elif items:
        f = _fn("attention_mma", "kipp_attn_prefill_mma",
                [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                 c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
        _check(f(_ptr(out), _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(meta.q_start),
                 _ptr(meta.context_len), _ptr(block_table), block_table.shape[1], page_size, _ptr(work),
                 items, n_q, n_kv, head_dim, float(scale), int(window or 0), _stream()),
               "attn_prefill_mma")
    if use_decode:
        scratch = decode_scratch(q.device, meta.n_decode, n_q, head_dim)
        f = _fn("attention_mma", "kipp_attn_decode_mma",
                [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                 c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                 c_void_p])
        ctas = stream_ctas(q.device) if stream and stream_ok(meta.n_decode) else 0
        _check(f(_ptr(out), _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(meta.q_start),
                 _ptr(meta.context_len), _ptr(block_table), block_table.shape[1], page_size,
                 _ptr(meta.decode_rows), meta.n_decode, n_q, n_kv, head_dim, float(scale),
                 int(window or 0), MAX_SPLITS, _ptr(meta.decode_split_keys), _split_stride(meta), ctas,
                 _ptr(scratch), _stream()),
               "attn_decode_mma")


def _split_stride(meta) -> int:
    """1 when ``meta.decode_split_keys`` holds one split length per decoded token,
    0 when it holds one for the whole step."""
    return 1 if meta.decode_split_keys.numel() >= max(meta.n_decode, 2) else 0


def decode_replan(split_keys: torch.Tensor, context_len: torch.Tensor, rows: torch.Tensor, pairs_per_entry: int,
                  resident_ctas: int, fixed_tiles: int, max_splits: int, own_length: bool) -> None:
    """The keys per split of every decoded token, chosen on the device from the
    cached lengths (between the steps of a burst that runs without the host)."""
    n = rows.numel()
    for t in (split_keys, context_len, rows):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("decode_replan takes contiguous int32 tensors")
    if split_keys.numel() < n:
        raise KernelError("decode_replan: one split length per decoded token")
    f = _fn("attention_mma", "kipp_attn_decode_replan",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(split_keys), _ptr(context_len), _ptr(rows), n, pairs_per_entry, resident_ctas, fixed_tiles,
             max_splits, 1 if own_length else 0, _stream()), "attn_decode_replan")


def decode_fused_ok(meta, q_dtype, n_q: int, n_kv: int, head_dim: int, rotary_dim: int) -> bool:
    """Whether a step can take :func:`decode_fused`: decoded tokens only, bfloat16,
    a head size and group the split-K kernel takes, the whole head rotated or none of it."""
    return (q_dtype == torch.bfloat16 and meta.n_decode == meta.entries == meta.tokens and meta.n_decode > 0
            and rotary_dim in (0, head_dim) and decode_supported(head_dim, n_q, n_kv))


def decode_fused(out, qkv, k_pages, v_pages, q_norm_w, k_norm_w, eps, cos_sin, write_cache: bool, meta,
                 block_table, page_size, n_q, n_kv, head_dim, scale, window, status, stream: bool = True) -> None:
    """Attention of a step of decoded tokens straight from the raw q/k/v projection:
    the per-head norm, the rotation and the write of the new key and value happen in
    the attention kernel (no launch of their own)."""
    from .ops import dtype_code
    if qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1 or qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError("decode_fused: qkv must be bfloat16 [tokens, (n_q + 2 n_kv) * head_dim]")
    if (q_norm_w is None) != (k_norm_w is None):
        raise KernelError("decode_fused: q and k norm weights must come together")
    norm_dtype = dtype_code(q_norm_w.dtype) if q_norm_w is not None else 0
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous()):
        raise KernelError("decode_fused: cos_sin must be contiguous float32 [tokens, head_dim / 2, 2]")
    scratch = decode_scratch(qkv.device, meta.n_decode, n_q, head_dim)
    f = _fn("attention_mma", "kipp_attn_decode_mma_fused",
            [c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float,
             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
             c_float, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    ctas = stream_ctas(qkv.device) if stream and stream_ok(meta.n_decode) else 0
    _check(f(_ptr(out), _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(q_norm_w), _ptr(k_norm_w),
             norm_dtype, float(eps), _ptr(cos_sin), 1 if write_cache else 0, _ptr(meta.q_start),
             _ptr(meta.context_len), _ptr(block_table), block_table.shape[1], page_size,
             _ptr(meta.decode_rows), meta.n_decode, n_q, n_kv, head_dim, float(scale), int(window or 0),
             MAX_SPLITS, _ptr(meta.decode_split_keys), _split_stride(meta), ctas, _ptr(scratch), _ptr(status),
             _stream()),
           "attn_decode_mma_fused")
