from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_library

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

EPILOGUES = {"store": 0, "add": 1, "swiglu": 2}


from ..native import KernelError  # noqa: E402  (the library's and these wrappers' refusals are one type)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels need CUDA tensors; there is no CPU path")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far in this process."""
    return _launches


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code == -1:
        raise KernelError(f"{what}: the kernel refuses these sizes")
    if code == -2:
        raise KernelError(f"{what}: unsupported dtype combination")
    if code == -3:
        raise KernelError(f"{what}: a pointer or stride is not aligned as the kernel needs")
    if code == -4:
        raise KernelError(f"{what}: these sizes need more scratch than the library holds")
    raise KernelError(f"{what}: CUDA error {code}")


_fn_cache: dict[tuple[str, str], object] = {}


def _fn(lib: str, name: str, argtypes: list, restype=c_int) -> object:
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = argtypes
        f.restype = restype
        _fn_cache[key] = f
    return f


def _int32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------
def embed_gather(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor,
                 status: torch.Tensor) -> None:
    """out[t, :] = float32(table[ids[t], :])."""
    _int32(ids, "ids")
    tokens, hidden = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed_gather: out must be contiguous float32, table contiguous")
    if table.shape[1] != hidden or ids.numel() < tokens:
        raise KernelError("embed_gather: shape mismatch")
    f = _fn("elementwise", "kipp_embed_gather",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(out), _ptr(table), dtype_code(table.dtype), _ptr(ids), tokens, hidden,
             table.shape[0], _ptr(status), _stream()), "embed_gather")


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight, float32 arithmetic."""
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("rmsnorm: x must be contiguous float32")
    size = x.shape[-1]
    if weight.numel() != size or out.shape[-1] != size:
        raise KernelError("rmsnorm: size mismatch")
    if n_rows is None:
        n_rows = rows.numel() if rows is not None else x.shape[0]
    if rows is not None:
        _int32(rows, "rows")
    if out.shape[0] < n_rows:
        raise KernelError("rmsnorm: out has too few rows")
    f = _fn("elementwise", "kipp_rmsnorm",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(out), dtype_code(out.dtype), _ptr(x), _ptr(weight), dtype_code(weight.dtype),
             _ptr(rows), n_rows, size, float(eps), _stream()), "rmsnorm")


def rmsnorm_deferred(out: torch.Tensor, ssq: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                     rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
    """The norm with its row factor left to the reader: out[r] = x[rows[r] or r] * weight
    (rounded to out's type), ssq[r] = sum(x[row]^2); rmsnorm(x)[r] = out[r] * rsqrt(ssq[r] / size + eps)."""
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("rmsnorm_deferred: x must be contiguous float32")
    size = x.shape[-1]
    if weight.numel() != size or out.shape[-1] != size:
        raise KernelError("rmsnorm_deferred: size mismatch")
    if n_rows is None:
        n_rows = rows.numel() if rows is not None else x.shape[0]
    if rows is not None:
        _int32(rows, "rows")
    if out.shape[0] < n_rows or ssq.dtype != torch.float32 or ssq.numel() < n_rows:
        raise KernelError("rmsnorm_deferred: out or ssq has too few rows")
    f = _fn("elementwise", "kipp_rmsnorm_deferred",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(out), dtype_code(out.dtype), _ptr(ssq), _ptr(x), _ptr(weight), dtype_code(weight.dtype),
             _ptr(rows), n_rows, size, _stream()), "rmsnorm_deferred")


def gemm(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: str = "store",
         m: Optional[int] = None, impl: Optional[str] = None) -> None:
    """out = a @ w.T with float32 accumulation; ``a`` [M, K], ``w`` [N, K].

    epilogue "store": out[M, N]; "add": float32 out[M, N] += product;
    "swiglu": out[M, N/2] = silu(p[:, 0::2]) * p[:, 1::2].
    ``m`` limits the rows used.  ``impl`` forces a kernel ("simt", "tc",
    "smallm"); by default float32 runs on the CUDA cores and bfloat16 on the
    tensor-core kernels where they take the shape.
    """
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelError(f"gemm: a {tuple(a.shape)} and w {tuple(w.shape)} do not match")
    if a.dtype != w.dtype:
        raise KernelError("gemm: a and w must have the same dtype")
    M = a.shape[0] if m is None else m
    N, K = w.shape
    n_out = N // 2 if epilogue == "swiglu" else N
    if out.dim() != 2 or out.shape[1] != n_out or out.shape[0] < M:
        raise KernelError(f"gemm: out {tuple(out.shape)} does not fit [{M}, {n_out}]")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: innermost strides must be 1")
    if M == 0:
        return
    if impl is None:
        impl = "simt"
        if a.dtype == torch.bfloat16:
            from . import gemm_bf16
            impl = gemm_bf16.choose(M, N, K, a, w, out, epilogue)
    if impl == "simt":
        f = _fn("gemm_simt", "kipp_gemm_simt",
                [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                 c_int, c_void_p])
        _check(f(_ptr(out), dtype_code(out.dtype), _ptr(a), _ptr(w), dtype_code(a.dtype), M, N, K,
                 a.stride(0), w.stride(0), out.stride(0), EPILOGUES[epilogue], _stream()),
               "gemm_simt")
    else:
        from . import gemm_bf16
        gemm_bf16.run(impl, out, a, w, epilogue, M)


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, tokens: int,
               out: Optional[torch.Tensor] = None, by_pair: bool = False) -> torch.Tensor:
    """float32 [tokens, len(inv_freq), 2]: (cos, sin) of position * inv_freq, made
    once per step and read by every layer's rotation.  ``by_pair``: the same values
    as [len(inv_freq), tokens, 2], for the projection that rotates its own heads."""
    _int32(positions, "positions")
    if inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous():
        raise KernelError("rope_table: inv_freq must be contiguous float32")
    half = inv_freq.numel()
    if out is None:
        shape = (half, tokens, 2) if by_pair else (tokens, half, 2)
        out = torch.empty(shape, dtype=torch.float32, device=positions.device)
    f = _fn("rope_cache", "kipp_rope_table_by_pair" if by_pair else "kipp_rope_table",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(positions), _ptr(inv_freq), tokens, half, _stream()), "rope_table")
    return out


def qk_norm_rope_write(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: Optional[torch.Tensor],
                       v_pages: Optional[torch.Tensor], q_norm_w: Optional[torch.Tensor],
                       k_norm_w: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], rotary_dim: int,
                       positions: torch.Tensor, entry_of_token: torch.Tensor,
                       block_table: torch.Tensor, page_size: int, tokens: int, n_q: int, n_kv: int,
                       head_dim: int, write_cache: bool, status: torch.Tensor,
                       cos_sin: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm of q and k, rotation, q to ``q_out`` [T, n_q, D], k and v
    into pages [page, n_kv, page_size, D] through ``block_table`` [entries, width].
    ``cos_sin`` is the step's ``rope_table``; without it the table is made here."""
    if qkv.stride(1) != 1 or qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError("qk_norm_rope_write: qkv has the wrong width")
    if q_out.dtype != qkv.dtype or not q_out.is_contiguous():
        raise KernelError("qk_norm_rope_write: q_out must be contiguous and of qkv's dtype")
    if write_cache:
        for p in (k_pages, v_pages):
            if p is None or p.dtype != qkv.dtype or not p.is_contiguous() or \
                    tuple(p.shape[1:]) != (n_kv, page_size, head_dim):
                raise KernelError("qk_norm_rope_write: pages must be [pages, n_kv, page_size, D]")
    _int32(positions, "positions"); _int32(entry_of_token, "entry_of_token")
    _int32(block_table, "block_table")
    norm_dtype = 0
    if q_norm_w is not None:
        if k_norm_w is None or q_norm_w.dtype != k_norm_w.dtype:
            raise KernelError("qk_norm_rope_write: q and k norm weights must come together")
        norm_dtype = dtype_code(q_norm_w.dtype)
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != rotary_dim):
        raise KernelError("qk_norm_rope_write: inv_freq must be float32 [rotary_dim / 2]")
    if inv_freq is not None and rotary_dim > 0 and cos_sin is None:
        cos_sin = rope_table(positions, inv_freq, tokens)
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.numel() < tokens * rotary_dim):
        raise KernelError("qk_norm_rope_write: cos_sin must be float32 [tokens, rotary_dim / 2, 2]")
    f = _fn("rope_cache", "kipp_qk_norm_rope_write",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float,
             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_void_p, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
             dtype_code(qkv.dtype), _ptr(q_norm_w), _ptr(k_norm_w), norm_dtype, float(eps),
             _ptr(cos_sin), rotary_dim if cos_sin is not None else 0, _ptr(positions),
             _ptr(entry_of_token), _ptr(block_table), block_table.shape[1], page_size, tokens, n_q,
             n_kv, head_dim, 1 if write_cache else 0, _ptr(status), _stream()),
           "qk_norm_rope_write")


def attention(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
              meta, block_table: torch.Tensor, page_size: int, n_q: int, n_kv: int, head_dim: int,
              scale: float, window: Optional[int], status: torch.Tensor,
              impl: Optional[str] = None) -> None:
    """Causal grouped-query attention of the step's tokens over the paged cache.

    ``meta`` is the step's metadata (``tokens``, ``positions``, ``entry_of_token``
    and the work lists the tensor-core kernels use)."""
    if q.dtype != k_pages.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, pages and out must share a dtype")
    if impl is None:
        impl = "simt"
        if q.dtype == torch.bfloat16:
            from . import attention_bf16
            impl = attention_bf16.choose(meta, n_q, n_kv, head_dim, page_size)
    if impl == "simt":
        f = _fn("attention_simt", "kipp_paged_attention_simt",
                [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                 c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
        _check(f(_ptr(out), _ptr(q), _ptr(k_pages), _ptr(v_pages), dtype_code(q.dtype),
                 _ptr(meta.positions), _ptr(meta.entry_of_token), _ptr(block_table),
                 block_table.shape[1], page_size, meta.tokens, n_q, n_kv, head_dim, float(scale),
                 int(window or 0), _ptr(status), _stream()), "attention_simt")
    else:
        from . import attention_bf16
        attention_bf16.run(impl, out, q, k_pages, v_pages, meta, block_table, page_size, n_q, n_kv,
                           head_dim, scale, window, status)


def attention_decode_fused_ok(meta, dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int,
                              rotary_dim: int) -> bool:
    """Whether :func:`attention_decode_fused` takes this step (decoded tokens only, bfloat16,
    sizes of the split-K kernel, the whole head rotated or none of it)."""
    if dtype != torch.bfloat16:
        return False
    from . import attention_bf16
    return attention_bf16.decode_fused_ok(meta, dtype, n_q, n_kv, head_dim, rotary_dim)


def attention_decode_fused(out: torch.Tensor, qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                           cos_sin: Optional[torch.Tensor], write_cache: bool, meta, block_table: torch.Tensor,
                           page_size: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                           window: Optional[int], status: torch.Tensor) -> None:
    """``qk_norm_rope_write`` and ``attention`` of a step of decoded tokens in one pair of
    launches: the attention kernel normalises and rotates the raw queries and the new key
    itself and writes the new key and value into the pages."""
    from . import attention_bf16
    attention_bf16.decode_fused(out, qkv, k_pages, v_pages, q_norm_w, k_norm_w, eps, cos_sin, write_cache, meta,
                                block_table, page_size, n_q, n_kv, head_dim, scale, window, status)


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of each row's maximum (strict '>' as src/kipp.c:3459-3464)."""
    from . import sampling
    return sampling.argmax_rows(logits, out)


def sample_rows(*args, **kwargs):
    from . import sampling
    return sampling.sample_rows(*args, **kwargs)
