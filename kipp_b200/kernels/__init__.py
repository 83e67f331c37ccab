"""Python face of the hand-written sm_100a kernels (``kipp_b200/csrc``).

Every function takes CUDA tensors, launches on the current CUDA stream and
returns nothing or its output tensor.  There is no CPU or library fallback: a
tensor that is not on a CUDA device, a size a kernel refuses, or a library
that cannot be built raises.
"""
from .ops import (KernelError, argmax_rows, attention, attention_decode_fused, attention_decode_fused_ok,
                  embed_gather, gemm, qk_norm_rope_write, rmsnorm, rmsnorm_deferred, rope_table, sample_rows,
                  dtype_code)

__all__ = ["KernelError", "argmax_rows", "attention", "attention_decode_fused", "attention_decode_fused_ok",
           "embed_gather", "gemm", "qk_norm_rope_write", "rmsnorm", "rmsnorm_deferred", "rope_table", "sample_rows", "dtype_code"]
