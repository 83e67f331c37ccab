"""Choice among the bfloat16 attention kernels."""
from __future__ import annotations


def choose(meta, n_q, n_kv, head_dim, page_size) -> str:
    return "simt"


def run(impl, *args) -> None:
    raise NotImplementedError(impl)
