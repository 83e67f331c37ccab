"""Random-weights mode: make every tensor a model declares from a seed, and
write a model folder (``config.json`` + ``model.safetensors``).

The reference has no such mode (it always needs a real checkpoint).  Each
tensor draws from its own generator seeded by ``(seed, tensor name)``, so a
tensor's values do not depend on which other tensors exist or on their order.
"""
from __future__ import annotations

import hashlib
import os
from typing import Iterable, Iterator

import torch

from ..config.base import ModelConfig
from .safetensors_io import write_safetensors
from .spec import INIT_INT, INIT_NEAR_ONE, INIT_NORMAL, TensorSpec


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(specs: Iterable[TensorSpec], seed: int, *, sigma: float = 0.02,
                   norm_jitter: float = 0.1, dtype: torch.dtype = torch.float32,
                   device: str | torch.device = "cpu",
                   skip_aliased: bool = True) -> Iterator[tuple[str, torch.Tensor]]:
    """Yield ``(name, tensor)``: matrices N(0, sigma), norm scales
    1 + U(-norm_jitter, norm_jitter), drawn in float32 and stored as ``dtype``."""
    device = torch.device(device)
    for s in specs:
        if skip_aliased and s.optional and s.alias_of is not None:
            continue
        gen = torch.Generator(device=device)
        gen.manual_seed(_tensor_seed(seed, s.name))
        if s.init == INIT_NORMAL:
            t = torch.empty(s.shape, dtype=torch.float32, device=device).normal_(0.0, sigma, generator=gen)
        elif s.init == INIT_NEAR_ONE:
            t = torch.empty(s.shape, dtype=torch.float32, device=device).uniform_(-norm_jitter, norm_jitter, generator=gen)
            t += 1.0
        elif s.init == INIT_INT:
            yield s.name, torch.zeros(s.shape, dtype=torch.int32, device=device)
            continue
        else:
            raise ValueError(f"unknown init {s.init!r} for {s.name}")
        yield s.name, t.to(dtype)


def write_random_model(folder: str, config: ModelConfig, seed: int, *, sigma: float | None = None,
                       norm_jitter: float = 0.1, dtype: torch.dtype = torch.float32) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for
    ``config`` with weights from ``seed``.  Returns ``folder``."""
    from ..config.registry import get_architecture
    spec = get_architecture(config.architecture).build(config)
    if sigma is None:
        sigma = float(getattr(config, "initializer_range", 0.02))
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    write_safetensors(
        os.path.join(folder, "model.safetensors"),
        random_tensors(spec.tensor_specs(), seed, sigma=sigma, norm_jitter=norm_jitter, dtype=dtype),
        metadata={"format": "pt", "seed": str(seed)})
    return folder
