"""The Qwen3 dense decoder.  Its configuration checks and its plan (per layer:
RMSNorm -> attention with per-head q/k RMSNorm and rotary encoding -> add ->
RMSNorm -> SwiGLU feed-forward -> add; a final RMSNorm and the output head, tied
to the embedding or not) are the host core's (csrc/host/qwen3.hpp); this module
registers the typed configuration class on the Python side.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from .spec import ModelSpec


def build_qwen3(config: Qwen3Config) -> ModelSpec:
    return ModelSpec.from_library(config)


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3)
