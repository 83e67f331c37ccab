"""The host core without a device: every kernel launcher it names exists in the
kernel library it names, and its C interface answers for configuration, plans
and registries (no GPU)."""
import ctypes
import json
import os
import re

import pytest

from kipp_b200 import native as N
from kipp_b200.csrc import build
from tiny import TINY_A, TINY_B

HOST = os.path.join(os.path.dirname(os.path.abspath(build.__file__)), "host")


def test_every_launcher_the_host_core_names_exists():
    src = open(os.path.join(HOST, "kernels.hpp")).read()
    named = re.findall(r'kernel_symbol<\w+>\("(\w+)", "(\w+)"\)', src)
    assert len(named) >= 15
    for library, symbol in named:
        lib = ctypes.CDLL(build.compile_library(library, verbose=False))
        assert hasattr(lib, symbol), f"lib{library}.so lacks {symbol}"


def test_registries_and_plans():
    lib = N.lib()
    reg = json.loads(lib.kipp_registered().decode())
    assert "Qwen3ForCausalLM" in reg["architectures"]
    assert {"attention", "swiglu", "rmsnorm", "rotary", "token_embedding", "output_head", "pre_norm_block",
            "external", "frequency_table", "no_position"} <= set(reg["part_kinds"])
    plan = json.loads(N.text_result(lib.kipp_plan_from_config, json.dumps(TINY_B).encode()))
    assert len(plan["layers"]) == 3 and plan["head"]["part"]["tied_to"] is None
    mixer = plan["layers"][1]["part"]["mixer"]
    assert (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == (8, 1, 32)
    assert mixer["position"] == {"kind": "rotary", "head_dim": 32, "theta": 1000000.0}
    tied = json.loads(N.text_result(lib.kipp_plan_from_config, json.dumps(TINY_A).encode()))
    assert tied["head"]["part"]["tied_to"] == "model.embed_tokens.weight"
    # a plan with a part kind nobody registered is refused by name
    plan["layers"][0]["part"]["ffn"]["kind"] = "gelu_mlp"
    with pytest.raises(ValueError, match="unknown part kind 'gelu_mlp'"):
        N.text_result(lib.kipp_plan_tensor_specs, json.dumps(plan).encode())


def test_split_rule_of_the_decode_attention():
    lib = N.lib()
    # few (token, kv head) pairs: many short splits; many pairs: few long ones
    few, many = lib.kipp_attention_split_length(1, 2048, 8, 148, 0), lib.kipp_attention_split_length(64, 2048, 8, 148, 0)
    assert few == 64 and many >= 512 and many % 64 == 0        # one token: one tile per split (latency)
    assert lib.kipp_attention_split_length(1, 100, 8, 148, 0) == 64
    assert lib.kipp_attention_split_length(8, 2048, 8, 148, 0) == 384      # 6 splits: 384 CTAs, one wave
    # from the token's own context: an eighth of it, in whole 64-key tiles, at least one tile
    assert lib.kipp_attention_split_length(1, 8192, 8, 148, 1) == 1024
    assert lib.kipp_attention_split_length(1, 700, 8, 148, 1) == 128
    assert lib.kipp_attention_split_length(1, 300, 8, 148, 1) == 64
    assert lib.kipp_attention_split_length(1, 2049, 8, 148, 1) == 320
    # dealt out as a stream where splits of one length would need several waves or leave one half empty
    def stream(n, keys):
        arr = (ctypes.c_int * n)(*([keys] * n))
        return lib.kipp_attention_stream_pays(n, arr, 8, 148)
    assert [stream(n, 2049) for n in (1, 8, 16, 64)] == [0, 0, 0, 1]      # 512 pairs on 444 places: four waves of splits
    assert stream(8, 8031) == 0 and stream(64, 4097) == 1
