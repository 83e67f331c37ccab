"""Weights: safetensors reading, binding by name, the one error that lists
everything, random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from kipp_b200.config import config_from_dict, get_architecture
from kipp_b200.weights import (WeightError, load_tensors, open_checkpoint, random_tensors,
                               write_random_model, write_safetensors)
from tiny import CONFIGS, TINY_A, TINY_B, make_model_folder, read_weights


def spec_of(cfg):
    c = config_from_dict(cfg)
    return get_architecture(c.architecture).build(c)


def test_tensor_count_and_names():
    a, b = spec_of(TINY_A), spec_of(TINY_B)
    # 2 + 11 L, plus the head: optional alias when tied (src/kipp.c:1108-1111)
    assert len([s for s in a.tensor_specs() if not s.optional]) == 2 + 11 * 2
    assert len(b.tensor_specs()) == 2 + 11 * 3 + 1
    names = {s.name: s.shape for s in b.tensor_specs()}
    assert names["model.layers.2.self_attn.q_proj.weight"] == (256, 128)
    assert names["model.layers.0.self_attn.k_proj.weight"] == (32, 128)
    assert names["model.layers.0.self_attn.o_proj.weight"] == (128, 256)
    assert names["model.layers.1.self_attn.q_norm.weight"] == (32,)
    assert names["model.layers.1.mlp.down_proj.weight"] == (128, 352)
    assert names["lm_head.weight"] == (1000, 128)
    assert names["model.norm.weight"] == (128,)


def test_random_folder_roundtrip_and_dtypes(tmp_path):
    d = make_model_folder(str(tmp_path / "a"), "A")
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    t = load_tensors(d, spec_of(TINY_A).tensor_specs())
    ref = read_weights(d)                                  # the safetensors package reads it too
    assert set(t) == set(ref)
    for k in t:
        assert t[k].dtype == torch.float32                 # stored in 32-bit stays so
        assert torch.equal(t[k], ref[k])
    w = t["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002
    n = t["model.norm.weight"]
    assert 0.9 <= float(n.min()) and float(n.max()) <= 1.1 and float(n.std()) > 0.01
    # same seed -> same values; another seed -> other values; bf16 stays bf16
    d2 = make_model_folder(str(tmp_path / "a2"), "A")
    assert torch.equal(read_weights(d2)["model.norm.weight"], n)
    d3 = make_model_folder(str(tmp_path / "b16"), "A", dtype=torch.bfloat16)
    t3 = load_tensors(d3, spec_of(TINY_A).tensor_specs())
    assert all(v.dtype == torch.bfloat16 for v in t3.values())
    assert torch.equal(t3["model.norm.weight"], n.to(torch.bfloat16))


def test_tensor_values_do_not_depend_on_other_tensors():
    specs = spec_of(TINY_B).tensor_specs()
    full = dict(random_tensors(specs, 1))
    alone = dict(random_tensors([s for s in specs if s.name == "model.norm.weight"], 1))
    assert torch.equal(full["model.norm.weight"], alone["model.norm.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_folder(str(tmp_path / "b"), "B")
    w = read_weights(d)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["lm_head.weight"]                                   # untied: the head is required
    w["model.layers.9.extra.weight"] = torch.zeros(3)
    w["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(16)
    w["model.embed_tokens.weight"] = w["model.embed_tokens.weight"].to(torch.float64)
    write_safetensors(os.path.join(d, "model.safetensors"), w.items())
    with pytest.raises(WeightError) as e:
        load_tensors(d, spec_of(TINY_B).tensor_specs())
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"] or \
        set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "lm_head.weight"}
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_norm.weight", (16,), (32,))]
    assert err.wrong_dtype and err.wrong_dtype[0][0] == "model.embed_tokens.weight"
    text = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape", "expected [32]",
                   "unsupported dtype"):
        assert needle in text


def test_tied_head_may_be_absent_or_present(tmp_path):
    d = make_model_folder(str(tmp_path / "a"), "A")
    specs = spec_of(TINY_A).tensor_specs()
    assert "lm_head.weight" not in read_weights(d)
    load_tensors(d, specs)
    w = read_weights(d)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), w.items())
    t = load_tensors(d, specs)                              # accepted and ignored
    assert "lm_head.weight" not in t


def test_sharded_checkpoint_and_bad_files(tmp_path):
    d = make_model_folder(str(tmp_path / "a"), "A")
    w = read_weights(d)
    names = sorted(w)
    half = len(names) // 2
    os.remove(os.path.join(d, "model.safetensors"))
    write_safetensors(os.path.join(d, "s1.safetensors"), [(n, w[n]) for n in names[:half]])
    write_safetensors(os.path.join(d, "s2.safetensors"), [(n, w[n]) for n in names[half:]])
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors")
                            for i, n in enumerate(names)}}
    json.dump(index, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    t = load_tensors(d, spec_of(TINY_A).tensor_specs())
    assert all(torch.equal(t[n], w[n]) for n in names)
    # a truncated file and a header that lies about a byte range are refused
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps(TINY_A))
    (bad / "model.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(WeightError, match="truncated"):
        load_tensors(str(bad), spec_of(TINY_A).tensor_specs())
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 64]}}).encode()
    (bad / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 16)
    with pytest.raises(WeightError, match="byte range"):
        load_tensors(str(bad), spec_of(TINY_A).tensor_specs())
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(WeightError, match="neither"):
        load_tensors(str(empty), spec_of(TINY_A).tensor_specs())
