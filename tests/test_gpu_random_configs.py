"""Random configurations of the architecture with the head sizes the tensor-core
attention takes (64 and 128), long prompts cut so that the prompt-sized kernels
run (a portion of 1,024 tokens and more: the CTA-pair GEMM; 512 and more: the
persistent GEMM and the reducing stores; 64 and more: the tcgen05 attention),
odd portions and single tokens after them, windows, every page size: the
engine in bfloat16 against the plain model."""
import os
import random

import pytest
import torch

import plain_qwen3 as P
from tiny import nmse, read_config, read_weights

pytestmark = pytest.mark.gpu


def _random_config(rng: random.Random) -> tuple[dict, int, int]:
    head_dim = rng.choice([64, 128])
    kv_heads = rng.choice([1, 2, 3])
    heads = kv_heads * rng.choice([1, 2, 4, 5])
    layers = rng.choice([1, 2])
    window = rng.choice([None, 100, 333, 700])
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=rng.choice([300, 515, 1000]),
               hidden_size=rng.choice([64, 96, 136, 200]), intermediate_size=rng.choice([96, 168, 264]),
               num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
               head_dim=head_dim, max_position_embeddings=2048, rope_theta=rng.choice([1e4, 1e6]),
               rms_norm_eps=rng.choice([1e-6, 1e-5]), tie_word_embeddings=rng.random() < 0.5, hidden_act="silu",
               attention_bias=False, initializer_range=0.05, torch_dtype="float32")
    if window:
        cfg["sliding_window"] = window
        cfg["layer_types"] = [rng.choice(["sliding_attention", "full_attention"]) for _ in range(layers)]
    return cfg, rng.choice([8, 16, 32, 64, 128]), rng.choice([1030, 1100, 1300, 1536])


@pytest.mark.parametrize("seed", [101, 202, 303, 110, 155, 214])
def test_random_configuration_against_the_plain_model(tmp_path, seed):
    from kipp_b200.config import config_from_dict
    from kipp_b200.engine import Engine, StepEntry
    from kipp_b200.weights import write_random_model
    rng = random.Random(seed)
    cfg, page, T = _random_config(rng)
    folder = write_random_model(str(tmp_path / "m"), config_from_dict(cfg), seed=seed, sigma=0.05)
    c, w = read_config(folder), read_weights(folder)
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, cfg["vocab_size"], (T + 12,), generator=g).tolist()
    eng = Engine.from_folder(folder, dtype="bfloat16", page_size=page, cache_tokens=T + 12 + 4 * page,
                             max_requests=2, max_batch_tokens=1600)
    first = rng.choice([1024, 1025, max(1024, T - 200), 600])
    cuts, at = [first], first
    while at < T:
        n = min(T - at, rng.choice([2, 7, 64, 65, 130, 300]))
        cuts.append(n)
        at += n
    cuts += [1] * 12
    rows, at = [], 0
    for n in cuts:
        want = sorted({0, n - 1, rng.randrange(n)})
        out = eng.step([StepEntry("r", toks[at:at + n], want)], check=True).double().cpu()
        rows += [(at + i, out[k]) for k, i in enumerate(want)]
        at += n
    wb = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in w.items()}
    ref = P.plain_forward(c, wb, toks[:at], kv_rounding=P.bf16_round, **P.BF16_PATH).double()
    worst = max((nmse(r, ref[pos]), pos) for pos, r in rows)
    assert worst[0] < 1e-4, (cfg, page, cuts, worst)
    eng.finish("r")
    eng.cache.check()
    assert eng.cache.free_pages() == [g.pool.n_pages for g in eng.cache.groups]
