"""Each part alone against the plain functions, at sizes that are not the
engine's test configurations.  A part is run the way a step runs it
(``Engine.run_part``: the same reservation and metadata, then only that part's
forward pass) inside a model whose other parts are filler."""
import pytest
import torch

import plain_qwen3 as P
from gpu_util import part_engine, part_tol
from kipp_b200.parts import (AttentionMixer, NoPositionEncoding, OutputHead, PagedKVSpec, PreNormBlock,
                             RMSNorm, RotaryEncoding, SwiGLUFeedForward, TokenEmbedding)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"


def rounding(dtype):
    return P.bf16_round if dtype == "bfloat16" else P.no_round


def torch_dtype(dtype):
    return torch.bfloat16 if dtype == "bfloat16" else torch.float32


def filler(hidden):
    return (AttentionMixer(hidden, 1, 1, 16, NoPositionEncoding()), RMSNorm(hidden, 1e-5),
            SwiGLUFeedForward(hidden, 16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    mixer, norm2, ffn = filler(200)
    eng, w = part_engine(dtype, 200, block=PreNormBlock(RMSNorm(200, 3e-5), mixer, norm2, ffn))
    x = torch.randn(6, 200, device=DEV) * 2
    out = torch.empty(6, 200, dtype=torch_dtype(dtype), device=DEV)
    eng.run_part([("a", [0] * 6, [])], 0, "input_norm", residual=x, output=out)
    want = P.plain_rmsnorm(x.cpu(), w["model.layers.0.input_layernorm.weight"], 3e-5)
    assert torch.allclose(out.double().cpu(), want, **part_tol(dtype))
    # the final norm gathers the wanted rows
    out2 = torch.empty(2, 200, dtype=torch_dtype(dtype), device=DEV)
    eng.run_part([("b", [0] * 6, [1, 4])], 0, "final_norm", residual=x, output=out2)
    want2 = P.plain_rmsnorm(x.cpu()[[1, 4]], w["model.norm.weight"], 1e-5)
    assert torch.allclose(out2.double().cpu(), want2, **part_tol(dtype))


def test_rotary_frequencies_and_none():
    rope = RotaryEncoding(48, 5e4)
    f = rope.frequencies()
    assert f.dtype == torch.float32 and f.shape == (24,)
    want = [5e4 ** (-(2.0 * i) / 48) for i in range(24)]
    assert torch.allclose(f.double(), torch.tensor(want, dtype=torch.float64), rtol=2e-7)
    assert RotaryEncoding(64, 1e4, rotary_dim=16).frequencies().shape == (8,)
    with pytest.raises(ValueError):
        RotaryEncoding(64, 1e4, rotary_dim=70)
    none = NoPositionEncoding()
    assert none.rotary_dim == 0 and none.frequencies() is None


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_heads(dtype):
    eng, w = part_engine(dtype, 40, vocab=333, sigma=1.0)
    ids = [0, 332, 7, 7, 100]
    x = torch.zeros(5, 40, device=DEV)
    eng.run_part([("a", ids, [])], 0, "embedding", residual=x)
    assert torch.equal(x.cpu(), w["model.embed_tokens.weight"][ids])
    hidden = torch.randn(3, 40, device=DEV).to(torch_dtype(dtype))
    assert [s.optional for s in OutputHead(333, 40, tied_to="model.embed_tokens.weight").tensor_specs("lm_head.")] \
        == [True]
    logits = torch.empty(3, 333, device=DEV)
    eng.run_part([("b", [1, 2, 3], [0, 1, 2])], 0, "head", input=hidden, output=logits)
    ref = P.plain_linear(hidden.float().cpu(), w["model.embed_tokens.weight"])
    assert torch.allclose(logits.double().cpu(), ref, **part_tol(dtype))
    # a head of its own
    eng2, w2 = part_engine(dtype, 40, vocab=77, head=OutputHead(77, 40), seed=3)
    logits = torch.empty(3, 77, device=DEV)
    eng2.run_part([("b", [1, 2, 3], [0, 1, 2])], 0, "head", input=hidden, output=logits)
    assert torch.allclose(logits.double().cpu(), P.plain_linear(hidden.float().cpu(), w2["lm_head.weight"]),
                          **part_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part_adds_to_the_residual(dtype):
    mixer, norm2, _ = filler(72)
    eng, w = part_engine(dtype, 72, sigma=0.2,
                         block=PreNormBlock(RMSNorm(72, 1e-5), mixer, norm2, SwiGLUFeedForward(72, 200)))
    hid = torch.randn(9, 72, device=DEV).to(torch_dtype(dtype))
    res = torch.randn(9, 72, device=DEV)
    pre = "model.layers.0.mlp."
    want = res.double().cpu() + P.plain_feed_forward(hid.float().cpu(), w[pre + "gate_proj.weight"],
                                                     w[pre + "up_proj.weight"], w[pre + "down_proj.weight"],
                                                     rounding(dtype))
    eng.run_part([("a", [0] * 9, [])], 0, "feed_forward", input=hid, residual=res)
    assert torch.allclose(res.double().cpu(), want, **part_tol(dtype))


def plain_mixer(x_norm, w, pre, n_q, n_kv, D, positions, theta, eps, window, rot, rnd):
    T = x_norm.shape[0]
    q = rnd(P.plain_linear(x_norm, w[pre + "q_proj.weight"])).reshape(T, n_q, D)
    k = rnd(P.plain_linear(x_norm, w[pre + "k_proj.weight"])).reshape(T, n_kv, D)
    v = rnd(P.plain_linear(x_norm, w[pre + "v_proj.weight"])).reshape(T, n_kv, D)
    if eps is not None:
        q = P.plain_head_norm(q, w[pre + "q_norm.weight"], eps)
        k = P.plain_head_norm(k, w[pre + "k_norm.weight"], eps)
    if rot:
        q = torch.cat([P.plain_rope(q[..., :rot], positions, theta), q[..., rot:].double()], -1)
        k = torch.cat([P.plain_rope(k[..., :rot], positions, theta), k[..., rot:].double()], -1)
    a = rnd(P.plain_attention(rnd(q), rnd(k), v, window)).reshape(T, n_q * D)
    return P.plain_linear(a, w[pre + "o_proj.weight"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [
    dict(hidden=72, n_q=6, n_kv=2, D=24, eps=1e-5, window=None, rot=24),
    dict(hidden=64, n_q=4, n_kv=4, D=64, eps=None, window=21, rot=64),          # no q/k norm, a window
    dict(hidden=96, n_q=3, n_kv=1, D=80, eps=2e-6, window=None, rot=32),        # partial rotation
    dict(hidden=64, n_q=2, n_kv=2, D=128, eps=1e-6, window=None, rot=0)])       # no position encoding
def test_attention_mixer_alone_in_two_steps(case, dtype):
    c = case
    pos = RotaryEncoding(c["D"], 7e4, rotary_dim=c["rot"]) if c["rot"] else NoPositionEncoding()
    mixer = AttentionMixer(c["hidden"], c["n_q"], c["n_kv"], c["D"], pos, qk_norm_eps=c["eps"],
                           window=c["window"])
    assert mixer.cache_spec() == PagedKVSpec(c["n_kv"], c["D"], c["window"])
    _, norm2, ffn = filler(c["hidden"])
    eng, w = part_engine(dtype, c["hidden"], sigma=0.15, page_size=8, n_pages=32,
                         block=PreNormBlock(RMSNorm(c["hidden"], 1e-5), mixer, norm2, ffn))
    total = 45
    hid = torch.randn(total, c["hidden"]).to(torch_dtype(dtype))
    want = plain_mixer(hid.float(), w, "model.layers.0.self_attn.", c["n_q"], c["n_kv"], c["D"], list(range(total)),
                       7e4, c["eps"], c["window"], c["rot"], rounding(dtype))
    got = []
    for a, b in ((0, 30), (30, 32), (32, 33), (33, 45)):          # a portion, two tokens, one, a portion
        res = torch.zeros(b - a, c["hidden"], device=DEV)
        eng.run_part([("r", [0] * (b - a), [])], 0, "mixer", input=hid[a:b].to(DEV).contiguous(), residual=res)
        got.append(res.cpu())
    assert eng.length("r") == total
    assert torch.allclose(torch.cat(got).double(), want, **part_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_alone(dtype):
    cfg = dict(hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
               intermediate_size=144, rms_norm_eps=1e-5, rope_theta=3e4)
    mixer = AttentionMixer(80, 5, 5, 16, RotaryEncoding(16, 3e4), qk_norm_eps=1e-5)
    block = PreNormBlock(RMSNorm(80, 1e-5), mixer, RMSNorm(80, 1e-5), SwiGLUFeedForward(80, 144))
    assert len(block.tensor_specs("model.layers.0.")) == 11
    eng, w = part_engine(dtype, 80, sigma=0.12, page_size=4, n_pages=32, block=block)
    x = torch.randn(23, 80)
    want = P.plain_block(x.double(), cfg, w, "model.layers.0.", 0, **(P.BF16_PATH if dtype == "bfloat16" else P.F32_PATH))
    xd = x.to(DEV)
    eng.run_part([("r", [0] * 23, [])], 0, "block", residual=xd)
    assert torch.allclose(xd.double().cpu(), want, **part_tol(dtype))
