"""Each part alone against the plain functions, at sizes that are not the
engine's test configurations."""
import math

import pytest
import torch

import plain_qwen3 as P
from gpu_util import PartHarness, part_tol
from kipp_b200.models.spec import LayerRun
from kipp_b200.parts import (AttentionMixer, NoPositionEncoding, OutputHead, PagedKVSpec, PreNormBlock,
                             RMSNorm, RotaryEncoding, SwiGLUFeedForward, TokenEmbedding)
from kipp_b200.weights import random_tensors

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def weights_for(part, prefix, dtype, seed=0, sigma=0.1):
    t = dict(random_tensors(part.tensor_specs(prefix), seed, sigma=sigma, norm_jitter=0.2))
    if dtype == "bfloat16":
        t = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in t.items()}
    return t


def rounding(dtype):
    return P.bf16_round if dtype == "bfloat16" else P.no_round


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    h = PartHarness(dtype, {})
    norm = RMSNorm(200, 3e-5)
    w = weights_for(norm, "n.", dtype)
    norm.bind(w, "n.", h.runtime)
    ctx = h.context([("a", 6)])
    x = torch.randn(6, 200, device="cuda:0") * 2
    out = norm.forward(ctx, x)
    assert out.dtype == h.runtime.dtype
    assert torch.allclose(out.double().cpu(), P.plain_rmsnorm(x.cpu(), w["n.weight"], 3e-5), **part_tol(dtype))


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
    assert none.rotary_dim == 0 and none.inv_freq("cuda:0") is None


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_heads(dtype):
    h = PartHarness(dtype, {})
    emb = TokenEmbedding(333, 40)
    w = weights_for(emb, "model.embed_tokens.", dtype, sigma=1.0)
    emb.bind(w, "model.embed_tokens.", h.runtime)
    ctx = h.context([("a", 5)])
    ids = torch.tensor([0, 332, 7, 7, 100], dtype=torch.int32, device="cuda:0")
    ctx.meta.token_ids = ids
    x = emb.forward(ctx)
    assert x.dtype == torch.float32
    assert torch.equal(x.cpu(), w["model.embed_tokens.weight"][ids.cpu().long()])
    hidden = torch.randn(3, 40, device="cuda:0").to(h.runtime.dtype)
    tied = OutputHead(333, 40, tied_to=emb)
    assert [s.optional for s in tied.tensor_specs("lm_head.")] == [True]
    tied.bind({}, "lm_head.", h.runtime)
    logits = tied.forward(ctx, hidden, 3)
    ref = P.plain_linear(hidden.float().cpu(), w["model.embed_tokens.weight"])
    assert logits.dtype == torch.float32 and torch.allclose(logits.double().cpu(), ref, **part_tol(dtype))
    own = OutputHead(77, 40)
    wo = weights_for(own, "lm_head.", dtype, seed=3)
    own.bind(wo, "lm_head.", h.runtime)
    logits = own.forward(ctx, hidden, 3)
    assert torch.allclose(logits.double().cpu(), P.plain_linear(hidden.float().cpu(), wo["lm_head.weight"]),
                          **part_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part_adds_to_the_residual(dtype):
    h = PartHarness(dtype, {})
    ffn = SwiGLUFeedForward(72, 200)
    w = weights_for(ffn, "mlp.", dtype, sigma=0.2)
    ffn.bind(w, "mlp.", h.runtime)
    ctx = h.context([("a", 9)])
    hid = torch.randn(9, 72, device="cuda:0").to(h.runtime.dtype)
    res = torch.randn(9, 72, device="cuda:0")
    want = res.double().cpu() + P.plain_feed_forward(hid.float().cpu(), w["mlp.gate_proj.weight"],
                                                     w["mlp.up_proj.weight"], w["mlp.down_proj.weight"],
                                                     rounding(dtype))
    ffn.forward(ctx, hid, res)
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
    spec = mixer.cache_spec()
    assert spec == PagedKVSpec(c["n_kv"], c["D"], c["window"])
    h = PartHarness(dtype, {5: spec}, page_size=8, n_pages=32)
    w = weights_for(mixer, "attn.", dtype, sigma=0.15)
    mixer.bind(w, "attn.", h.runtime)
    run = LayerRun(layer=0, cache=5)
    total = 45
    hid = torch.randn(total, c["hidden"]).to(h.runtime.dtype)
    want = plain_mixer(hid.float(), w, "attn.", c["n_q"], c["n_kv"], c["D"], list(range(total)), 7e4,
                       c["eps"], c["window"], c["rot"], rounding(dtype))
    got = []
    for a, b in ((0, 30), (30, 32), (32, 33), (33, 45)):          # a portion, two tokens, one, a portion
        ctx = h.context([("r", b - a)])
        res = torch.zeros(b - a, c["hidden"], device="cuda:0")
        mixer.forward(ctx, run, hid[a:b].to("cuda:0"), res)
        h.commit()
        got.append(res.cpu())
    assert torch.allclose(torch.cat(got).double(), want, **part_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_alone(dtype):
    cfg = dict(hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
               intermediate_size=144, rms_norm_eps=1e-5, rope_theta=3e4)
    mixer = AttentionMixer(80, 5, 5, 16, RotaryEncoding(16, 3e4), qk_norm_eps=1e-5)
    block = PreNormBlock(RMSNorm(80, 1e-5), mixer, RMSNorm(80, 1e-5), SwiGLUFeedForward(80, 144))
    h = PartHarness(dtype, {0: mixer.cache_spec()}, page_size=4, n_pages=32)
    w = weights_for(block, "model.layers.0.", dtype, sigma=0.12)
    assert len(w) == 11
    block.bind(w, "model.layers.0.", h.runtime)
    x = torch.randn(23, 80)
    want = P.plain_block(x.double(), cfg, w, "model.layers.0.", 0, rounding(dtype))
    ctx = h.context([("r", 23)])
    xd = x.to("cuda:0")
    block.forward(ctx, LayerRun(0, 0), xd)
    h.commit()
    assert torch.allclose(xd.double().cpu(), want, **part_tol(dtype))
