"""Generality of the parts: a toy mixer with state of its own, a layer that is
run twice and a layer that reads another layer's cache are defined HERE,
registered, built and stepped without a change to the framework's files."""
import dataclasses
import math
import os

import pytest
import torch

import plain_qwen3 as P
from tiny import nmse

pytestmark = pytest.mark.gpu


def _register():
    from kipp_b200.config import register_architecture, unregister_architecture
    from kipp_b200.config.base import ModelConfig
    from kipp_b200.models.spec import LayerRun, ModelSpec
    from kipp_b200.parts import (AttentionMixer, Mixer, OutputHead, PreNormBlock, RMSNorm, RotaryEncoding,
                                 StateSpec, SwiGLUFeedForward, TokenEmbedding)
    from kipp_b200.weights import TensorSpec

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int = 97
        hidden_size: int = 48
        state_size: int = 20
        decay: float = 0.8
        intermediate_size: int = 64
        order: tuple = (0, 1, 0)
        share_cache: bool = False
        rms_norm_eps: float = 1e-5
        initializer_range: float = 0.2

    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + W_in h_t ; out_t = W_out s_t, the state s kept
        per request in a slot.  Written with plain torch calls: it is a test
        double, not a kernel."""

        def __init__(self, hidden, state, decay):
            self.hidden, self.state, self.decay = hidden, state, decay

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + "in.weight", (self.state, self.hidden)),
                    TensorSpec(prefix + "out.weight", (self.hidden, self.state))]

        def state_spec(self):
            return StateSpec((self.state,), torch.float32)

        def bind(self, tensors, prefix, runtime):
            self.w_in = tensors[prefix + "in.weight"].to(runtime.device).float()
            self.w_out = tensors[prefix + "out.weight"].to(runtime.device).float()

        def forward(self, ctx, run, h, residual):
            state = ctx.state_view(run)                       # [max_requests, state]
            slots = ctx.meta.slots.tolist()
            at = 0
            for slot, n in zip(slots, ctx.meta.q_lens):       # tokens of a request in order
                u = h[at:at + n].float() @ self.w_in.t()
                s = state[slot].clone()
                for i in range(n):
                    s = self.decay * s + u[i]
                    residual[at + i] += s @ self.w_out.t()
                state[slot] = s
                at += n

    def build(c):
        emb = TokenEmbedding(c.vocab_size, c.hidden_size)
        attn = AttentionMixer(c.hidden_size, 4, 2, 16, RotaryEncoding(16, 1e4), qk_norm_eps=c.rms_norm_eps)
        mk = lambda mixer: PreNormBlock(RMSNorm(c.hidden_size, c.rms_norm_eps), mixer,
                                        RMSNorm(c.hidden_size, c.rms_norm_eps),
                                        SwiGLUFeedForward(c.hidden_size, c.intermediate_size))
        layers = [("model.layers.0.", mk(DecayMixer(c.hidden_size, c.state_size, c.decay))),
                  ("model.layers.1.", mk(attn))]
        if c.share_cache:
            # layers 1 and 2 are attention; run 2 reads the keys and values run 1 wrote
            attn2 = AttentionMixer(c.hidden_size, 4, 2, 16, RotaryEncoding(16, 1e4), qk_norm_eps=c.rms_norm_eps)
            layers.append(("model.layers.2.", mk(attn2)))
            order = [LayerRun(0, cache=0), LayerRun(1, cache=1), LayerRun(2, cache=1, writes_cache=False)]
        else:
            order = [LayerRun(layer, cache=i) for i, layer in enumerate(c.order)]
        return ModelSpec(config=c, hidden_size=c.hidden_size, vocab_size=c.vocab_size, embedding=emb,
                         layers=layers, order=order,
                         final_norm=("model.norm.", RMSNorm(c.hidden_size, c.rms_norm_eps)),
                         head=("lm_head.", OutputHead(c.vocab_size, c.hidden_size, tied_to=emb)),
                         max_positions=256)

    unregister_architecture("ToyStateLM")
    register_architecture("ToyStateLM", ToyConfig, build)
    return ToyConfig


def plain_toy(cfg, w, tokens, share_cache):
    """The same model, whole sequence, float64, no cache and no slots."""
    x = P.plain_embedding(w["model.embed_tokens.weight"], tokens)
    T = len(tokens)
    eps = cfg.rms_norm_eps

    def ffn(x, pre):
        n = P.plain_rmsnorm(x, w[pre + "post_attention_layernorm.weight"], eps)
        return x + P.plain_feed_forward(n, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"],
                                        w[pre + "mlp.down_proj.weight"])

    def decay_layer(x, pre):
        n = P.plain_rmsnorm(x, w[pre + "input_layernorm.weight"], eps)
        u = P.plain_linear(n, w[pre + "self_attn.in.weight"])
        s = torch.zeros(cfg.state_size, dtype=torch.float64)
        out = []
        for t in range(T):
            s = cfg.decay * s + u[t]
            out.append(P.plain_linear(s[None], w[pre + "self_attn.out.weight"])[0])
        return ffn(x + torch.stack(out), pre)

    def qkv(x, pre):
        n = P.plain_rmsnorm(x, w[pre + "input_layernorm.weight"], eps)
        q = P.plain_linear(n, w[pre + "self_attn.q_proj.weight"]).reshape(T, 4, 16)
        k = P.plain_linear(n, w[pre + "self_attn.k_proj.weight"]).reshape(T, 2, 16)
        v = P.plain_linear(n, w[pre + "self_attn.v_proj.weight"]).reshape(T, 2, 16)
        q = P.plain_rope(P.plain_head_norm(q, w[pre + "self_attn.q_norm.weight"], eps), range(T), 1e4)
        k = P.plain_rope(P.plain_head_norm(k, w[pre + "self_attn.k_norm.weight"], eps), range(T), 1e4)
        return q, k, v

    def attn_layer(x, pre, kv=None):
        q, k, v = qkv(x, pre)
        if kv is not None:
            k, v = kv
        a = P.plain_attention(q, k, v).reshape(T, 64)
        return ffn(x + P.plain_linear(a, w[pre + "self_attn.o_proj.weight"]), pre), (k, v)

    if share_cache:
        x = decay_layer(x, "model.layers.0.")
        x, kv = attn_layer(x, "model.layers.1.")
        x, _ = attn_layer(x, "model.layers.2.", kv=kv)
    else:
        for layer in cfg.order:
            x = decay_layer(x, "model.layers.0.") if layer == 0 else attn_layer(x, "model.layers.1.")[0]
    n = P.plain_rmsnorm(x, w["model.norm.weight"], eps)
    return P.plain_linear(n, w["model.embed_tokens.weight"])


@pytest.mark.parametrize("share_cache", [False, True])
def test_toy_architecture_with_state_repeated_layer_and_shared_cache(tmp_path, share_cache):
    ToyConfig = _register()
    from kipp_b200.config import load_config, unregister_architecture
    from kipp_b200.engine import Engine, StepEntry
    from kipp_b200.weights import write_random_model
    from tiny import read_weights
    try:
        cfg = ToyConfig(architecture="ToyStateLM", share_cache=share_cache)
        folder = write_random_model(str(tmp_path / "toy"), cfg, seed=4, sigma=0.2)
        assert load_config(folder) == cfg                        # config.json names the architecture
        w = read_weights(folder)
        eng = Engine.from_folder(folder, dtype="float32", page_size=4, cache_tokens=96, max_requests=3)
        assert len(eng.states) == (1 if share_cache else 2)      # a state per run of the state mixer
        assert [len(g.cache_ids) for g in eng.cache.groups] == [1]
        g = torch.Generator().manual_seed(0)
        seqs = {r: torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
                for r, n in (("a", 31), ("b", 18), ("c", 25), ("d", 9))}
        want = {r: plain_toy(cfg, w, s, share_cache) for r, s in seqs.items()}
        # whole
        got = eng.step([StepEntry("a", seqs["a"], list(range(31)))], check=True).cpu()
        assert nmse(got, want["a"]) < 1e-10
        eng.finish("a")
        # mixed portions: state and pages are carried from step to step; slots and pages are reused
        cuts = {"a": [5, 2, 13, 1, 10], "b": [1, 1, 16], "c": [24, 1], "d": [2, 7]}
        at = {r: 0 for r in seqs}
        live, queue = [], ["a", "b", "c", "d"]
        rows = {}
        while queue or live:
            while queue and len(live) < 3:
                live.append(queue.pop(0))
            entries = []
            for r in live:
                n = cuts[r].pop(0)
                entries.append(StepEntry(r, seqs[r][at[r]:at[r] + n], list(range(n))))
            out = eng.step(entries, check=True).cpu()
            k = 0
            for e in entries:
                for i in range(len(e.tokens)):
                    rows[(e.request, at[e.request] + i)] = out[k]
                    k += 1
                at[e.request] += len(e.tokens)
            for r in list(live):
                if not cuts[r]:
                    live.remove(r)
                    eng.finish(r)
        for (r, pos), row in rows.items():
            assert nmse(row, want[r][pos]) < 1e-10, (r, pos)
        assert len(rows) == sum(len(s) for s in seqs.values())
        eng.cache.check()
        assert eng.cache.slots.free_slots == 3
    finally:
        unregister_architecture("ToyStateLM")
