"""Generality of the parts: a toy mixer with state of its own, a layer that is
run twice, a layer that reads another layer's cache, a feed-forward with
routing, a scaled partial rotation and positions learned at the embedding are
defined HERE, registered, built and stepped without a change to the
framework's files."""
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
                         head=("lm_head.", OutputHead(c.vocab_size, c.hidden_size,
                                                      tied_to="model.embed_tokens.weight")),
                         embedding_prefix="model.embed_tokens.", max_positions=256)

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


def test_state_mixer_in_bfloat16_with_graphs_asked_for(tmp_path):
    """A part defined in Python is not captured in CUDA graphs (it does not say it
    may be): with graphs switched on the engine runs such a model's decode steps as
    plain launches, and the state of a request advances once per step."""
    ToyConfig = _register()
    from kipp_b200.config import unregister_architecture
    from kipp_b200.engine import Engine, StepEntry
    from kipp_b200.weights import write_random_model
    from tiny import read_weights
    try:
        cfg = ToyConfig(architecture="ToyStateLM")
        folder = write_random_model(str(tmp_path / "toy16"), cfg, seed=5, sigma=0.2)
        w = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in read_weights(folder).items()}
        eng = Engine.from_folder(folder, dtype="bfloat16", page_size=4, cache_tokens=96, max_requests=3,
                                 cuda_graphs=True)
        assert not eng.cuda_graphs and eng.info()["cuda_graphs"] is False
        g = torch.Generator().manual_seed(1)
        seq = torch.randint(0, cfg.vocab_size, (30,), generator=g).tolist()
        want = plain_toy(cfg, w, seq, False)
        rows = [eng.step([StepEntry("a", seq[:12], [11])], check=True).cpu().clone()]
        for t in seq[12:]:                                    # decode steps: each advances the state once
            rows.append(eng.step([StepEntry("a", [t], [0])], check=True).cpu().clone())
        got = torch.cat(rows)
        assert nmse(got, want[11:]) < 2e-3                    # bfloat16 activations against a float64 model
        assert eng.graph_replays == 0
    finally:
        unregister_architecture("ToyStateLM")


# ---------------------------------------------------------------------------------------
# A feed-forward with routing, a rotation of another kind and a position encoding that is
# not a rotation at all: toy parts again, defined here, beside the framework's attention.
def _register_routed():
    from kipp_b200.config import register_architecture, unregister_architecture
    from kipp_b200.config.base import ModelConfig
    from kipp_b200.models.spec import LayerRun, ModelSpec
    from kipp_b200.parts import (AttentionMixer, EmbeddingStage, FeedForward, NoPositionEncoding, OutputHead,
                                 PositionEncoding, PreNormBlock, RMSNorm, SwiGLUFeedForward, TokenEmbedding)
    from kipp_b200.weights import TensorSpec

    @dataclasses.dataclass(frozen=True)
    class ToyRoutedConfig(ModelConfig):
        vocab_size: int = 61
        hidden_size: int = 40
        num_experts: int = 5
        experts_per_token: int = 2
        expert_size: int = 24
        intermediate_size: int = 56
        max_positions: int = 96
        rotary_dim: int = 8
        rope_theta: float = 500.0
        rope_scale: float = 4.0
        rms_norm_eps: float = 1e-5
        initializer_range: float = 0.3

    class RoutedFeedForward(FeedForward):
        """Router logits and softmax in float32, the experts_per_token largest
        probabilities renormalised, each chosen expert a SwiGLU of its own.
        Plain torch calls: a test double, not a kernel."""

        def __init__(self, hidden, experts, top_k, size):
            self.hidden, self.experts, self.top_k, self.size = hidden, experts, top_k, size

        def tensor_specs(self, prefix):
            e, h, s = self.experts, self.hidden, self.size
            return [TensorSpec(prefix + "router.weight", (e, h)), TensorSpec(prefix + "experts.gate", (e, s, h)),
                    TensorSpec(prefix + "experts.up", (e, s, h)), TensorSpec(prefix + "experts.down", (e, h, s))]

        def bind(self, tensors, prefix, runtime):
            get = lambda n: tensors[prefix + n].to(runtime.device).float()
            self.router, self.gate, self.up, self.down = (get("router.weight"), get("experts.gate"),
                                                          get("experts.up"), get("experts.down"))

        def forward(self, ctx, h, residual):
            T = ctx.meta.tokens
            x = h[:T].float()
            prob = torch.softmax(x @ self.router.t(), dim=-1)
            top, idx = torch.topk(prob, self.top_k, dim=-1)
            top = top / top.sum(-1, keepdim=True)
            for e in range(self.experts):
                rows, slot = (idx == e).nonzero(as_tuple=True)
                if rows.numel() == 0:
                    continue
                xe = x[rows]
                act = torch.nn.functional.silu(xe @ self.gate[e].t()) * (xe @ self.up[e].t())
                residual[:T].index_add_(0, rows, (act @ self.down[e].t()) * top[rows, slot, None])

    class ScaledPartialRotary(PositionEncoding):
        """The first rotary_dim dims of a head rotate, with frequencies divided
        by a scale (positions stretched): another table than the dense layer's."""

        def __init__(self, rotary_dim, theta, scale):
            self.rotary_dim, self.theta, self.scale = rotary_dim, theta, scale

        def frequencies(self):
            i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            return (self.theta ** (-2.0 * i / self.rotary_dim) / self.scale).float()

        def table_key(self):
            return ("toy-scaled", self.theta, self.rotary_dim, self.scale)

    class LearnedPositions(EmbeddingStage):
        """x_t += P[position_t]: positions enter at the bottom, after the token
        embedding and not in the mixer."""

        def __init__(self, hidden, max_positions):
            self.hidden_size, self.max_positions = hidden, max_positions

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + "weight", (self.max_positions, self.hidden_size))]

        def bind(self, tensors, prefix, runtime):
            self.positions = tensors[prefix + "weight"].to(runtime.device).float()

        def forward(self, ctx, x):
            T = ctx.meta.tokens
            x[:T] += self.positions[ctx.meta.positions[:T].long()]

    def build(c):
        emb = [("model.embed_tokens.", TokenEmbedding(c.vocab_size, c.hidden_size)),
               ("model.embed_positions.", LearnedPositions(c.hidden_size, c.max_positions))]
        norm = lambda: RMSNorm(c.hidden_size, c.rms_norm_eps)
        rotary = ScaledPartialRotary(c.rotary_dim, c.rope_theta, c.rope_scale)
        layers = [
            ("model.layers.0.", PreNormBlock(
                norm(), AttentionMixer(c.hidden_size, 4, 2, 16, NoPositionEncoding(), qk_norm_eps=c.rms_norm_eps),
                norm(), RoutedFeedForward(c.hidden_size, c.num_experts, c.experts_per_token, c.expert_size))),
            ("model.layers.1.", PreNormBlock(
                norm(), AttentionMixer(c.hidden_size, 6, 3, 16, rotary, qk_norm_eps=c.rms_norm_eps),
                norm(), SwiGLUFeedForward(c.hidden_size, c.intermediate_size))),
        ]
        return ModelSpec(config=c, hidden_size=c.hidden_size, vocab_size=c.vocab_size, embedding=emb,
                         layers=layers, order=[LayerRun(0, cache=0), LayerRun(1, cache=1)],
                         final_norm=("model.norm.", norm()),
                         head=("lm_head.", OutputHead(c.vocab_size, c.hidden_size,
                                                      tied_to="model.embed_tokens.weight")),
                         max_positions=c.max_positions)

    unregister_architecture("ToyRoutedLM")
    register_architecture("ToyRoutedLM", ToyRoutedConfig, build)
    return ToyRoutedConfig, ScaledPartialRotary


def plain_routed(cfg, w, tokens, inv_freq):
    """Whole sequence, float64.  Returns the logits and, per token, the gap
    between the last chosen and the first rejected router probability."""
    T = len(tokens)
    eps = cfg.rms_norm_eps
    x = P.plain_embedding(w["model.embed_tokens.weight"], tokens) + w["model.embed_positions.weight"][:T].double()

    def attention(x, pre, heads, kv_heads, rotate):
        n = P.plain_rmsnorm(x, w[pre + "input_layernorm.weight"], eps)
        q = P.plain_linear(n, w[pre + "self_attn.q_proj.weight"]).reshape(T, heads, 16)
        k = P.plain_linear(n, w[pre + "self_attn.k_proj.weight"]).reshape(T, kv_heads, 16)
        v = P.plain_linear(n, w[pre + "self_attn.v_proj.weight"]).reshape(T, kv_heads, 16)
        q = P.plain_head_norm(q, w[pre + "self_attn.q_norm.weight"], eps)
        k = P.plain_head_norm(k, w[pre + "self_attn.k_norm.weight"], eps)
        if rotate:
            rot = cfg.rotary_dim
            # angle = float32(position) * float32(frequency), as the kernel forms it
            angle = (torch.arange(T, dtype=torch.float32)[:, None] * inv_freq[None, :]).double()[:, None, :]

            def turn(h):
                lo, hi = h[..., :rot // 2], h[..., rot // 2:rot]
                return torch.cat([lo * torch.cos(angle) - hi * torch.sin(angle),
                                  hi * torch.cos(angle) + lo * torch.sin(angle), h[..., rot:]], -1)
            q, k = turn(q), turn(k)
        a = P.plain_attention(q, k, v).reshape(T, heads * 16)
        return x + P.plain_linear(a, w[pre + "self_attn.o_proj.weight"])

    x = attention(x, "model.layers.0.", 4, 2, False)
    pre = "model.layers.0."
    n = P.plain_rmsnorm(x, w[pre + "post_attention_layernorm.weight"], eps)
    prob = torch.softmax(P.plain_linear(n, w[pre + "mlp.router.weight"]), dim=-1)
    ranked = torch.sort(prob, dim=-1, descending=True)
    k_top = cfg.experts_per_token
    gaps = ranked.values[:, k_top - 1] - ranked.values[:, k_top]
    out = torch.zeros_like(x)
    for t in range(T):
        chosen = ranked.indices[t, :k_top]
        share = prob[t, chosen] / prob[t, chosen].sum()
        for e, s in zip(chosen.tolist(), share):
            act = P.plain_silu(P.plain_linear(n[t], w[pre + "mlp.experts.gate"][e])) * \
                P.plain_linear(n[t], w[pre + "mlp.experts.up"][e])
            out[t] += s * P.plain_linear(act, w[pre + "mlp.experts.down"][e])
    x = x + out
    x = attention(x, "model.layers.1.", 6, 3, True)
    pre = "model.layers.1."
    n = P.plain_rmsnorm(x, w[pre + "post_attention_layernorm.weight"], eps)
    x = x + P.plain_feed_forward(n, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"],
                                 w[pre + "mlp.down_proj.weight"])
    n = P.plain_rmsnorm(x, w["model.norm.weight"], eps)
    return P.plain_linear(n, w["model.embed_tokens.weight"]), gaps


def test_toy_routed_feed_forward_and_other_position_encodings(tmp_path):
    """Layer by layer different parts: a routed feed-forward under an attention
    without rotation (positions are learned vectors added at the embedding),
    then the dense feed-forward under an attention with a scaled, partial
    rotation.  Whole sequences and mixed portions against the plain model."""
    ToyRoutedConfig, ScaledPartialRotary = _register_routed()
    from kipp_b200.config import load_config, unregister_architecture
    from kipp_b200.engine import Engine, StepEntry
    from kipp_b200.weights import write_random_model
    from tiny import read_weights
    try:
        cfg = ToyRoutedConfig(architecture="ToyRoutedLM")
        folder = write_random_model(str(tmp_path / "routed"), cfg, seed=7, sigma=cfg.initializer_range)
        assert load_config(folder) == cfg
        w = read_weights(folder)
        inv_freq = ScaledPartialRotary(cfg.rotary_dim, cfg.rope_theta, cfg.rope_scale).frequencies()
        eng = Engine.from_folder(folder, dtype="float32", page_size=8, cache_tokens=160, max_requests=3)
        assert [len(g.cache_ids) for g in eng.cache.groups] == [1, 1]     # 2 and 3 kv heads: pages of their own
        g = torch.Generator().manual_seed(3)
        seqs = {r: torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
                for r, n in (("a", 40), ("b", 23), ("c", 9))}
        want = {r: plain_routed(cfg, w, s, inv_freq) for r, s in seqs.items()}
        # a token whose router choice hangs on less than float32 can tell is not compared
        sure = {r: (gaps > 1e-5) for r, (_, gaps) in want.items()}
        assert sum(int(s.sum()) for s in sure.values()) >= 0.9 * sum(len(s) for s in seqs.values())
        got = eng.step([StepEntry("a", seqs["a"], list(range(40)))], check=True).cpu()
        first_unsure = int((~sure["a"]).nonzero()[0]) if (~sure["a"]).any() else 40
        assert nmse(got[:first_unsure], want["a"][0][:first_unsure]) < 1e-10
        eng.finish("a")
        cuts = {"a": [3, 20, 1, 1, 15], "b": [22, 1], "c": [2, 2, 5]}
        at = {r: 0 for r in seqs}
        live = ["a", "b", "c"]
        rows = {}
        while live:
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
        checked = 0
        for (r, pos), row in rows.items():
            if bool(sure[r][:pos + 1].all()):          # an unsure choice changes every later position
                assert nmse(row, want[r][0][pos]) < 1e-10, (r, pos)
                checked += 1
        assert checked >= 0.6 * len(rows)
        eng.cache.check()
    finally:
        unregister_architecture("ToyRoutedLM")
