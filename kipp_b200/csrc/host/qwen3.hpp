// The Qwen3 dense decoder: its configuration read from the keys of its own config.json, and
// its plan as a list of parts.
//
// The reference fixes 8 KV heads, head_dim 128, vocab 151,936 and eps 1e-6 in code
// (src/kipp.h:19-21, src/kipp.c:29) and takes the other sizes from a registry row
// (src/kipp_backend.h:19-34); the converter lists the matching config.json keys
// (tools/convert_to_gguf.py:471-485).  Here every one of them is a key that is read.
//
// Per layer: RMSNorm -> attention (q/k/v projections, per-head q/k RMSNorm, rotary encoding,
// causal grouped-query attention, output projection) -> add -> RMSNorm -> SwiGLU feed-forward
// -> add; then a final RMSNorm and the output head, tied to the embedding or not
// (docs/ARCHITECTURE.md:77-92; tensor names src/kipp.c:947-994; 2 + 11*L (+1) tensors,
// src/kipp.c:1108-1111).
#pragma once
#include "model.hpp"

namespace kipp {
namespace qwen3 {

inline long long need_int(const Json& c, const char* key) {
    const Json* v = c.find(key);
    if (!v) fail(KIPP_E_CONFIG, format("config.json lacks required key '%s'", key));
    if (v->is_null()) fail(KIPP_E_CONFIG, format("config key '%s' must not be null", key));
    if (v->is_bool() || !v->is_number() || (v->kind() == Json::Real && std::floor(v->as_double()) != v->as_double()))
        fail(KIPP_E_CONFIG, format("config key '%s' must be an integer, got %s", key, v->dump().c_str()));
    return v->as_int();
}
inline double need_number(const Json& c, const char* key) {
    const Json* v = c.find(key);
    if (!v) fail(KIPP_E_CONFIG, format("config.json lacks required key '%s'", key));
    if (v->is_bool() || !v->is_number())
        fail(KIPP_E_CONFIG, format("config key '%s' must be a number, got %s", key, v->dump().c_str()));
    return v->as_double();
}
inline bool opt_bool(const Json& c, const char* key, bool fallback) {
    const Json* v = c.find(key);
    if (!v) return fallback;
    if (!v->is_bool()) fail(KIPP_E_CONFIG, format("config key '%s' must be true or false, got %s", key, v->dump().c_str()));
    return v->as_bool();
}
inline std::optional<long long> opt_int(const Json& c, const char* key) {
    const Json* v = c.find(key);
    if (!v || v->is_null()) return std::nullopt;
    return need_int(c, key);
}

// The keys after defaults and checks.  Options the engine lacks are refused here, by name.
inline Json normalize(const Json& c) {
    if (!c.is_object()) fail(KIPP_E_CONFIG, "config.json must hold a JSON object");
    Json out = Json::object();
    Json archs = Json::array();
    archs.push(architecture_of(c));
    out.set("architectures", std::move(archs));
    const char* sizes[] = {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                           "num_attention_heads", "num_key_value_heads", "max_position_embeddings"};
    for (const char* k : sizes) {
        const long long v = need_int(c, k);
        if (v <= 0) fail(KIPP_E_CONFIG, format("config key '%s' must be positive, got %lld", k, v));
        out.set(k, v);
    }
    const long long hidden = out.get("hidden_size").as_int(), heads = out.get("num_attention_heads").as_int();
    const long long kv_heads = out.get("num_key_value_heads").as_int(), layers = out.get("num_hidden_layers").as_int();
    // head_dim may differ from hidden_size / num_attention_heads (the q width is never conflated
    // with the hidden width, src/kipp_backend.h:50-53)
    long long head_dim;
    if (auto hd = opt_int(c, "head_dim")) {
        head_dim = *hd;
    } else {
        if (hidden % heads) fail(KIPP_E_CONFIG, "head_dim is absent and hidden_size is not a multiple of num_attention_heads");
        head_dim = hidden / heads;
    }
    if (head_dim <= 0) fail(KIPP_E_CONFIG, format("config key 'head_dim' must be positive, got %lld", head_dim));
    out.set("head_dim", head_dim);
    if (heads % kv_heads)
        fail(KIPP_E_CONFIG, format("num_attention_heads (%lld) must be a multiple of num_key_value_heads (%lld)", heads,
                                   kv_heads));
    if (head_dim % 2) fail(KIPP_E_CONFIG, format("head_dim (%lld) must be even for rotary pairs", head_dim));
    const double theta = need_number(c, "rope_theta"), eps = need_number(c, "rms_norm_eps");
    if (!(theta > 0)) fail(KIPP_E_CONFIG, "rope_theta must be positive");
    if (!(eps > 0)) fail(KIPP_E_CONFIG, "rms_norm_eps must be positive");
    out.set("rope_theta", theta);
    out.set("rms_norm_eps", eps);
    out.set("tie_word_embeddings", opt_bool(c, "tie_word_embeddings", false));
    const std::string act = c.get_string("hidden_act", "silu");
    if (act != "silu") fail(KIPP_E_CONFIG, "hidden_act '" + act + "' is not supported (only 'silu')");
    out.set("hidden_act", act);
    if (opt_bool(c, "attention_bias", false) || opt_bool(c, "mlp_bias", false))
        fail(KIPP_E_CONFIG, "attention_bias / mlp_bias are not supported (Qwen3 dense has none)");
    out.set("attention_bias", false);
    out.set("mlp_bias", false);
    if (const Json* rs = c.find("rope_scaling"); rs && !rs->is_null()) {
        if (!rs->is_object()) fail(KIPP_E_CONFIG, "rope_scaling must be an object or null");
        std::string kind = rs->get_string("rope_type", rs->get_string("type", "default"));
        if (kind != "default") fail(KIPP_E_CONFIG, "rope_scaling '" + kind + "' is not supported");
    }
    out.set("rope_scaling", nullptr);
    // Window options.  A layer with a window of w sees keys j with pos - w < j <= pos.  The
    // reference runs full attention only (docs/ARCHITECTURE.md:48-57); the keys are honoured
    // because the checkpoint format has them.
    const bool use_window = opt_bool(c, "use_sliding_window", false);
    const auto window = opt_int(c, "sliding_window");
    const auto first_window_layer = opt_int(c, "max_window_layers");
    out.set("use_sliding_window", use_window);
    out.set("sliding_window", window ? Json(*window) : Json(nullptr));
    out.set("max_window_layers", first_window_layer ? Json(*first_window_layer) : Json(nullptr));
    Json windows = Json::array();                       // per layer: the window in keys, 0 = full
    if (const Json* lt = c.find("layer_types"); lt && !lt->is_null()) {
        if (!lt->is_array()) fail(KIPP_E_CONFIG, "config key 'layer_types' must be a list");
        if ((long long)lt->size() != layers) fail(KIPP_E_CONFIG, "layer_types must have one entry per layer");
        bool sliding = false;
        for (auto& k : lt->items()) {
            const std::string kind = k.is_string() ? k.as_string() : k.dump();
            if (kind != "full_attention" && kind != "sliding_attention")
                fail(KIPP_E_CONFIG, "unknown layer type '" + kind + "'");
            sliding = sliding || kind == "sliding_attention";
        }
        if (sliding && (!window || *window <= 0))
            fail(KIPP_E_CONFIG, "layer_types names sliding_attention but sliding_window is unset");
        for (auto& k : lt->items()) windows.push(k.as_string() == "sliding_attention" ? *window : 0LL);
        out.set("layer_types", *lt);
    } else {
        if (use_window && (!window || *window <= 0))
            fail(KIPP_E_CONFIG, "use_sliding_window is true but sliding_window is not a positive integer");
        const long long first = first_window_layer ? *first_window_layer : 0;
        for (long long i = 0; i < layers; ++i) windows.push(use_window && window && i >= first ? *window : 0LL);
        out.set("layer_types", nullptr);
    }
    out.set("layer_windows", std::move(windows));
    out.set("initializer_range", c.get_double("initializer_range", 0.02));
    std::string dtype = c.get_string("torch_dtype", c.get_string("dtype", "bfloat16"));
    out.set("torch_dtype", dtype);
    out.set("model_type", c.get_string("model_type", "qwen3"));
    if (const Json* eos = c.find("eos_token_id"); eos && eos->is_int()) out.set("eos_token_id", eos->as_int());
    else out.set("eos_token_id", nullptr);
    return out;
}

inline Json rmsnorm(long long size, double eps) {
    Json j = Json::object();
    j.set("kind", "rmsnorm");
    j.set("size", size);
    j.set("eps", eps);
    return j;
}

inline Json plan(const Json& c) {
    const long long hidden = c.get("hidden_size").as_int(), vocab = c.get("vocab_size").as_int();
    const long long heads = c.get("num_attention_heads").as_int(), kv_heads = c.get("num_key_value_heads").as_int();
    const long long head_dim = c.get("head_dim").as_int(), inter = c.get("intermediate_size").as_int();
    const long long layers = c.get("num_hidden_layers").as_int();
    const double eps = c.get("rms_norm_eps").as_double(), theta = c.get("rope_theta").as_double();
    const bool tied = c.get("tie_word_embeddings").as_bool();
    const char* embed_prefix = "model.embed_tokens.";

    Json p = Json::object();
    p.set("hidden_size", hidden);
    p.set("vocab_size", vocab);
    p.set("max_positions", c.get("max_position_embeddings").as_int());
    p.set("config", c);
    Json emb = Json::object();
    emb.set("kind", "token_embedding");
    emb.set("vocab_size", vocab);
    emb.set("hidden_size", hidden);
    Json stage = Json::object();
    stage.set("prefix", embed_prefix);
    stage.set("part", std::move(emb));
    Json stages = Json::array();
    stages.push(std::move(stage));
    p.set("embedding", std::move(stages));

    Json blocks = Json::array(), order = Json::array();
    for (long long i = 0; i < layers; ++i) {
        Json rope = Json::object();
        rope.set("kind", "rotary");
        rope.set("head_dim", head_dim);
        rope.set("theta", theta);
        Json attn = Json::object();
        attn.set("kind", "attention");
        attn.set("hidden_size", hidden);
        attn.set("num_heads", heads);
        attn.set("num_kv_heads", kv_heads);
        attn.set("head_dim", head_dim);
        attn.set("position", std::move(rope));
        attn.set("qk_norm_eps", eps);
        attn.set("window", c.get("layer_windows").at((size_t)i).as_int());
        Json ffn = Json::object();
        ffn.set("kind", "swiglu");
        ffn.set("hidden_size", hidden);
        ffn.set("intermediate_size", inter);
        Json names = Json::array();
        for (const char* n : {"input_layernorm.", "self_attn.", "post_attention_layernorm.", "mlp."}) names.push(n);
        Json block = Json::object();
        block.set("kind", "pre_norm_block");
        block.set("names", std::move(names));
        block.set("input_norm", rmsnorm(hidden, eps));
        block.set("mixer", std::move(attn));
        block.set("post_norm", rmsnorm(hidden, eps));
        block.set("ffn", std::move(ffn));
        Json layer = Json::object();
        layer.set("prefix", format("model.layers.%lld.", i));
        layer.set("part", std::move(block));
        blocks.push(std::move(layer));
        Json run = Json::object();
        run.set("layer", i);
        run.set("cache", i);
        run.set("writes_cache", true);
        order.push(std::move(run));
    }
    p.set("layers", std::move(blocks));
    p.set("order", std::move(order));
    Json fn = Json::object();
    fn.set("prefix", "model.norm.");
    fn.set("part", rmsnorm(hidden, eps));
    p.set("final_norm", std::move(fn));
    Json head = Json::object();
    head.set("kind", "output_head");
    head.set("vocab_size", vocab);
    head.set("hidden_size", hidden);
    head.set("tied_to", tied ? Json(std::string(embed_prefix) + "weight") : Json(nullptr));
    Json hd = Json::object();
    hd.set("prefix", "lm_head.");
    hd.set("part", std::move(head));
    p.set("head", std::move(hd));
    return p;
}

}  // namespace qwen3

inline void register_builtin_architectures() {
    Registry::get().add_architecture("Qwen3ForCausalLM", Architecture{qwen3::normalize, qwen3::plan});
}

}  // namespace kipp
