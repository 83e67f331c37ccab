// What a model is made of, as the host core sees it: the interfaces of the parts, what a
// part sees of a step, the plan of a model (its parts and the order in which its layers run)
// and the two registries: part kinds by name, architectures by name.
//
// A part is built from sizes and constants only (the JSON object of its kind); it never
// learns which model it is in.  Its life has three stages: construction (tensor_specs
// already works, so checkpoints can be checked and random weights made without a device);
// bind (take the checkpoint tensors it declared, in the form its kernels want); forward
// inside a step.
//
// Adding a part: derive from Norm, PositionEncoding, Mixer, FeedForward, EmbeddingStage,
// Head or Block and call register_part_kind("name", factory).  Adding an architecture: call
// register_architecture("NameForCausalLM", {normalize config, plan from config}); the plan
// names part kinds, so a model may put different mixers and feed-forwards in different
// layers, name a layer twice in its run order, or let a run read another run's cache.
#pragma once
#include <functional>
#include <optional>

#include "kernels.hpp"
#include "weights.hpp"

namespace kipp {

// One entry of the run order.  `layer` indexes the plan's layers (a layer may be named
// twice); runs with the same `cache` id share pages and state; writes_cache false lets a run
// read what another run wrote without adding its own keys and values.
struct LayerRun {
    int layer = 0;
    int cache = 0;
    bool writes_cache = true;
};

// Cache need of a mixer: keys and values of kv_heads heads of head_dim per token.  window 0
// keeps every key; a window of w keeps keys j with pos - w < j <= pos.  Runs with equal
// specs share a group of the cache manager (own pool, own block tables, own retention).
struct PagedKVSpec {
    int kv_heads = 0, head_dim = 0, window = 0;
    bool operator==(const PagedKVSpec& o) const {
        return kv_heads == o.kv_heads && head_dim == o.head_dim && window == o.window;
    }
    bool operator<(const PagedKVSpec& o) const {
        return std::tie(kv_heads, head_dim, window) < std::tie(o.kv_heads, o.head_dim, o.window);
    }
};

// Fixed-size per-request state of a mixer: one tensor per request, zeroed on admission.
struct StateSpec {
    std::vector<int64_t> shape;
    int dtype = F32;
    size_t bytes() const {
        size_t n = dtype_size(dtype);
        for (auto d : shape) n *= (size_t)d;
        return n;
    }
    bool operator==(const StateSpec& o) const { return shape == o.shape && dtype == o.dtype; }
};

struct DeviceInfo {
    int sm_count = 0;
};

// ---------------------------------------------------------------------------------------------
// The shape of a step on the host: what decides sizes and kernel choice.
struct StepShape {
    int entries = 0, tokens = 0, logit_rows = 0;
    std::vector<int> q_lens;          // tokens each entry brings
    std::vector<int> starts;          // tokens each entry has cached before the step
    std::vector<int> slots;
};

// Work lists that a kind of mixer's kernels read beside the common metadata.  The engine packs
// them into the step's one metadata buffer without knowing what they hold: a planner says how
// many int32 sections it needs and how long each is (from the q_lens alone, so that steps of one
// shape keep one layout), fills them on the host, and can bring them up to date on the device
// between the steps of a burst that runs without the host.
class WorkPlanner {
public:
    virtual ~WorkPlanner() = default;
    virtual std::string key() const = 0;                 // mixers with equal keys share one planner
    virtual int sections() const = 0;
    virtual void sizes(const StepShape& shape, int* ints_per_section) const = 0;
    virtual void fill(const StepShape& shape, int* const* host_sections) const = 0;
    // after every entry moved on by one token on the device (a burst of decode steps); `shape`
    // is the step's as the host packed it
    virtual void advance_on_device(Ops& ops, const StepShape& shape, int* const* device_sections,
                                   const int* context_len, int entries) const {}
};

struct StepMeta {
    StepShape shape;
    const int* token_ids = nullptr;       // int32 [T]
    const int* positions = nullptr;       // int32 [T] absolute position of each token
    const int* entry_of_token = nullptr;  // int32 [T]
    const int* q_start = nullptr;         // int32 [entries + 1]
    const int* context_len = nullptr;     // int32 [entries]
    const int* slots = nullptr;           // int32 [entries]
    const int* logit_rows = nullptr;      // int32 [R] token rows whose logits are wanted
    std::vector<const int*> block_tables; // per cache group: int32 [entries, width]
    std::vector<int> table_widths;
    std::map<std::string, std::vector<int*>> work;        // planner key -> device sections
    std::map<std::string, std::vector<int>> work_sizes;   // planner key -> ints per section
};

// What a norm that is a plain RMSNorm tells the parts around it, so that they can fold it
// into their products (see NormFold): y = x * rsqrt(mean(x^2) + eps) * weight.
struct RmsNormSpec {
    const void* weight = nullptr;
    int weight_dtype = F32;
    float eps = 0.f;
    int size = 0;
};

// An input whose rows lack the factor rsqrt(sum(ssq[t, :slots]) * inv_n + eps).
struct RowScale {
    const float* ssq = nullptr;
    int slots = 0;
    float inv_n = 0.f, eps = 0.f;
    bool valid() const { return ssq != nullptr; }
};

class Engine;
class Norm;

// What a part sees during one step.
struct StepContext {
    Engine* engine = nullptr;
    StepMeta* meta = nullptr;
    int dtype = BF16;                      // compute dtype of activations between kernels
    Ops* ops = nullptr;
    Workspace* workspace = nullptr;
    cudaStream_t stream = nullptr;
    bool kv_round_bf16 = false;            // 32-bit cache: keys and values are rounded to bfloat16 when stored
    std::map<std::string, void*> step_cache;   // what parts share within ONE forward pass (rotary tables)

    // Norms in deferred form (set by a block around the calls of its parts; a part that says
    // folds_rms() honours them, any other part never sees them set).  Deferred: the part's input
    // h is bf16(x * norm weight) and the per-row factor rsqrt(mean(x^2) + eps) is applied by the
    // part's first product to its result rows, in float32.  Whether a part takes its input so is
    // a matter of the model, never of the step: the same rounding at every way of cutting.
    RowScale input_scale;                  // the part's input h lacks this per-row factor
    const RmsNormSpec* emit_for = nullptr; // the part's residual add may also leave this norm's deferred form in `normed`
    bool emitted = false;                  //   ... and says so here, with the sums in emitted_scale
    RowScale emitted_scale;
    const Norm* pending_norm = nullptr;    // `normed` holds the deferred form of this norm of the NEXT block
    RowScale pending_scale;
    const Norm* following_norm = nullptr;  // Block::deferred_first_norm of the block that runs next (set by the engine)

    size_t element() const { return dtype_size(dtype); }
    int tokens() const { return meta->shape.tokens; }
    PagedCacheView cache_view(const LayerRun& run, int mixer_slot = 0) const;
    // [max_requests, state bytes] state of this run's cache id; index it with meta->slots.
    void* state_view(const LayerRun& run, int mixer_slot, size_t* bytes_per_slot) const;
    int max_requests() const;
};

// Gives parts their tensors at bind time.
class Binder {
public:
    virtual ~Binder() = default;
    virtual int compute_dtype() const = 0;
    virtual bool has(const std::string& name) = 0;
    virtual int stored_dtype(const std::string& name) = 0;          // DType in the checkpoint
    virtual void* allocate(size_t bytes, const std::string& what) = 0;   // device memory that lives with the engine
    // dst[r * dst_pitch + c] = convert(tensor viewed as [rows, cols]); pitch in elements
    virtual void load(const std::string& name, void* dst, int dst_dtype, int64_t dst_pitch, int64_t rows,
                      int64_t cols) = 0;
    // the whole tensor as [rows, cols] in `dtype`; asked for twice it is the same memory (tied weights)
    virtual void* shared(const std::string& name, int dtype, int64_t rows, int64_t cols) = 0;
    virtual Ops& ops() = 0;
};

// ---------------------------------------------------------------------------------------------
class Part {
public:
    virtual ~Part() = default;
    virtual void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const {}
    virtual void bind(Binder& binder, const std::string& prefix) {}
    virtual size_t weight_bytes() const { return 0; }     // bytes of weights one forward pass reads
    // false: the part's forward cannot be captured in a CUDA graph (it reads the step on the host,
    // allocates, or keeps state that a captured pass would not advance)
    virtual bool graph_safe() const { return true; }
};

class Norm : public Part {
public:
    // out[r, :] (compute dtype) = norm(x[rows ? rows[r] : r, :]); x float32 [T, size]
    virtual void forward(StepContext& ctx, const float* x, void* out, const int* rows, int n_rows) = 0;
    virtual int size() const = 0;
    // a plain RMSNorm says what it is, so that the products around it can fold it
    virtual std::optional<RmsNormSpec> rms_spec() const { return std::nullopt; }
};

class PositionEncoding : public Part {
public:
    // Leading dims of each head that rotate (0: none): pair (i, i + rotary_dim/2) turns by
    // position * inv_freq[i].
    virtual int rotary_dim() const = 0;
    virtual const float* inv_freq_device() const = 0;     // float32 [rotary_dim / 2], after bind
    virtual std::string table_key() const = 0;            // encodings with equal keys share a step's (cos, sin) table
};

class Mixer : public Part {
public:
    virtual std::optional<PagedKVSpec> cache_spec() const { return std::nullopt; }
    virtual std::optional<StateSpec> state_spec() const { return std::nullopt; }
    // the planner of the work lists this mixer's kernels read beside the common metadata, if any
    virtual std::shared_ptr<WorkPlanner> planner(const DeviceInfo& device, bool own_length_splits) { return nullptr; }
    // ADDS its output to the float32 residual [T, hidden]; h [T, hidden] in the compute dtype
    virtual void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) = 0;
    // true: the part applies ctx.input_scale to its first product, at every size of step, and may
    // honour ctx.emit_for in its residual add
    virtual bool folds_rms() const { return false; }
};

class FeedForward : public Part {
public:
    virtual void forward(StepContext& ctx, const void* h, float* residual) = 0;
    virtual bool folds_rms() const { return false; }      // as Mixer::folds_rms
};

// A stage at the bottom of the model: the first one writes the residual stream x [T, hidden]
// from the token ids, later ones may add to it (learned positions, say).
class EmbeddingStage : public Part {
public:
    virtual void forward(StepContext& ctx, float* x) = 0;
};

class Head : public Part {
public:
    virtual void forward(StepContext& ctx, const void* h, int n_rows, float* logits) = 0;
    virtual int vocab_size() const = 0;
};

// The arrangement of norms, mixers and feed-forward in one layer.
class Block : public Part {
public:
    virtual std::vector<Mixer*> mixers() = 0;
    virtual void forward(StepContext& ctx, const LayerRun& run, float* x) = 0;
    // the norm the block applies to the residual stream first, if the part after it takes its
    // input in deferred form (see StepContext::input_scale)
    virtual const Norm* deferred_first_norm() const { return nullptr; }
};

// ---------------------------------------------------------------------------------------------
struct ModelPlan {
    int hidden_size = 0, vocab_size = 0;
    long long max_positions = 0;                                        // 0: no limit of the model's own
    Json config;                                                        // the configuration it was built from
    std::vector<std::pair<std::string, std::unique_ptr<EmbeddingStage>>> embedding;
    std::vector<std::pair<std::string, std::unique_ptr<Block>>> layers;
    std::vector<LayerRun> order;
    std::pair<std::string, std::unique_ptr<Norm>> final_norm;
    std::pair<std::string, std::unique_ptr<Head>> head;

    std::vector<TensorSpec> tensor_specs() const {
        std::vector<TensorSpec> specs;
        for (auto& e : embedding) e.second->tensor_specs(e.first, specs);
        for (auto& l : layers) l.second->tensor_specs(l.first, specs);
        final_norm.second->tensor_specs(final_norm.first, specs);
        head.second->tensor_specs(head.first, specs);
        std::set<std::string> seen;
        for (auto& s : specs)
            if (!seen.insert(s.name).second) fail(KIPP_E_CONFIG, "tensor " + s.name + " is declared twice");
        return specs;
    }
};

// What building a plan can look up: the caller's external parts.
struct BuildContext {
    const kipp_external_part* external = nullptr;
    int n_external = 0;
};

using PartFactory = std::function<std::unique_ptr<Part>(const Json& params, const BuildContext& ctx)>;

struct Architecture {
    // config.json keys after defaults and checks (throws KIPP_E_CONFIG)
    std::function<Json(const Json& config)> normalize;
    // the plan (JSON) of a normalized configuration
    std::function<Json(const Json& normalized)> plan;
};

class Registry {
public:
    static Registry& get() {
        static Registry r;
        return r;
    }
    void add_part_kind(const std::string& kind, PartFactory f) { kinds_[kind] = std::move(f); }
    void add_architecture(const std::string& name, Architecture a) { archs_[name] = std::move(a); }
    const Architecture& architecture(const std::string& name) const {
        auto it = archs_.find(name);
        if (it == archs_.end()) {
            std::string known;
            for (auto& kv : archs_) known += (known.empty() ? "" : ", ") + kv.first;
            fail(KIPP_E_UNSUPPORTED, "unsupported architecture '" + name + "'; registered: [" + known + "]");
        }
        return it->second;
    }
    std::unique_ptr<Part> make(const Json& params, const BuildContext& ctx) const {
        if (!params.is_object() || !params.has("kind")) fail(KIPP_E_CONFIG, "a part of the plan lacks its 'kind'");
        const std::string kind = params.get("kind").as_string();
        auto it = kinds_.find(kind);
        if (it == kinds_.end()) {
            std::string known;
            for (auto& kv : kinds_) known += (known.empty() ? "" : ", ") + kv.first;
            fail(KIPP_E_UNSUPPORTED, "unknown part kind '" + kind + "'; registered: [" + known + "]");
        }
        try {
            return it->second(params, ctx);
        } catch (const JsonError& e) {
            fail(KIPP_E_CONFIG, "part of kind '" + kind + "': " + e.what());
        }
    }
    template <typename T> std::unique_ptr<T> make_as(const Json& params, const BuildContext& ctx, const char* role) const {
        std::unique_ptr<Part> p = make(params, ctx);
        T* t = dynamic_cast<T*>(p.get());
        if (!t)
            fail(KIPP_E_CONFIG, "part of kind '" + params.get("kind").as_string() + "' cannot stand as " + role);
        p.release();
        return std::unique_ptr<T>(t);
    }
    std::vector<std::string> part_kinds() const {
        std::vector<std::string> v;
        for (auto& kv : kinds_) v.push_back(kv.first);
        return v;
    }
    std::vector<std::string> architectures() const {
        std::vector<std::string> v;
        for (auto& kv : archs_) v.push_back(kv.first);
        return v;
    }

private:
    std::map<std::string, PartFactory> kinds_;
    std::map<std::string, Architecture> archs_;
};

void register_builtin_parts();           // parts.hpp
void register_builtin_architectures();   // qwen3.hpp

inline void ensure_registered() {
    static std::once_flag once;
    std::call_once(once, [] {
        register_builtin_parts();
        register_builtin_architectures();
    });
}

inline std::string architecture_of(const Json& config) {
    const Json* archs = config.is_object() ? config.find("architectures") : nullptr;
    if (!archs || !archs->is_array() || archs->size() == 0 || !archs->at(0).is_string())
        fail(KIPP_E_CONFIG, "config.json lacks 'architectures': [name]");
    return archs->at(0).as_string();
}

// Builds the parts a plan (JSON) names.
inline std::unique_ptr<ModelPlan> build_plan(const Json& j, const BuildContext& ctx) {
    ensure_registered();
    auto plan = std::make_unique<ModelPlan>();
    const Registry& reg = Registry::get();
    try {
        plan->hidden_size = (int)j.get("hidden_size").as_int();
        plan->vocab_size = (int)j.get("vocab_size").as_int();
        plan->max_positions = j.get_int("max_positions", 0);
        if (const Json* c = j.find("config")) plan->config = *c;
        for (auto& e : j.get("embedding").items())
            plan->embedding.emplace_back(e.get_string("prefix", ""),
                                         reg.make_as<EmbeddingStage>(e.get("part"), ctx, "an embedding stage"));
        if (plan->embedding.empty()) fail(KIPP_E_CONFIG, "the plan has no embedding stage");
        for (auto& l : j.get("layers").items())
            plan->layers.emplace_back(l.get_string("prefix", ""), reg.make_as<Block>(l.get("part"), ctx, "a block"));
        for (auto& r : j.get("order").items()) {
            LayerRun run;
            run.layer = (int)r.get("layer").as_int();
            run.cache = (int)r.get_int("cache", run.layer);
            run.writes_cache = r.get_bool("writes_cache", true);
            if (run.layer < 0 || run.layer >= (int)plan->layers.size())
                fail(KIPP_E_CONFIG, "the run order names layer " + std::to_string(run.layer) + ", which the plan lacks");
            if (run.cache < 0) fail(KIPP_E_CONFIG, "cache ids must not be negative");
            plan->order.push_back(run);
        }
        const Json& fn = j.get("final_norm");
        plan->final_norm = {fn.get_string("prefix", ""), reg.make_as<Norm>(fn.get("part"), ctx, "a norm")};
        const Json& hd = j.get("head");
        plan->head = {hd.get_string("prefix", ""), reg.make_as<Head>(hd.get("part"), ctx, "an output head")};
    } catch (const JsonError& e) {
        fail(KIPP_E_CONFIG, std::string("the model plan is malformed: ") + e.what());
    }
    if (plan->hidden_size <= 0 || plan->vocab_size <= 0) fail(KIPP_E_CONFIG, "the plan's sizes must be positive");
    return plan;
}

inline Json plan_from_config(const Json& config) {
    ensure_registered();
    const Architecture& arch = Registry::get().architecture(architecture_of(config));
    return arch.plan(arch.normalize(config));
}

}  // namespace kipp
