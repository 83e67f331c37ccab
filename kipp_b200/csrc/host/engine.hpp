// The engine: a model bound to a device, its cache, and the step function.
//
// step() takes a batch of (request, its next tokens), portions of prompts beside single
// decoded tokens, cut anywhere; runs exactly those tokens as one batch against the cache that
// earlier steps left; and returns the logits at the wanted places.  It generalises the
// reference's kipp_eval_batch (src/kipp.c:3984-4082): any mixture of items, nothing changes on
// error, lengths advance on success.  The host work of a step is: check, reserve pages, pack
// one buffer of metadata, one host-to-device copy, then the launches of the parts (or the
// replay of a captured graph of them).  (The reference launches 18 kernels per layer and token
// from the host, src/cuda/kipp_cuda.cu:358-462.)
#pragma once
#include <list>

#include "cache_core.h"
#include "parts.hpp"
#include "qwen3.hpp"

namespace kipp {

// Where tensors come from when a model is bound.
struct SourceTensor {
    const void* data = nullptr;
    bool on_device = false;
    int dtype = -1;
    std::vector<int64_t> shape;
    int64_t count() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};
class TensorSource {
public:
    virtual ~TensorSource() = default;
    virtual bool get(const std::string& name, SourceTensor& out) = 0;
    virtual void check(const std::vector<TensorSpec>& specs) = 0;
};
class CheckpointSource : public TensorSource {
public:
    explicit CheckpointSource(const std::string& folder) : ckpt_(folder) {}
    bool get(const std::string& name, SourceTensor& out) override {
        const StoredTensor* t = ckpt_.find(name);
        if (!t) return false;
        out.data = t->data;
        out.on_device = false;
        out.dtype = t->dtype;
        out.shape = t->shape;
        return true;
    }
    void check(const std::vector<TensorSpec>& specs) override { ckpt_.check(specs); }

private:
    Checkpoint ckpt_;
};
class ProviderSource : public TensorSource {
public:
    ProviderSource(kipp_tensor_provider fn, void* user) : fn_(fn), user_(user) {}
    bool get(const std::string& name, SourceTensor& out) override {
        kipp_tensor_view v{};
        if (fn_(user_, name.c_str(), &v) != 0) return false;
        if (v.ndim < 0 || v.ndim > 8) fail(KIPP_E_WEIGHTS, "the tensor provider gave " + name + " a bad rank");
        out.data = v.data;
        out.on_device = v.on_device != 0;
        out.dtype = v.dtype;
        out.shape.assign(v.shape, v.shape + v.ndim);
        return true;
    }
    // A provider makes tensors on demand: what it lacks or gives in a wrong shape shows as each
    // tensor is asked for, all of it listed in one error.
    void check(const std::vector<TensorSpec>& specs) override {
        std::vector<std::string> missing, lines;
        for (auto& s : specs) {
            if (s.optional && !s.alias_of.empty()) continue;
            SourceTensor t;
            if (!get(s.name, t)) {
                if (!s.optional) missing.push_back(s.name);
                continue;
            }
            if (t.shape != s.shape)
                lines.push_back("  wrong shape: " + s.name + " is " + shape_text(t.shape) + ", expected " +
                                shape_text(s.shape));
            if (t.dtype < 0 || t.dtype > U8) lines.push_back("  unsupported dtype: " + s.name);
        }
        if (missing.empty() && lines.empty()) return;
        std::string msg = "the given tensors do not match the model:";
        if (!missing.empty()) {
            msg += "\n  missing tensors (" + std::to_string(missing.size()) + "): ";
            for (size_t i = 0; i < missing.size(); ++i) msg += (i ? ", " : "") + missing[i];
        }
        for (auto& l : lines) msg += "\n" + l;
        fail(KIPP_E_WEIGHTS, msg);
    }

private:
    kipp_tensor_provider fn_;
    void* user_;
};

// ---------------------------------------------------------------------------------------------
// One step's metadata buffers: pinned host memory, its device copy, and the event that says
// the copy has read the host side (the host buffer is rewritten only after that).
struct MetaBuffers {
    PinnedBuffer host;
    DeviceBuffer device;
    cudaEvent_t copied = nullptr;
    bool pending = false;
    size_t ints = 0;
    ~MetaBuffers() {
        if (copied) cudaEventDestroy(copied);
    }
    void ensure(size_t n) {
        if (n <= ints) return;
        wait();
        size_t grown = std::max(n, ints * 2);
        grown = std::max<size_t>(grown, 1024);
        host.ensure(grown * sizeof(int));
        device.reset(grown * sizeof(int), "step metadata");
        ints = grown;
    }
    void wait() {
        if (pending) {
            cuda_check(cudaEventSynchronize(copied), "wait for the metadata copy");
            pending = false;
        }
    }
    void send(size_t n, cudaStream_t stream) {
        if (!copied) cuda_check(cudaEventCreateWithFlags(&copied, cudaEventDisableTiming), "event");
        cuda_check(cudaMemcpyAsync(device.get(), host.as<int>(), n * sizeof(int), cudaMemcpyHostToDevice, stream),
                   "copy of the step metadata");
        cuda_check(cudaEventRecord(copied, stream), "event record");
        pending = true;
    }
};

struct StepEntryView {
    int64_t request;
    const int32_t* tokens;
    int n_tokens;
    const int32_t* want;
    int n_want;
};

class Engine {
public:
    // steps a feedback graph runs before its ring of tokens is read out (KIPP_B200_BURST_RING_ROWS
    // in the environment of the process makes it shorter: tests do)
    int burst_ring_rows = 1024;
    static constexpr int MAX_GRAPHS = 24;

    Engine(std::unique_ptr<ModelPlan> plan, TensorSource& source, const kipp_engine_options& options);
    ~Engine();
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    // -- requests ------------------------------------------------------------------------------
    int add_request(int64_t rid);
    void finish(int64_t rid);
    void truncate(int64_t rid, int new_length);
    bool is_live(int64_t rid) const { return live_.count(rid) != 0; }
    int length(int64_t rid) const { return is_live(rid) ? kipp_cm_length(cm_, rid) : -1; }

    // -- the step --------------------------------------------------------------------------------
    const float* step(const StepEntryView* entries, int n, int* n_rows);
    void read_logits(float* out, size_t capacity);
    void synchronize();
    void decode_burst(const int64_t* requests, const int32_t* tokens, int n, int steps, int32_t* out_host);
    // kernel name -> milliseconds between profile(true) and profile(false), as JSON
    void profile(bool on) {
        if (on) { ops_.profile_start(); return; }
        Json j = Json::object();
        for (auto& kv : ops_.profile_stop()) j.set(kv.first, kv.second);
        profile_json_ = j.dump();
    }
    const std::string& profile_json() const { return profile_json_; }
    void sample(const kipp_sample_params* params, uint64_t* rng_states, int n_rows, int32_t* out_host);

    // one part of one layer alone, for tests of the parts (see api.cpp)
    void debug_part(const StepEntryView* entries, int n, int run_index, const std::string& which, const void* input,
                    float* residual, void* output);

    // -- accounting --------------------------------------------------------------------------------
    std::string info_json();
    size_t weight_bytes() const;
    size_t cache_bytes_per_token() const;
    void check_status();
    void debug_set_status(int word, int value) {
        if (word < 0 || word > 3) fail(KIPP_E_ARGUMENT, "there are four status words");
        cuda_check(cudaMemcpyAsync(status_.as<int>() + word, &value, sizeof(int), cudaMemcpyHostToDevice, stream_),
                   "status write");
        cuda_check(cudaStreamSynchronize(stream_), "synchronize");
    }

    // -- what parts and the scheduler reach ---------------------------------------------------------
    PagedCacheView cache_view(const StepMeta& meta, const LayerRun& run, int mixer_slot) const;
    void* state_view(const LayerRun& run, int mixer_slot, size_t* bytes_per_slot) const;
    int max_requests() const { return opt_.max_requests; }
    const kipp_engine_options& options() const { return opt_; }
    const ModelPlan& plan() const { return *plan_; }
    void* cache_manager() const { return cm_; }
    int groups() const { return (int)groups_.size(); }
    int group_pages(int g) const { return groups_[(size_t)g].n_pages; }
    int group_window(int g) const { return groups_[(size_t)g].spec.window; }
    int group_free_pages(int g) const { return kipp_pool_free_pages(kipp_cm_pool(cm_, g)); }
    int free_slots() const { return kipp_slots_free_count(kipp_cm_slots(cm_)); }
    cudaStream_t stream() const { return stream_; }
    long long max_positions() const { return plan_->max_positions; }
    const float* last_logits() const { return last_logits_; }
    int last_rows() const { return last_rows_; }

    std::string last_error;
    // counters (info_json reports them)
    long long steps_run = 0, graph_replays = 0, graph_kernel_launches = 0, graphs_captured = 0;
    long long last_h2d_bytes = 0, last_forward_launches = 0;

private:
    struct CacheGroup {
        PagedKVSpec spec;
        std::vector<long long> cache_keys;    // (cache id, mixer slot) of the runs that share these pools, in storage order
        int n_pages = 0;
        DeviceBuffer k, v;                    // [caches, pages, kv_heads, page_size, head_dim]
        size_t cache_stride = 0;              // bytes between two caches of the group
    };
    struct StateBuffer {
        StateSpec spec;
        DeviceBuffer data;                    // [max_requests, bytes]
    };
    struct StepGraph {
        std::string key;
        MetaBuffers meta_buffers;
        StepMeta meta;
        size_t ints = 0;
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        const float* logits = nullptr;
        int rows = 0;
        long long generation = -1;
        long long launches = 0;
        bool feedback = false;
        DeviceBuffer next_tokens, ring, counter;
        ~StepGraph() {
            if (exec) cudaGraphExecDestroy(exec);
            if (graph) cudaGraphDestroy(graph);
        }
    };
    class EngineBinder;

    static long long cache_key(int cache, int mixer_slot) { return (long long)cache * 16 + mixer_slot; }

    void check_memory(const std::vector<TensorSpec>& specs);
    size_t workspace_estimate() const;
    void build_cache();
    void validate(const StepEntryView* entries, int n, StepShape& shape, std::vector<int>& rows);
    std::vector<int> table_widths(const std::vector<int64_t>& rids, int bucket) const;
    size_t layout(const StepShape& shape, const std::vector<int>& widths, std::vector<size_t>& offsets) const;
    void pack(const StepEntryView* entries, const StepShape& shape, const std::vector<int>& rows,
              const std::vector<int64_t>& rids, const std::vector<int>& widths, MetaBuffers& mb, StepMeta& meta);
    const float* forward(StepMeta& meta);
    const float* run_graph(StepGraph& g, const StepEntryView* entries, const StepShape& shape,
                           const std::vector<int>& rows, const std::vector<int64_t>& rids,
                           const std::vector<int>& widths);
    StepGraph& graph_for(const std::string& key, bool feedback, int batch);
    void feedback_tail(StepGraph& g);
    bool shape_repeats(const StepShape& shape, const std::vector<int>& rows_per_entry);
    bool graphable() const { return opt_.cuda_graphs && graph_safe_ && !ops_.profiling; }

    std::string profile_json_ = "{}";
    kipp_engine_options opt_;
    int dtype_;
    DeviceInfo device_;
    cudaStream_t stream_ = nullptr;
    std::unique_ptr<ModelPlan> plan_;
    Ops ops_;
    Workspace workspace_;
    DeviceBuffer status_;
    std::vector<DeviceBuffer> weight_memory_;
    std::map<std::string, void*> shared_tensors_;
    size_t weight_bytes_allocated_ = 0;
    bool graph_safe_ = true;

    void* cm_ = nullptr;
    std::vector<CacheGroup> groups_;
    std::map<long long, std::pair<int, int>> group_of_cache_;    // cache key -> (group, index in group)
    std::map<long long, StateBuffer> states_;
    std::vector<std::shared_ptr<WorkPlanner>> planners_;
    std::set<int64_t> live_;

    MetaBuffers staging_[4];
    int staging_next_ = 0;
    std::list<std::unique_ptr<StepGraph>> graphs_;               // most recently used last
    std::map<std::string, int> shapes_seen_;

    const float* last_logits_ = nullptr;
    int last_rows_ = 0;
    std::string info_;
    PinnedBuffer sample_host_;
    friend struct StepContext;
};

// ---------------------------------------------------------------------------------------------
inline PagedCacheView StepContext::cache_view(const LayerRun& run, int mixer_slot) const {
    return engine->cache_view(*meta, run, mixer_slot);
}
inline void* StepContext::state_view(const LayerRun& run, int mixer_slot, size_t* bytes_per_slot) const {
    return engine->state_view(run, mixer_slot, bytes_per_slot);
}
inline int StepContext::max_requests() const { return engine->max_requests(); }

inline void AttentionMixer::forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h,
                                    float* residual) {
    const int T = ctx.tokens();
    const size_t es = ctx.element();
    Ops& ops = *ctx.ops;
    const StepMeta& m = *ctx.meta;
    const int qkv_cols = q_dim_ + 2 * kv_dim_;
    NormFold fold_in, fold_out;
    const PagedCacheView cache = ctx.cache_view(run, mixer_slot);       // pages of this run's cache id
    const int rot = position_->rotary_dim();
    const bool to_heads = ctx.dtype == dtype_ && !ctx.kv_round_bf16 &&
                          Ops::projection_to_heads_ok(dtype_, h, hidden_, w_qkv_, hidden_, T, head_dim_, rot);
    const float* cos_sin = nullptr;
    if (rot > 0) {
        // the step's (cos, sin) table: the same for every layer that rotates alike; laid out by
        // pair for the projection that rotates its own heads
        const std::string key = (to_heads ? "rope by pair/" : "rope/") + position_->table_key();
        auto it = ctx.step_cache.find(key);
        if (it == ctx.step_cache.end()) {
            int made = 0;
            for (auto& kv : ctx.step_cache) made += kv.first.rfind("rope", 0) == 0;
            float* table = ctx.workspace->get<float>("rope_table_" + std::to_string(made), (size_t)T * rot);
            if (to_heads) ops.rope_table_by_pair(table, m.positions, position_->inv_freq_device(), T, rot / 2);
            else ops.rope_table(table, m.positions, position_->inv_freq_device(), T, rot / 2);
            it = ctx.step_cache.emplace(key, table).first;
        }
        cos_sin = static_cast<const float*>(it->second);
    }
    void* attn = ctx.workspace->buffer("attn_out", (size_t)T * q_dim_ * es);
    const AttentionWork work = planner_->work_of(m);
    const void* qn = qk_norm_ ? q_norm_ : nullptr;
    const void* kn = qk_norm_ ? k_norm_ : nullptr;
    if (to_heads) {
        // a prompt-sized step: the projection's epilogue norms, rotates and writes the cache
        void* q = ctx.workspace->buffer("q", (size_t)T * q_dim_ * es);
        ops.projection_to_heads(h, hidden_, w_qkv_, hidden_, T, qkv_cols, hidden_, fold_input(ctx, fold_in), cache, q,
                                qn, kn, norm_dtype_, eps_, cos_sin, m.positions, m.entry_of_token, heads_, kv_heads_,
                                run.writes_cache);
        ops.attention(attn, q, cache, ctx.dtype, work, m.positions, m.entry_of_token, m.q_start, m.context_len,
                      heads_, kv_heads_, head_dim_, scale_, window_);
    } else {
        void* qkv = ctx.workspace->buffer("qkv", (size_t)T * qkv_cols * es);
        ops.gemm(qkv, ctx.dtype, qkv_cols, h, hidden_, w_qkv_, hidden_, dtype_, T, qkv_cols, hidden_, EPI_STORE,
                 fold_input(ctx, fold_in));
        if (Ops::attention_decode_fused_ok(work, ctx.dtype, heads_, kv_heads_, head_dim_, rot)) {
            // decoded tokens only: norm, rotation and the cache write happen inside the attention
            // kernel, straight from the projection's output
            ops.attention_decode_fused(attn, qkv, qkv_cols, cache, qn, kn, norm_dtype_, eps_, cos_sin,
                                       run.writes_cache, work, m.q_start, m.context_len, heads_, kv_heads_, head_dim_,
                                       scale_, window_);
        } else {
            void* q = ctx.workspace->buffer("q", (size_t)T * q_dim_ * es);
            const int write = (run.writes_cache ? 1 : 0) | (ctx.kv_round_bf16 && ctx.dtype == F32 ? 2 : 0);
            ops.qk_norm_rope_write(qkv, qkv_cols, q, cache, ctx.dtype, qn, kn, norm_dtype_, eps_, cos_sin, rot,
                                   m.positions, m.entry_of_token, T, heads_, kv_heads_, head_dim_, write);
            ops.attention(attn, q, cache, ctx.dtype, work, m.positions, m.entry_of_token, m.q_start, m.context_len,
                          heads_, kv_heads_, head_dim_, scale_, window_);
        }
    }
    const NormFold* emit = fold_emit(ctx, fold_out, hidden_);
    ops.gemm(residual, F32, hidden_, attn, q_dim_, w_o_, q_dim_, dtype_, T, hidden_, q_dim_, EPI_ADD, emit);
    fold_emitted(ctx, emit, hidden_);
}

// ---------------------------------------------------------------------------------------------
class Engine::EngineBinder : public Binder {
public:
    EngineBinder(Engine& e, TensorSource& s) : e_(e), source_(s) {}
    int compute_dtype() const override { return e_.dtype_; }
    bool has(const std::string& name) override {
        SourceTensor t;
        return source_.get(name, t);
    }
    int stored_dtype(const std::string& name) override { return fetch(name).dtype; }
    void* allocate(size_t bytes, const std::string& what) override {
        e_.weight_memory_.emplace_back(bytes, what.c_str());
        e_.weight_bytes_allocated_ += bytes;
        return e_.weight_memory_.back().get();
    }
    void load(const std::string& name, void* dst, int dst_dtype, int64_t dst_pitch, int64_t rows,
              int64_t cols) override {
        SourceTensor t = fetch(name);
        if (t.count() != rows * cols)
            fail(KIPP_E_WEIGHTS, format("tensor %s holds %lld elements, %lld x %lld were expected", name.c_str(),
                                        (long long)t.count(), (long long)rows, (long long)cols));
        const size_t es = dtype_size(t.dtype);
        if (t.on_device) {
            e_.ops_.convert_rows(dst, dst_dtype, dst_pitch, t.data, t.dtype, cols, rows, cols);
            // the provider may free or reuse the tensor's memory after its next call
            cuda_check(cudaStreamSynchronize(e_.stream_), "weight conversion");
            return;
        }
        // host memory (a mapped file): in pieces through a staging buffer on the device
        const int64_t chunk_rows = std::max<int64_t>(1, (int64_t)((256u << 20) / std::max<size_t>(1, (size_t)cols * es)));
        for (int64_t r0 = 0; r0 < rows; r0 += chunk_rows) {
            const int64_t n = std::min(chunk_rows, rows - r0);
            const size_t bytes = (size_t)n * cols * es;
            if (staging_.bytes() < bytes) {
                cuda_check(cudaStreamSynchronize(e_.stream_), "weight upload");
                staging_.reset(bytes, "weight staging");
            }
            const char* src = static_cast<const char*>(t.data) + (size_t)r0 * cols * es;
            cuda_check(cudaMemcpyAsync(staging_.get(), src, bytes, cudaMemcpyHostToDevice, e_.stream_), "weight upload");
            char* out = static_cast<char*>(dst) + (size_t)r0 * dst_pitch * dtype_size(dst_dtype);
            e_.ops_.convert_rows(out, dst_dtype, dst_pitch, staging_.get(), t.dtype, cols, n, cols);
        }
    }
    void* shared(const std::string& name, int dtype, int64_t rows, int64_t cols) override {
        const std::string key = name + "/" + dtype_name(dtype);
        auto it = e_.shared_tensors_.find(key);
        if (it != e_.shared_tensors_.end()) return it->second;
        void* p = allocate((size_t)rows * cols * dtype_size(dtype), name);
        load(name, p, dtype, cols, rows, cols);
        e_.shared_tensors_[key] = p;
        return p;
    }
    Ops& ops() override { return e_.ops_; }
    void finish() { cuda_check(cudaStreamSynchronize(e_.stream_), "weight upload"); }

private:
    Engine& e_;
    TensorSource& source_;
    DeviceBuffer staging_;
    SourceTensor fetch(const std::string& name) {
        SourceTensor t;
        if (!source_.get(name, t)) fail(KIPP_E_WEIGHTS, "tensor " + name + " is missing");
        if (t.dtype < 0 || t.dtype > U8) fail(KIPP_E_WEIGHTS, "tensor " + name + " has an unsupported element type");
        return t;
    }
};

inline Engine::Engine(std::unique_ptr<ModelPlan> plan, TensorSource& source, const kipp_engine_options& options)
    : opt_(options), dtype_(options.dtype), plan_(std::move(plan)) {
    if (dtype_ != BF16 && dtype_ != F32) fail(KIPP_E_ARGUMENT, "the compute dtype must be bfloat16 or float32");
    if (opt_.page_size <= 0) fail(KIPP_E_ARGUMENT, "page_size must be positive");
    if (opt_.max_requests <= 0) fail(KIPP_E_ARGUMENT, "max_requests must be positive");
    if (opt_.max_batch_tokens <= 0) fail(KIPP_E_ARGUMENT, "max_batch_tokens must be positive");
    if (opt_.cache_tokens < 0) fail(KIPP_E_ARGUMENT, "cache_tokens must not be negative");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        fail(KIPP_E_CUDA, "no CUDA device is available; kipp_b200 has no CPU fallback");
    }
    if (opt_.device < 0 || opt_.device >= count) fail(KIPP_E_ARGUMENT, format("there is no CUDA device %d", opt_.device));
    cuda_check(cudaSetDevice(opt_.device), "cudaSetDevice");
    cudaDeviceProp prop;
    cuda_check(cudaGetDeviceProperties(&prop, opt_.device), "device properties");
    device_.sm_count = prop.multiProcessorCount;
    cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "stream");
    // Kernels record refused accesses here instead of faulting: word 0 = 1 token id out of range,
    // 2 write to an unmapped page, 3 read of an unmapped page; words 1 and 2: a bounded wait of a
    // tensor-core kernel ran out.
    status_.reset(4 * sizeof(int), "status words");
    cuda_check(cudaMemset(status_.get(), 0, 4 * sizeof(int)), "status words");
    ops_.stream = stream_;
    ops_.status = status_.as<int>();
    ops_.workspace = &workspace_;

    if (const char* rows = getenv("KIPP_B200_BURST_RING_ROWS"); rows && atoi(rows) > 0) burst_ring_rows = atoi(rows);
    if (opt_.max_logit_rows <= 0) {
        // a default that keeps the logits buffer near half a GiB
        const long long by_bytes = (512ll << 20) / ((long long)plan_->vocab_size * 4);
        opt_.max_logit_rows = (int)std::min<long long>(opt_.max_batch_tokens, std::max<long long>(64, by_bytes));
    }
    const std::vector<TensorSpec> specs = plan_->tensor_specs();
    source.check(specs);
    for (auto& l : plan_->layers) graph_safe_ = graph_safe_ && l.second->graph_safe();
    for (auto& e : plan_->embedding) graph_safe_ = graph_safe_ && e.second->graph_safe();
    graph_safe_ = graph_safe_ && plan_->final_norm.second->graph_safe() && plan_->head.second->graph_safe();
    check_memory(specs);
    {
        EngineBinder binder(*this, source);
        for (auto& e : plan_->embedding) e.second->bind(binder, e.first);
        for (auto& l : plan_->layers) l.second->bind(binder, l.first);
        plan_->final_norm.second->bind(binder, plan_->final_norm.first);
        plan_->head.second->bind(binder, plan_->head.first);
        binder.finish();
    }
    build_cache();
}

inline Engine::~Engine() {
    if (stream_) cudaStreamSynchronize(stream_);
    graphs_.clear();
    if (cm_) kipp_cm_destroy(cm_);
    if (stream_) cudaStreamDestroy(stream_);
}

inline size_t Engine::workspace_estimate() const {
    // per token: the float32 residual, the normed copy, q/k/v, q, the attention output, the
    // feed-forward's activation (sizes are not known here per part: four hidden-wide rows of
    // slack stand for them), and the logits rows
    const size_t es = dtype_size(dtype_);
    const size_t per_token = (size_t)plan_->hidden_size * (4 + es * 12);
    return per_token * (size_t)opt_.max_batch_tokens + (size_t)opt_.max_logit_rows * plan_->vocab_size * 4 + (64u << 20);
}

// Refuse before anything is uploaded when weights, cache and workspace cannot fit (the
// reference does the same before its one allocation, src/cuda/kipp_cuda.cu:542-561).
inline void Engine::check_memory(const std::vector<TensorSpec>& specs) {
    const size_t es = dtype_size(dtype_);
    size_t weights = 0;
    for (auto& s : specs) {
        if (s.optional && !s.alias_of.empty()) continue;
        size_t n = es;
        for (auto d : s.shape) n *= (size_t)d;
        weights += n;
    }
    size_t per_token = 0;
    std::set<long long> seen;
    for (auto& run : plan_->order) {
        auto mixers = plan_->layers[(size_t)run.layer].second->mixers();
        for (size_t s = 0; s < mixers.size(); ++s)
            if (auto cs = mixers[s]->cache_spec(); cs && seen.insert(cache_key(run.cache, (int)s)).second)
                per_token += (size_t)2 * cs->kv_heads * cs->head_dim * es;
    }
    size_t free_bytes = 0, total = 0;
    cuda_check(cudaMemGetInfo(&free_bytes, &total), "cudaMemGetInfo");
    const size_t workspace = workspace_estimate();
    if (opt_.cache_tokens == 0) {
        // the cache takes what is left: nine tenths of the free memory after weights and
        // workspace, at most what max_requests requests of the model's longest context need
        const size_t fixed = weights + workspace;
        if (fixed >= free_bytes)
            fail(KIPP_E_MEMORY, format("the model needs about %zu device bytes (%zu of weights, %zu of workspace) but "
                                       "only %zu are free on device %d",
                                       fixed, weights, workspace, free_bytes, opt_.device));
        long long tokens = per_token ? (long long)((free_bytes - fixed) / 10 * 9 / per_token) : opt_.page_size;
        const long long ctx = plan_->max_positions > 0 ? plan_->max_positions : 8192;
        tokens = std::min(tokens, ctx * (long long)opt_.max_requests);
        tokens = tokens / opt_.page_size * opt_.page_size;
        if (tokens < opt_.page_size)
            fail(KIPP_E_MEMORY, format("no device memory is left for the cache after %zu bytes of weights and %zu of "
                                       "workspace (%zu free)", weights, workspace, free_bytes));
        opt_.cache_tokens = tokens;
    }
    const size_t pages = (size_t)std::max<long long>(1, (opt_.cache_tokens + opt_.page_size - 1) / opt_.page_size);
    const size_t cache = pages * opt_.page_size * per_token;
    const size_t need = weights + cache + workspace;
    if (need > free_bytes)
        fail(KIPP_E_MEMORY, format("the model needs about %zu device bytes (%zu of weights, %zu of cache for %lld "
                                   "tokens, %zu of workspace) but only %zu are free on device %d",
                                   need, weights, cache, opt_.cache_tokens, workspace, free_bytes, opt_.device));
}

inline void Engine::build_cache() {
    // runs whose mixers declared equal cache specs share a group: own pool, tables, retention
    std::map<long long, PagedKVSpec> cache_specs;
    std::map<long long, StateSpec> state_specs;
    std::map<std::string, std::shared_ptr<WorkPlanner>> planners;
    for (auto& run : plan_->order) {
        auto mixers = plan_->layers[(size_t)run.layer].second->mixers();
        for (size_t s = 0; s < mixers.size(); ++s) {
            const long long key = cache_key(run.cache, (int)s);
            if (auto cs = mixers[s]->cache_spec()) {
                auto it = cache_specs.emplace(key, *cs).first;
                if (!(it->second == *cs))
                    fail(KIPP_E_CONFIG, format("runs that share cache %d need equal cache specs", run.cache));
            }
            if (auto ss = mixers[s]->state_spec()) {
                auto it = state_specs.emplace(key, *ss).first;
                if (!(it->second == *ss))
                    fail(KIPP_E_CONFIG, format("runs that share cache %d need equal state specs", run.cache));
            }
            if (auto p = mixers[s]->planner(device_, opt_.own_length_splits != 0)) planners.emplace(p->key(), p);
        }
    }
    for (auto& kv : planners) planners_.push_back(kv.second);
    std::map<PagedKVSpec, std::vector<long long>> by_spec;
    std::vector<PagedKVSpec> spec_order;
    for (auto& kv : cache_specs) {
        if (!by_spec.count(kv.second)) spec_order.push_back(kv.second);
        by_spec[kv.second].push_back(kv.first);
    }
    const int n_pages = (int)std::max<long long>(1, (opt_.cache_tokens + opt_.page_size - 1) / opt_.page_size);
    const size_t es = dtype_size(dtype_);
    std::vector<int> pages, windows;
    for (auto& spec : spec_order) {
        groups_.emplace_back();
        CacheGroup& g = groups_.back();
        g.spec = spec;
        g.cache_keys = by_spec[spec];
        g.n_pages = n_pages;
        g.cache_stride = (size_t)n_pages * spec.kv_heads * opt_.page_size * spec.head_dim * es;
        const size_t bytes = g.cache_stride * g.cache_keys.size();
        g.k.reset(bytes, "key pages");
        g.v.reset(bytes, "value pages");
        cuda_check(cudaMemsetAsync(g.k.get(), 0, bytes, stream_), "clearing the key pages");
        cuda_check(cudaMemsetAsync(g.v.get(), 0, bytes, stream_), "clearing the value pages");
        for (size_t j = 0; j < g.cache_keys.size(); ++j)
            group_of_cache_[g.cache_keys[j]] = {(int)groups_.size() - 1, (int)j};
        pages.push_back(n_pages);
        windows.push_back(spec.window > 0 ? spec.window : -1);
    }
    int dummy = 1;
    cm_ = kipp_cm_create((int)groups_.size(), pages.empty() ? &dummy : pages.data(),
                         windows.empty() ? &dummy : windows.data(), opt_.page_size, opt_.max_requests);
    if (!cm_) fail(KIPP_E_ARGUMENT, "the cache manager could not be created");
    for (auto& kv : state_specs) {
        StateBuffer& sb = states_[kv.first];
        sb.spec = kv.second;
        const size_t bytes = sb.spec.bytes() * (size_t)opt_.max_requests;
        sb.data.reset(bytes, "per-request state");
        cuda_check(cudaMemsetAsync(sb.data.get(), 0, bytes, stream_), "clearing per-request state");
    }
    cuda_check(cudaStreamSynchronize(stream_), "cache set-up");
}

inline PagedCacheView Engine::cache_view(const StepMeta& meta, const LayerRun& run, int mixer_slot) const {
    auto it = group_of_cache_.find(cache_key(run.cache, mixer_slot));
    if (it == group_of_cache_.end()) fail(KIPP_E_STATE, format("cache %d has no pages", run.cache));
    const CacheGroup& g = groups_[(size_t)it->second.first];
    PagedCacheView v;
    v.k_pages = static_cast<char*>(g.k.get()) + g.cache_stride * (size_t)it->second.second;
    v.v_pages = static_cast<char*>(g.v.get()) + g.cache_stride * (size_t)it->second.second;
    v.n_pages = g.n_pages;
    v.block_table = meta.block_tables[(size_t)it->second.first];
    v.table_width = meta.table_widths[(size_t)it->second.first];
    v.page_size = opt_.page_size;
    return v;
}

inline void* Engine::state_view(const LayerRun& run, int mixer_slot, size_t* bytes_per_slot) const {
    auto it = states_.find(cache_key(run.cache, mixer_slot));
    if (it == states_.end()) fail(KIPP_E_STATE, format("cache %d has no per-request state", run.cache));
    if (bytes_per_slot) *bytes_per_slot = it->second.spec.bytes();
    return it->second.data.get();
}

// ---------------------------------------------------------------------------------------------
inline int Engine::add_request(int64_t rid) {
    const int slot = kipp_cm_admit(cm_, rid);
    if (slot == KIPP_CM_OUT_OF_SLOTS)
        fail(KIPP_E_OUT_OF_SLOTS, format("all %d request slots are in use", opt_.max_requests));
    if (slot == KIPP_CM_ARGUMENT) fail(KIPP_E_STATE, format("request %lld is already live", (long long)rid));
    if (slot < 0) fail(KIPP_E_STATE, format("admit: error %d", slot));
    live_.insert(rid);
    for (auto& kv : states_) {
        const size_t bytes = kv.second.spec.bytes();
        cuda_check(cudaMemsetAsync(kv.second.data.as<char>() + bytes * (size_t)slot, 0, bytes, stream_),
                   "clearing a request's state");
    }
    return slot;
}

// The request is over: its pages and its slot are given back.
inline void Engine::finish(int64_t rid) {
    if (!is_live(rid)) fail(KIPP_E_STATE, format("request %lld is not live", (long long)rid));
    const int rc = kipp_cm_release(cm_, rid);
    live_.erase(rid);
    if (rc) fail(KIPP_E_STATE, format("release of request %lld: error %d", (long long)rid, rc));
}

// Cut a live request back to its first new_length tokens; the pages beyond go back.  A model
// whose mixers keep state per request can only be cut back to nothing (the state is then
// cleared): a state cannot be unwound.
inline void Engine::truncate(int64_t rid, int new_length) {
    if (!is_live(rid)) fail(KIPP_E_STATE, format("request %lld is not live", (long long)rid));
    if (!states_.empty() && new_length != 0)
        fail(KIPP_E_ARGUMENT, "a model with per-request state can only be reset (truncate to 0)");
    int group = -1;
    const int rc = kipp_cm_truncate(cm_, rid, new_length, &group);
    if (rc == KIPP_CM_ARGUMENT)
        fail(KIPP_E_ARGUMENT, format("truncate to %d is outside 0..%d", new_length, kipp_cm_length(cm_, rid)));
    if (rc == KIPP_CM_WINDOW_REFUSES)
        fail(KIPP_E_ARGUMENT, format("request %lld cannot be cut back to %d: the window of cache group %d has already "
                                     "given back pages it would need", (long long)rid, new_length, group));
    if (rc) fail(KIPP_E_STATE, format("truncate: error %d", rc));
    if (new_length == 0) {
        const int slot = kipp_cm_slot(cm_, rid);
        for (auto& kv : states_) {
            const size_t bytes = kv.second.spec.bytes();
            cuda_check(cudaMemsetAsync(kv.second.data.as<char>() + bytes * (size_t)slot, 0, bytes, stream_),
                       "clearing a request's state");
        }
    }
}

// ---------------------------------------------------------------------------------------------
inline void Engine::validate(const StepEntryView* entries, int n, StepShape& shape, std::vector<int>& rows) {
    if (n <= 0) fail(KIPP_E_ARGUMENT, "a step needs at least one entry");
    std::set<int64_t> seen;
    long long total = 0;
    shape.entries = n;
    shape.q_lens.resize((size_t)n);
    for (int i = 0; i < n; ++i) {
        const StepEntryView& e = entries[i];
        if (!seen.insert(e.request).second)
            fail(KIPP_E_ARGUMENT, format("request %lld appears twice in one step", (long long)e.request));
        if (e.n_tokens <= 0 || !e.tokens) fail(KIPP_E_ARGUMENT, format("request %lld brings no tokens", (long long)e.request));
        for (int t = 0; t < e.n_tokens; ++t)
            if (e.tokens[t] < 0 || e.tokens[t] >= plan_->vocab_size)
                fail(KIPP_E_ARGUMENT, format("request %lld has a token id outside [0, %d)", (long long)e.request,
                                             plan_->vocab_size));
        for (int w = 0; w < e.n_want; ++w) {
            if (e.want[w] < 0 || e.want[w] >= e.n_tokens)
                fail(KIPP_E_ARGUMENT, format("want index %d is outside the entry's %d tokens", e.want[w], e.n_tokens));
            rows.push_back((int)total + e.want[w]);
        }
        shape.q_lens[(size_t)i] = e.n_tokens;
        total += e.n_tokens;
    }
    if (total > opt_.max_batch_tokens)
        fail(KIPP_E_ARGUMENT, format("step of %lld tokens exceeds max_batch_tokens %d", total, opt_.max_batch_tokens));
    if ((int)rows.size() > opt_.max_logit_rows)
        fail(KIPP_E_ARGUMENT, format("step wants %zu rows of logits, max_logit_rows is %d (an engine option: the logits "
                                     "buffer is rows x vocabulary x 4 bytes)", rows.size(), opt_.max_logit_rows));
    shape.tokens = (int)total;
    shape.logit_rows = (int)rows.size();
}

// Block-table width per cache group: what the longest entry needs; for a captured step rounded
// up to `bucket` pages so that one graph serves many steps and little is copied for short contexts.
inline std::vector<int> Engine::table_widths(const std::vector<int64_t>& rids, int bucket) const {
    std::vector<int> widths;
    for (int g = 0; g < (int)groups_.size(); ++g) {
        int need = 1;
        for (int64_t r : rids) need = std::max(need, kipp_cm_table_len(cm_, r, g));
        if (bucket > 0) {
            int cap = groups_[(size_t)g].n_pages;
            if (plan_->max_positions > 0)
                cap = std::min<long long>(cap, (plan_->max_positions + opt_.page_size - 1) / opt_.page_size);
            const int rounded = (need + bucket) / bucket * bucket;
            need = std::max(1, std::min(std::max(cap, need), rounded));
        }
        widths.push_back(need);
    }
    return widths;
}

// Offsets (in ints) of the sections of the packed buffer: token ids, positions, entry of token,
// q_start, context lengths, slots, logit rows, then the planners' sections, then the block
// tables.  Every section starts on a 16-byte boundary.
inline size_t Engine::layout(const StepShape& s, const std::vector<int>& widths, std::vector<size_t>& offsets) const {
    std::vector<size_t> sizes = {(size_t)s.tokens, (size_t)s.tokens, (size_t)s.tokens, (size_t)s.entries + 1,
                                 (size_t)s.entries, (size_t)s.entries, (size_t)s.logit_rows};
    for (auto& p : planners_) {
        std::vector<int> n((size_t)p->sections());
        p->sizes(s, n.data());
        for (int v : n) sizes.push_back((size_t)v);
    }
    for (int w : widths) sizes.push_back((size_t)s.entries * (size_t)w);
    size_t total = 0;
    offsets.clear();
    for (size_t v : sizes) {
        offsets.push_back(total);
        total += (v + 3) / 4 * 4;
    }
    return std::max<size_t>(total, 4);
}

inline void Engine::pack(const StepEntryView* entries, const StepShape& shape, const std::vector<int>& rows,
                         const std::vector<int64_t>& rids, const std::vector<int>& widths, MetaBuffers& mb,
                         StepMeta& meta) {
    std::vector<size_t> off;
    const size_t total = layout(shape, widths, off);
    mb.ensure(total);
    mb.wait();                                   // the copy of the step before has read the host buffer
    int* host = mb.host.as<int>();
    int* dev = mb.device.as<int>();
    int at = 0;
    for (int i = 0; i < shape.entries; ++i) {
        const int q = shape.q_lens[(size_t)i], start = shape.starts[(size_t)i];
        host[off[3] + (size_t)i] = at;
        for (int t = 0; t < q; ++t) {
            host[off[0] + (size_t)at + t] = entries[i].tokens[t];
            host[off[1] + (size_t)at + t] = start + t;
            host[off[2] + (size_t)at + t] = i;
        }
        host[off[4] + (size_t)i] = start;
        host[off[5] + (size_t)i] = shape.slots[(size_t)i];
        at += q;
    }
    host[off[3] + (size_t)shape.entries] = at;
    for (size_t r = 0; r < rows.size(); ++r) host[off[6] + r] = rows[r];
    meta = StepMeta{};
    meta.shape = shape;
    meta.token_ids = dev + off[0];
    meta.positions = dev + off[1];
    meta.entry_of_token = dev + off[2];
    meta.q_start = dev + off[3];
    meta.context_len = dev + off[4];
    meta.slots = dev + off[5];
    meta.logit_rows = rows.empty() ? nullptr : dev + off[6];
    size_t sec = 7;
    for (auto& p : planners_) {
        const int k = p->sections();
        std::vector<int> n((size_t)k);
        p->sizes(shape, n.data());
        std::vector<int*> host_sections, dev_sections;
        for (int j = 0; j < k; ++j) {
            host_sections.push_back(host + off[sec + (size_t)j]);
            dev_sections.push_back(dev + off[sec + (size_t)j]);
        }
        p->fill(shape, host_sections.data());
        meta.work[p->key()] = dev_sections;
        meta.work_sizes[p->key()] = n;
        sec += (size_t)k;
    }
    for (int g = 0; g < (int)groups_.size(); ++g) {
        const int w = widths[(size_t)g];
        if (kipp_cm_rows(cm_, g, shape.entries, rids.data(), w, host + off[sec]))
            fail(KIPP_E_STATE, "a block table is longer than the width of its step");
        meta.block_tables.push_back(dev + off[sec]);
        meta.table_widths.push_back(w);
        ++sec;
    }
    mb.send(total, stream_);
    last_h2d_bytes = (long long)total * 4;
}

inline const float* Engine::forward(StepMeta& meta) {
    StepContext ctx;
    ctx.engine = this;
    ctx.meta = &meta;
    ctx.dtype = dtype_;
    ctx.ops = &ops_;
    ctx.workspace = &workspace_;
    ctx.stream = stream_;
    ctx.kv_round_bf16 = opt_.kv_round_bf16 != 0;
    const long long before = ops_.launches;
    const int T = meta.shape.tokens;
    float* x = workspace_.get<float>("residual", (size_t)T * plan_->hidden_size);
    for (auto& e : plan_->embedding) e.second->forward(ctx, x);
    for (size_t i = 0; i < plan_->order.size(); ++i) {
        const LayerRun& run = plan_->order[i];
        // the block that runs next starts with this norm: the last residual add of this one may
        // leave its deferred form
        ctx.following_norm = i + 1 < plan_->order.size()
                                 ? plan_->layers[(size_t)plan_->order[i + 1].layer].second->deferred_first_norm()
                                 : nullptr;
        plan_->layers[(size_t)run.layer].second->forward(ctx, run, x);
    }
    const float* logits = nullptr;
    const int rows = meta.shape.logit_rows;
    if (rows > 0) {
        void* h = workspace_.buffer("final_normed", (size_t)rows * plan_->hidden_size * dtype_size(dtype_));
        plan_->final_norm.second->forward(ctx, x, h, meta.logit_rows, rows);
        float* out = workspace_.get<float>("logits", (size_t)rows * plan_->vocab_size);
        plan_->head.second->forward(ctx, h, rows, out);
        logits = out;
    }
    last_forward_launches = ops_.launches - before;
    return logits;
}

// Whether steps of this shape (tokens and wanted rows per entry) have been run twice before:
// only shapes that keep coming back are worth a capture.
inline bool Engine::shape_repeats(const StepShape& shape, const std::vector<int>& rows_per_entry) {
    std::string sig;
    for (int i = 0; i < shape.entries; ++i) sig += format("%d/%d,", shape.q_lens[(size_t)i], rows_per_entry[(size_t)i]);
    int& n = shapes_seen_[sig];
    if (n >= 2) return true;
    if (shapes_seen_.size() > 512) {
        shapes_seen_.clear();
        shapes_seen_[sig] = 1;
        return false;
    }
    ++n;
    return false;
}

inline Engine::StepGraph& Engine::graph_for(const std::string& key, bool feedback, int batch) {
    for (auto it = graphs_.begin(); it != graphs_.end(); ++it)
        if ((*it)->key == key) {
            graphs_.splice(graphs_.end(), graphs_, it);          // kept in order of use
            return *graphs_.back();
        }
    if ((int)graphs_.size() >= MAX_GRAPHS) {
        cuda_check(cudaStreamSynchronize(stream_), "before dropping a graph");
        graphs_.pop_front();                                     // the least recently used
    }
    auto g = std::make_unique<StepGraph>();
    g->key = key;
    g->feedback = feedback;
    if (feedback) {
        g->next_tokens.reset((size_t)batch * sizeof(int), "burst tokens");
        g->ring.reset((size_t)burst_ring_rows * batch * sizeof(int), "burst ring");
        g->counter.reset(sizeof(int), "burst counter");
    }
    graphs_.push_back(std::move(g));
    return *graphs_.back();
}

// argmax of the step's logits -> next tokens, ring row, positions + 1, then what each mixer's
// kernels derive from the lengths.
inline void Engine::feedback_tail(StepGraph& g) {
    const int n = g.meta.shape.entries;
    ops_.argmax_rows(g.logits, plan_->vocab_size, n, plan_->vocab_size, g.next_tokens.as<int>());
    ops_.burst_advance(const_cast<int*>(g.meta.token_ids), const_cast<int*>(g.meta.positions),
                       const_cast<int*>(g.meta.context_len), g.next_tokens.as<int>(), g.ring.as<int>(),
                       g.counter.as<int>(), n, burst_ring_rows);
    for (auto& p : planners_) p->advance_on_device(ops_, g.meta.shape, g.meta.work.at(p->key()).data(), g.meta.context_len, n);
}

// Runs a step through its captured graph.  The first step of a key runs the kernels directly and
// is then captured (a capture itself executes nothing), so that a part with per-request state
// advances once; later steps replay.
inline const float* Engine::run_graph(StepGraph& g, const StepEntryView* entries, const StepShape& shape,
                                      const std::vector<int>& rows, const std::vector<int64_t>& rids,
                                      const std::vector<int>& widths) {
    pack(entries, shape, rows, rids, widths, g.meta_buffers, g.meta);
    if (g.exec && g.generation != workspace_.generation) {        // a buffer moved since the capture
        cudaGraphExecDestroy(g.exec);
        cudaGraphDestroy(g.graph);
        g.exec = nullptr;
        g.graph = nullptr;
    }
    if (g.exec) {
        cuda_check(cudaGraphLaunch(g.exec, stream_), "graph launch");
        ++graph_replays;
        graph_kernel_launches += g.launches;
        return g.logits;
    }
    const long long before = ops_.launches;
    g.logits = forward(g.meta);
    g.rows = shape.logit_rows;
    if (g.feedback) feedback_tail(g);
    g.launches = ops_.launches - before;
    const long long generation = workspace_.generation;
    workspace_.capturing = true;
    cudaError_t e = cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        workspace_.capturing = false;
        cuda_check(e, "begin of a graph capture");
    }
    try {
        const float* again = forward(g.meta);
        if (g.feedback) feedback_tail(g);
        if (again != g.logits) fail(KIPP_E_STATE, "the logits buffer moved between a step and its capture");
    } catch (...) {
        cudaGraph_t broken = nullptr;
        cudaStreamEndCapture(stream_, &broken);
        if (broken) cudaGraphDestroy(broken);
        cudaGetLastError();
        workspace_.capturing = false;
        ops_.launches = before + g.launches;
        throw;
    }
    workspace_.capturing = false;
    ops_.launches = before + g.launches;                          // the capture launched nothing
    cuda_check(cudaStreamEndCapture(stream_, &g.graph), "end of a graph capture");
    cuda_check(cudaGraphInstantiate(&g.exec, g.graph, 0), "graph instantiation");
    g.generation = generation;
    ++graphs_captured;
    return g.logits;
}

inline const float* Engine::step(const StepEntryView* entries, int n, int* n_rows) {
    StepShape shape;
    std::vector<int> rows;
    validate(entries, n, shape, rows);
    cuda_check(cudaSetDevice(opt_.device), "cudaSetDevice");
    std::vector<int64_t> rids((size_t)n), admitted;
    std::vector<int> new_lengths((size_t)n);
    shape.starts.resize((size_t)n);
    shape.slots.resize((size_t)n);
    try {
        for (int i = 0; i < n; ++i) {
            rids[(size_t)i] = entries[i].request;
            if (!is_live(entries[i].request)) {
                add_request(entries[i].request);
                admitted.push_back(entries[i].request);
            }
            const int start = kipp_cm_length(cm_, entries[i].request);
            shape.starts[(size_t)i] = start;
            shape.slots[(size_t)i] = kipp_cm_slot(cm_, entries[i].request);
            new_lengths[(size_t)i] = start + entries[i].n_tokens;
            if (plan_->max_positions > 0 && new_lengths[(size_t)i] > plan_->max_positions)
                fail(KIPP_E_ARGUMENT, format("request %lld would pass max positions %lld", (long long)entries[i].request,
                                             plan_->max_positions));
        }
        const int rc = kipp_cm_reserve(cm_, n, rids.data(), new_lengths.data());
        if (rc == KIPP_CM_OUT_OF_PAGES) fail(KIPP_E_OUT_OF_PAGES, "page pool exhausted");
        if (rc == KIPP_CM_BEHIND_WINDOW) fail(KIPP_E_STATE, "a page behind the window was asked for");
        if (rc) fail(KIPP_E_STATE, format("reserve: error %d", rc));
        // the forward pass
        bool decode_only = true;
        std::vector<int> rows_per_entry((size_t)n);
        for (int i = 0; i < n; ++i) {
            rows_per_entry[(size_t)i] = entries[i].n_want;
            decode_only = decode_only && entries[i].n_tokens == 1 && entries[i].n_want == 1;
        }
        const float* logits;
        if (graphable() && (decode_only || shape_repeats(shape, rows_per_entry))) {
            // decode steps, and prompt steps of a shape that keeps coming back (the chunks of long
            // prompts): one graph launch instead of nine launches per layer
            const std::vector<int> widths = table_widths(rids, decode_only ? 64 : 512);
            std::string key = decode_only ? format("decode/%d", n) : std::string("shape/");
            if (!decode_only)
                for (int i = 0; i < n; ++i) key += format("%d/%d,", shape.q_lens[(size_t)i], rows_per_entry[(size_t)i]);
            for (int w : widths) key += format("/w%d", w);
            logits = run_graph(graph_for(key, false, n), entries, shape, rows, rids, widths);
        } else {
            MetaBuffers& mb = staging_[staging_next_];
            staging_next_ = (staging_next_ + 1) % 4;
            StepMeta meta;
            pack(entries, shape, rows, rids, table_widths(rids, 0), mb, meta);
            logits = forward(meta);
        }
        last_logits_ = logits;
        last_rows_ = shape.logit_rows;
    } catch (...) {
        // nothing changes on error: requests this call admitted go away again
        for (int64_t r : admitted) {
            kipp_cm_release(cm_, r);
            live_.erase(r);
        }
        throw;
    }
    for (int i = 0; i < n; ++i) kipp_cm_advance(cm_, rids[(size_t)i], new_lengths[(size_t)i]);
    ++steps_run;
    if (n_rows) *n_rows = shape.logit_rows;
    return last_logits_;
}

// One part of one run alone, on a step of its own: the same checks, reservation and metadata as
// step(), then only that part's forward pass.  The lengths advance as after a step, so that a
// mixer's keys and values stay in the cache for the next call.
inline void Engine::debug_part(const StepEntryView* entries, int n, int run_index, const std::string& which,
                               const void* input, float* residual, void* output) {
    StepShape shape;
    std::vector<int> rows;
    validate(entries, n, shape, rows);
    cuda_check(cudaSetDevice(opt_.device), "cudaSetDevice");
    const bool layer_part = which != "embedding" && which != "final_norm" && which != "head";
    if (layer_part && (run_index < 0 || run_index >= (int)plan_->order.size())) fail(KIPP_E_ARGUMENT, "no such run");
    const LayerRun run = layer_part ? plan_->order[(size_t)run_index] : LayerRun{};
    std::vector<int64_t> rids((size_t)n);
    std::vector<int> new_lengths((size_t)n);
    shape.starts.resize((size_t)n);
    shape.slots.resize((size_t)n);
    for (int i = 0; i < n; ++i) {
        rids[(size_t)i] = entries[i].request;
        if (!is_live(entries[i].request)) add_request(entries[i].request);
        shape.starts[(size_t)i] = kipp_cm_length(cm_, entries[i].request);
        shape.slots[(size_t)i] = kipp_cm_slot(cm_, entries[i].request);
        new_lengths[(size_t)i] = shape.starts[(size_t)i] + entries[i].n_tokens;
    }
    const int rc = kipp_cm_reserve(cm_, n, rids.data(), new_lengths.data());
    if (rc == KIPP_CM_OUT_OF_PAGES) fail(KIPP_E_OUT_OF_PAGES, "page pool exhausted");
    if (rc) fail(KIPP_E_STATE, format("reserve: error %d", rc));
    MetaBuffers& mb = staging_[staging_next_];
    staging_next_ = (staging_next_ + 1) % 4;
    StepMeta meta;
    pack(entries, shape, rows, rids, table_widths(rids, 0), mb, meta);
    StepContext ctx;
    ctx.engine = this;
    ctx.meta = &meta;
    ctx.dtype = dtype_;
    ctx.ops = &ops_;
    ctx.workspace = &workspace_;
    ctx.stream = stream_;
    ctx.kv_round_bf16 = opt_.kv_round_bf16 != 0;
    const int T = shape.tokens;
    Block* block = layer_part ? plan_->layers[(size_t)run.layer].second.get() : nullptr;
    PreNormBlock* pre = dynamic_cast<PreNormBlock*>(block);
    auto need_pre = [&] {
        if (!pre) fail(KIPP_E_UNSUPPORTED, "this layer's block does not name its parts");
        return pre;
    };
    if (which == "embedding") {
        for (auto& e : plan_->embedding) e.second->forward(ctx, residual);
    } else if (which == "input_norm") {
        need_pre()->input_norm()->forward(ctx, residual, output, nullptr, T);
    } else if (which == "post_norm") {
        need_pre()->post_norm()->forward(ctx, residual, output, nullptr, T);
    } else if (which == "mixer") {
        block->mixers().at(0)->forward(ctx, run, 0, input, residual);
    } else if (which == "feed_forward") {
        need_pre()->feed_forward()->forward(ctx, input, residual);
    } else if (which == "block") {
        block->forward(ctx, run, residual);
    } else if (which == "final_norm") {
        plan_->final_norm.second->forward(ctx, residual, output, meta.logit_rows, meta.logit_rows ? shape.logit_rows : T);
    } else if (which == "head") {
        plan_->head.second->forward(ctx, input, shape.logit_rows > 0 ? shape.logit_rows : T, static_cast<float*>(output));
    } else {
        fail(KIPP_E_ARGUMENT, "unknown part '" + which + "'");
    }
    for (int i = 0; i < n; ++i) kipp_cm_advance(cm_, rids[(size_t)i], new_lengths[(size_t)i]);
    check_status();
}

inline void Engine::check_status() {
    int words[4] = {0, 0, 0, 0};
    cuda_check(cudaMemcpyAsync(words, status_.get(), sizeof words, cudaMemcpyDeviceToHost, stream_), "status read");
    cuda_check(cudaStreamSynchronize(stream_), "synchronize");
    if (!words[0] && !words[1] && !words[2] && !words[3]) return;
    cuda_check(cudaMemsetAsync(status_.get(), 0, sizeof words, stream_), "status reset");
    std::string what;
    if (words[0]) {
        const char* names[] = {"", "a token id outside the vocabulary", "a write to an unmapped cache page",
                               "a read of an unmapped cache page"};
        what += words[0] >= 1 && words[0] <= 3 ? std::string("a kernel refused ") + names[words[0]]
                                               : format("a kernel reported code %d", words[0]);
    }
    for (int i = 1; i < 4; ++i)
        if (words[i])
            what += format("%sa bounded wait of a tensor-core kernel ran out (status word %d = %d): its results are "
                           "not to be trusted", what.empty() ? "" : "; ", i, words[i]);
    fail(KIPP_E_KERNEL, what);
}

inline void Engine::synchronize() {
    cuda_check(cudaSetDevice(opt_.device), "cudaSetDevice");
    check_status();
}

inline void Engine::read_logits(float* out, size_t capacity) {
    const size_t n = (size_t)last_rows_ * plan_->vocab_size;
    if (!last_logits_ || n == 0) fail(KIPP_E_STATE, "the last step wanted no logits");
    if (capacity < n) fail(KIPP_E_ARGUMENT, format("the logits need room for %zu floats", n));
    cuda_check(cudaMemcpyAsync(out, last_logits_, n * sizeof(float), cudaMemcpyDeviceToHost, stream_), "logits read");
    check_status();
}

// Greedy decoding of `steps` tokens for every request without the host in the loop.  The step is
// captured in a CUDA graph together with its argmax, the hand-over of the chosen tokens and the
// move of every request to its next position, so a burst is a run of graph replays with no copy
// and no other launch in between.  Pages for all steps are taken first (out of pages leaves every
// request as it was).  Callers that must look at every token (stop tokens, sampling) use step().
inline void Engine::decode_burst(const int64_t* requests, const int32_t* tokens, int n, int steps, int32_t* out_host) {
    if (n <= 0 || steps <= 0) return;
    cuda_check(cudaSetDevice(opt_.device), "cudaSetDevice");
    std::set<int64_t> seen;
    std::vector<int64_t> rids(requests, requests + n);
    std::vector<int> starts((size_t)n), ends((size_t)n);
    for (int i = 0; i < n; ++i) {
        if (!seen.insert(requests[i]).second)
            fail(KIPP_E_ARGUMENT, format("request %lld appears twice in one burst", (long long)requests[i]));
        if (!is_live(requests[i]))
            fail(KIPP_E_STATE, format("decode_burst: request %lld is not live (feed its prompt with step)",
                                      (long long)requests[i]));
        if (tokens[i] < 0 || tokens[i] >= plan_->vocab_size) fail(KIPP_E_ARGUMENT, "a token id is outside the vocabulary");
        starts[(size_t)i] = kipp_cm_length(cm_, requests[i]);
        ends[(size_t)i] = starts[(size_t)i] + steps;
        if (plan_->max_positions > 0 && ends[(size_t)i] > plan_->max_positions)
            fail(KIPP_E_ARGUMENT, format("a request would pass max positions %lld", plan_->max_positions));
    }
    if (!graphable()) {
        // no graphs: the same tokens, one step at a time
        std::vector<int32_t> cur(tokens, tokens + n);
        const int32_t zero = 0;
        for (int k = 0; k < steps; ++k) {
            std::vector<StepEntryView> entries((size_t)n);
            for (int i = 0; i < n; ++i) entries[(size_t)i] = {requests[i], &cur[(size_t)i], 1, &zero, 1};
            int rows = 0;
            const float* logits = step(entries.data(), n, &rows);
            int* picked = workspace_.get<int>("burst_tokens", (size_t)n);
            ops_.argmax_rows(logits, plan_->vocab_size, n, plan_->vocab_size, picked);
            cuda_check(cudaMemcpyAsync(out_host + (size_t)k * n, picked, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost,
                                       stream_), "burst tokens");
            cuda_check(cudaStreamSynchronize(stream_), "synchronize");
            for (int i = 0; i < n; ++i) cur[(size_t)i] = out_host[(size_t)k * n + i];
        }
        return;
    }
    // the pages of all steps are mapped first: all or nothing, and the block tables then stay
    const int rc = kipp_cm_reserve(cm_, n, rids.data(), ends.data());
    if (rc == KIPP_CM_OUT_OF_PAGES) fail(KIPP_E_OUT_OF_PAGES, "page pool exhausted");
    if (rc) fail(KIPP_E_STATE, format("reserve: error %d", rc));
    StepShape shape;
    shape.entries = shape.tokens = shape.logit_rows = n;
    shape.q_lens.assign((size_t)n, 1);
    shape.starts = starts;
    shape.slots.resize((size_t)n);
    std::vector<int> rows((size_t)n);
    std::vector<StepEntryView> entries((size_t)n);
    const int32_t zero = 0;
    for (int i = 0; i < n; ++i) {
        shape.slots[(size_t)i] = kipp_cm_slot(cm_, requests[i]);
        rows[(size_t)i] = i;
        entries[(size_t)i] = {requests[i], tokens + i, 1, &zero, 1};
    }
    const std::vector<int> widths = table_widths(rids, 64);
    std::string key = format("burst/%d", n);
    for (int w : widths) key += format("/w%d", w);
    StepGraph& g = graph_for(key, true, n);
    int done = 0;
    bool first = true;
    while (done < steps) {
        const int chunk = std::min(steps - done, burst_ring_rows);
        cuda_check(cudaMemsetAsync(g.counter.get(), 0, sizeof(int), stream_), "burst counter");
        int replays = chunk;
        if (first) {
            run_graph(g, entries.data(), shape, rows, rids, widths);     // packs, captures if need be, runs once
            first = false;
            --replays;
        }
        for (int k = 0; k < replays; ++k) cuda_check(cudaGraphLaunch(g.exec, stream_), "graph launch");
        graph_replays += replays;
        graph_kernel_launches += (long long)replays * g.launches;
        cuda_check(cudaMemcpyAsync(out_host + (size_t)done * n, g.ring.get(), (size_t)chunk * n * sizeof(int),
                                   cudaMemcpyDeviceToHost, stream_), "burst tokens");
        cuda_check(cudaStreamSynchronize(stream_), "synchronize");
        done += chunk;
    }
    for (int i = 0; i < n; ++i) kipp_cm_advance(cm_, requests[i], ends[(size_t)i]);
    steps_run += steps;
    last_logits_ = g.logits;
    last_rows_ = n;
}

// ---------------------------------------------------------------------------------------------
// One step of the reference's generator (xorshift64*, src/kipp.c:3322-3333): uniform in [0, 1)
// with 53 bits.
inline double next_uniform(uint64_t& state) {
    uint64_t x = state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    state = x;
    const uint64_t r = x * 2685821657736338717ull;
    return (double)(r >> 11) / 9007199254740992.0;
}

// Turns the logits of the last step into one token per row, on the device.  The host keeps each
// request's generator state and draws the uniform number; the kernels do everything that touches
// the vocabulary (bias, penalties, maximum, candidate cut, top-k, min-p, nucleus, the draw).
inline void Engine::sample(const kipp_sample_params* params, uint64_t* rng_states, int n_rows, int32_t* out_host) {
    if (n_rows <= 0) return;
    if (!last_logits_ || n_rows != last_rows_)
        fail(KIPP_E_ARGUMENT, format("one set of sampling options per row of the last step's logits (%d rows)", last_rows_));
    cuda_check(cudaSetDevice(opt_.device), "cudaSetDevice");
    const int vocab = plan_->vocab_size;
    float* logits = const_cast<float*>(last_logits_);
    bool any_penalty = false, any_bias = false, any_random = false;
    int recent_width = 0, bias_width = 0;
    for (int i = 0; i < n_rows; ++i) {
        const kipp_sample_params& p = params[i];
        if (!(p.top_p > 0.f && p.top_p <= 1.f)) fail(KIPP_E_ARGUMENT, "top_p must be greater than 0 and at most 1");
        if (!(p.min_p >= 0.f && p.min_p <= 1.f)) fail(KIPP_E_ARGUMENT, "min_p must be between 0 and 1");
        if (p.top_k < 0) fail(KIPP_E_ARGUMENT, "top_k must not be negative");
        if (p.temperature > 0.f && rng_states[i] == 0) fail(KIPP_E_ARGUMENT, "sampling requires a nonzero generator state");
        const bool pen = p.frequency_penalty != 0.f || p.presence_penalty != 0.f ||
                         (p.repetition_penalty != 0.f && p.repetition_penalty != 1.f);
        if (pen && p.recent_count > 0) {
            any_penalty = true;
            recent_width = std::max(recent_width, p.recent_count);
        }
        if (p.logit_bias_count > 0) {
            any_bias = true;
            bias_width = std::max(bias_width, p.logit_bias_count);
        }
        any_random = any_random || p.temperature > 0.f;
    }
    // host block: [recent n x rw][recent_count n][rep n][pres n][freq n][bias tok n x bw][bias val n x bw]
    //             [bias count n][temperature n][top_k n][top_p n][min_p n][uniform n (double)]
    const size_t n = (size_t)n_rows, rw = (size_t)recent_width, bw = (size_t)bias_width;
    size_t words = n * rw + n * 4 + 2 * n * bw + n + 4 * n;
    words = (words + 1) / 2 * 2;
    const size_t bytes = words * 4 + n * 8 + 16;
    sample_host_.ensure(bytes);
    int* hw = sample_host_.as<int>();
    std::fill(hw, hw + words + 2 * n, 0);
    int* recent = hw;
    int* recent_count = recent + n * rw;
    float* rep = reinterpret_cast<float*>(recent_count + n);
    float* pres = rep + n;
    float* freq = pres + n;
    int* bias_tok = reinterpret_cast<int*>(freq + n);
    float* bias_val = reinterpret_cast<float*>(bias_tok + n * bw);
    int* bias_count = reinterpret_cast<int*>(bias_val + n * bw);
    float* temperature = reinterpret_cast<float*>(bias_count + n);
    int* top_k = reinterpret_cast<int*>(temperature + n);
    float* top_p = reinterpret_cast<float*>(top_k + n);
    float* min_p = top_p + n;
    double* uniform = reinterpret_cast<double*>(hw + words);
    for (int i = 0; i < n_rows; ++i) {
        const kipp_sample_params& p = params[i];
        const bool pen = p.frequency_penalty != 0.f || p.presence_penalty != 0.f ||
                         (p.repetition_penalty != 0.f && p.repetition_penalty != 1.f);
        for (size_t j = 0; j < rw; ++j) recent[(size_t)i * rw + j] = -1;
        if (pen && p.recent_count > 0) {
            for (int j = 0; j < p.recent_count; ++j) recent[(size_t)i * rw + (size_t)j] = p.recent_tokens[j];
            recent_count[i] = p.recent_count;
        }
        rep[i] = p.repetition_penalty;
        pres[i] = p.presence_penalty;
        freq[i] = p.frequency_penalty;
        for (int j = 0; j < p.logit_bias_count; ++j) {
            bias_tok[(size_t)i * bw + (size_t)j] = p.logit_bias_tokens[j];
            bias_val[(size_t)i * bw + (size_t)j] = p.logit_bias_values[j];
        }
        bias_count[i] = p.logit_bias_count;
        temperature[i] = p.temperature;
        top_k[i] = p.top_k;
        top_p[i] = p.top_p;
        min_p[i] = p.min_p;
        // the generator moves for rows with temperature > 0 only, as the reference leaves it
        // untouched on the greedy path
        uniform[i] = p.temperature > 0.f ? next_uniform(rng_states[i]) : 0.0;
    }
    char* dev = static_cast<char*>(workspace_.buffer("sample_params", bytes + n * 4));
    cuda_check(cudaMemcpyAsync(dev, hw, bytes, cudaMemcpyHostToDevice, stream_), "sampling options");
    auto at = [&](const void* host_ptr) { return dev + (static_cast<const char*>(host_ptr) - reinterpret_cast<char*>(hw)); };
    int* out_dev = reinterpret_cast<int*>(dev + bytes);
    if (any_penalty || any_bias)
        ops_.apply_penalties(logits, vocab, n_rows, vocab, any_penalty ? (const int*)at(recent) : nullptr,
                             any_penalty ? recent_width : 0, any_penalty ? (const int*)at(recent_count) : nullptr,
                             any_penalty ? (const float*)at(rep) : nullptr, any_penalty ? (const float*)at(pres) : nullptr,
                             any_penalty ? (const float*)at(freq) : nullptr, any_bias ? (const int*)at(bias_tok) : nullptr,
                             any_bias ? (const float*)at(bias_val) : nullptr, any_bias ? bias_width : 0,
                             any_bias ? (const int*)at(bias_count) : nullptr);
    if (!any_random)
        ops_.argmax_rows(logits, vocab, n_rows, vocab, out_dev);
    else
        ops_.sample_rows(logits, vocab, n_rows, vocab, (const float*)at(temperature), (const int*)at(top_k),
                         (const float*)at(top_p), (const float*)at(min_p), (const double*)at(uniform), out_dev);
    cuda_check(cudaMemcpyAsync(out_host, out_dev, n * sizeof(int), cudaMemcpyDeviceToHost, stream_), "sampled tokens");
    cuda_check(cudaStreamSynchronize(stream_), "synchronize");
}

// ---------------------------------------------------------------------------------------------
inline size_t Engine::weight_bytes() const {
    // bytes of weights one step reads (each weight once)
    size_t n = 0;
    for (auto& run : plan_->order) n += plan_->layers[(size_t)run.layer].second->weight_bytes();
    return n + plan_->final_norm.second->weight_bytes() + plan_->head.second->weight_bytes();
}

inline size_t Engine::cache_bytes_per_token() const {
    size_t n = 0;
    for (auto& g : groups_)
        n += (size_t)2 * g.cache_keys.size() * g.spec.kv_heads * g.spec.head_dim * dtype_size(dtype_);
    return n;
}

// What is loaded and what it may hold (the reference's kipp_model_info and kipp_session_info in
// one, src/kipp.h:109-145, 172-200).
inline std::string Engine::info_json() {
    Json j = Json::object();
    if (plan_->config.is_object() && plan_->config.has("architectures"))
        j.set("architecture", architecture_of(plan_->config));
    j.set("dtype", dtype_name(dtype_));
    j.set("device", opt_.device);
    j.set("sm_count", device_.sm_count);
    j.set("layers", (long long)plan_->layers.size());
    j.set("runs", (long long)plan_->order.size());
    j.set("hidden_size", plan_->hidden_size);
    j.set("vocab_size", plan_->vocab_size);
    j.set("max_positions", plan_->max_positions > 0 ? Json(plan_->max_positions) : Json(nullptr));
    j.set("weight_bytes", (long long)weight_bytes());
    j.set("weight_bytes_allocated", (long long)weight_bytes_allocated_);
    j.set("cache_bytes_per_token", (long long)cache_bytes_per_token());
    j.set("cache_tokens", opt_.cache_tokens);
    j.set("page_size", opt_.page_size);
    j.set("max_requests", opt_.max_requests);
    j.set("free_slots", free_slots());
    j.set("max_batch_tokens", opt_.max_batch_tokens);
    j.set("max_logit_rows", opt_.max_logit_rows);
    j.set("cuda_graphs", graphable());
    j.set("kv_round_bf16", opt_.kv_round_bf16 != 0);
    j.set("own_length_splits", opt_.own_length_splits != 0);
    j.set("workspace_bytes", (long long)workspace_.bytes());
    Json groups = Json::array();
    for (size_t g = 0; g < groups_.size(); ++g) {
        Json o = Json::object();
        o.set("caches", (long long)groups_[g].cache_keys.size());
        o.set("kv_heads", groups_[g].spec.kv_heads);
        o.set("head_dim", groups_[g].spec.head_dim);
        o.set("window", groups_[g].spec.window > 0 ? Json(groups_[g].spec.window) : Json(nullptr));
        o.set("pages", groups_[g].n_pages);
        o.set("free_pages", group_free_pages((int)g));
        groups.push(std::move(o));
    }
    j.set("cache_groups", std::move(groups));
    Json states = Json::array();
    for (auto& kv : states_) {
        Json o = Json::object();
        o.set("cache", kv.first / 16);
        o.set("bytes_per_request", (long long)kv.second.spec.bytes());
        states.push(std::move(o));
    }
    j.set("states", std::move(states));
    Json live = Json::object();
    for (int64_t r : live_) live.set(std::to_string((long long)r), kipp_cm_length(cm_, r));
    j.set("live_requests", std::move(live));
    Json counters = Json::object();
    counters.set("steps_run", steps_run);
    counters.set("kernel_launches", ops_.launches + graph_kernel_launches);
    counters.set("graph_replays", graph_replays);
    counters.set("graphs_captured", graphs_captured);
    counters.set("last_forward_launches", last_forward_launches);
    counters.set("last_h2d_bytes", last_h2d_bytes);
    counters.set("tc_prefill_launches", ops_.tc_prefill_launches);
    counters.set("fused_decode_launches", ops_.fused_decode_launches);
    counters.set("folded_norms", ops_.folded_norms);
    counters.set("stream_decode_launches", ops_.stream_decode_launches);
    counters.set("projections_to_heads", ops_.projections_to_heads);
    j.set("counters", std::move(counters));
    info_ = j.dump();
    return info_;
}

}  // namespace kipp
