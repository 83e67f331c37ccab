// The parts the library brings: token embedding, RMSNorm, rotary position encodings, causal
// grouped-query attention over the paged cache, the SwiGLU feed-forward, the output head, the
// pre-norm block, and the wrapper behind parts whose forward pass the caller supplies.  Each
// is registered under a kind name; a plan builds them from JSON objects of sizes and constants.
#pragma once
#include "model.hpp"

namespace kipp {

// ---------------------------------------------------------------------------------------------
// x_t = float(E[id_t, :]) with no scale (src/kipp.c:2940-2942).
class TokenEmbedding : public EmbeddingStage {
public:
    TokenEmbedding(int vocab, int hidden) : vocab_(vocab), hidden_(hidden) {
        if (vocab <= 0 || hidden <= 0) fail(KIPP_E_CONFIG, "token_embedding: sizes must be positive");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + "weight";
        s.shape = {vocab_, hidden_};
        out.push_back(s);
    }
    void bind(Binder& b, const std::string& prefix) override {
        dtype_ = b.compute_dtype();
        weight_ = b.shared(prefix + "weight", dtype_, vocab_, hidden_);
    }
    void forward(StepContext& ctx, float* x) override {
        ctx.ops->embed_gather(x, weight_, dtype_, ctx.meta->token_ids, ctx.tokens(), hidden_, vocab_);
    }

private:
    int vocab_, hidden_, dtype_ = BF16;
    void* weight_ = nullptr;
};

// logits = W n for the wanted rows only; W is the tensor `tied_to` when the checkpoint has no
// head of its own (src/kipp.c:951-956, 3013-3018).
class OutputHead : public Head {
public:
    OutputHead(int vocab, int hidden, std::string tied_to) : vocab_(vocab), hidden_(hidden), tied_to_(std::move(tied_to)) {
        if (vocab <= 0 || hidden <= 0) fail(KIPP_E_CONFIG, "output_head: sizes must be positive");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + "weight";
        s.shape = {vocab_, hidden_};
        if (!tied_to_.empty()) {
            s.optional = true;
            s.alias_of = tied_to_;
            s.ignore_if_present = true;
        }
        out.push_back(s);
    }
    void bind(Binder& b, const std::string& prefix) override {
        dtype_ = b.compute_dtype();
        weight_ = b.shared(tied_to_.empty() ? prefix + "weight" : tied_to_, dtype_, vocab_, hidden_);
    }
    size_t weight_bytes() const override { return (size_t)vocab_ * hidden_ * dtype_size(dtype_); }
    int vocab_size() const override { return vocab_; }
    void forward(StepContext& ctx, const void* h, int n_rows, float* logits) override {
        ctx.ops->gemm(logits, F32, vocab_, h, hidden_, weight_, hidden_, dtype_, n_rows, vocab_, hidden_, EPI_STORE);
    }

private:
    int vocab_, hidden_, dtype_ = BF16;
    std::string tied_to_;
    void* weight_ = nullptr;
};

// y = x * rsqrt(mean(x^2) + eps) * w, computed in float32 (src/kipp.c:2221-2231).
class RMSNorm : public Norm {
public:
    RMSNorm(int size, double eps, std::string weight_name) : size_(size), eps_((float)eps), name_(std::move(weight_name)) {
        if (size <= 0 || !(eps > 0)) fail(KIPP_E_CONFIG, "rmsnorm: size and eps must be positive");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + name_;
        s.shape = {size_};
        s.init = "near_one";
        out.push_back(s);
    }
    void bind(Binder& b, const std::string& prefix) override {
        // the scale keeps its storage type (bfloat16 or float32)
        wdtype_ = storage_dtype(b.stored_dtype(prefix + name_));
        weight_ = b.allocate((size_t)size_ * dtype_size(wdtype_), prefix + name_);
        b.load(prefix + name_, weight_, wdtype_, size_, 1, size_);
    }
    size_t weight_bytes() const override { return (size_t)size_ * dtype_size(wdtype_); }
    int size() const override { return size_; }
    std::optional<RmsNormSpec> rms_spec() const override { return RmsNormSpec{weight_, wdtype_, eps_, size_}; }
    void forward(StepContext& ctx, const float* x, void* out, const int* rows, int n_rows) override {
        ctx.ops->rmsnorm(out, ctx.dtype, x, weight_, wdtype_, rows, n_rows, size_, eps_);
    }

private:
    int size_;
    float eps_;
    std::string name_;
    int wdtype_ = F32;
    void* weight_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Rotations given by a table of frequencies: pair (i, i + rotary_dim/2) of a head turns by
// position * inv_freq[i].
class FrequencyTable : public PositionEncoding {
public:
    FrequencyTable(std::vector<float> inv_freq, std::string key) : freq_(std::move(inv_freq)), key_(std::move(key)) {}
    int rotary_dim() const override { return 2 * (int)freq_.size(); }
    const float* inv_freq_device() const override { return device_; }
    std::string table_key() const override { return key_; }
    void bind(Binder& b, const std::string&) override {
        if (freq_.empty() || device_) return;
        device_ = static_cast<float*>(b.allocate(freq_.size() * sizeof(float), "rotary frequencies"));
        cuda_check(cudaMemcpy(device_, freq_.data(), freq_.size() * sizeof(float), cudaMemcpyHostToDevice),
                   "upload of rotary frequencies");
    }
    const std::vector<float>& frequencies() const { return freq_; }

private:
    std::vector<float> freq_;
    std::string key_;
    float* device_ = nullptr;
};

// Half-split rotary encoding (src/kipp.c:2368-2382): the frequency of pair i is
// theta^(-2i/rot) as the reference's powf(theta, -(2.0f * i) / rot): a float32 exponent, the
// power rounded to float32 once.
inline std::vector<float> rotary_frequencies(int rotary_dim, double theta) {
    std::vector<float> f((size_t)rotary_dim / 2);
    const double base = (double)(float)theta;
    for (int i = 0; i < rotary_dim / 2; ++i) {
        const float exponent = -(2.0f * (float)i) / (float)rotary_dim;
        f[(size_t)i] = (float)std::pow(base, (double)exponent);
    }
    return f;
}

// ---------------------------------------------------------------------------------------------
// The work lists of the paged attention kernels and the rule for the decode splits.  The
// constants are those kernels': 64-token query tiles (mma.sync prompt kernel), 128-token tiles
// (tcgen05 prompt kernel), three decode CTAs resident per SM.
class AttentionPlanner : public WorkPlanner {
public:
    static constexpr int TILE = 64;
    static constexpr int CTA_FIXED_TILES = 5;   // what a decode CTA costs beside its key tiles, in 64-key tiles
    static constexpr int CTAS_PER_SM = 3;
    static constexpr double STREAM_MARGIN = 1.15;   // the stream cut must look this much better to be taken

    AttentionPlanner(int kv_heads, int sm_count, bool own_length)
        : kv_heads_(kv_heads), resident_(CTAS_PER_SM * std::max(sm_count, 1)), own_length_(own_length) {}

    static std::string key_for(int kv_heads, int sm_count, bool own_length) {
        return format("paged_attention/kv%d/sm%d/%s", kv_heads, sm_count, own_length ? "own" : "step");
    }
    std::string key() const override { return key_for(kv_heads_, resident_ / CTAS_PER_SM, own_length_); }
    int sections() const override { return 5; }

    void sizes(const StepShape& s, int* n) const override {
        int decode = 0, items = 0, all = 0, items128 = 0;
        for (int q : s.q_lens) {
            all += (q + TILE - 1) / TILE;
            if (q == 1) { ++decode; continue; }
            items += (q + TILE - 1) / TILE;
            items128 += (q + 2 * TILE - 1) / (2 * TILE);
        }
        n[0] = decode; n[1] = decode; n[2] = 2 * items; n[3] = 2 * all; n[4] = 2 * items128;
    }

    // Keys per split for the decoded tokens of a step, in whole 64-key tiles.  A CTA takes one
    // split of one (token, kv head) pair and costs its k tiles plus a fixed part (its set-up, the
    // merge of its four warps, its partial results); the CTAs run in waves of as many as the GPU
    // holds at once.  Among the numbers of tiles per split k (splits = total tiles / k, rounded
    // up, at most DECODE_MAX_SPLITS) the one with the least waves x (k + fixed part) is taken: many
    // short splits when there are few pairs (a single token's attention is bound by latency, so
    // down to one tile per split), few long ones once the pairs alone fill the GPU.  On a tie the
    // fewer splits.  The device makes the same choice between the steps of a burst
    // (kipp_attn_decode_replan): integers only, so both agree.
    int step_split_length(int decoded, int longest) const {
        if (decoded <= 0 || longest <= 0) return TILE;
        const long long pairs = (long long)decoded * kv_heads_;
        const int total = (longest + TILE - 1) / TILE;
        int best = total;
        long long best_cost = -1;
        for (int k = total; k >= 1; --k) {
            const int splits = (total + k - 1) / k;
            if (splits > Ops::DECODE_MAX_SPLITS) break;
            const long long waves = (pairs * splits + resident_ - 1) / resident_;
            const long long cost = waves * (k + CTA_FIXED_TILES);
            if (best_cost < 0 || cost < best_cost) { best = k; best_cost = cost; }
        }
        return best * TILE;
    }
    // From the token's own context only (an eighth of it): the grouping of its partial sums then
    // does not depend on what else is in the batch (the reference's lesson,
    // metal/kipp_kernels.metal:82-100).
    static int own_split_length(int kv_len) {
        const int own = (kv_len + 7) / 8;
        return std::max(TILE, (own + TILE - 1) / TILE * TILE);
    }

    void fill(const StepShape& s, int* const* sec) const override {
        int d = 0, a = 0, b = 0, c = 0, longest = 0;
        for (int i = 0; i < s.entries; ++i)
            if (s.q_lens[(size_t)i] == 1) longest = std::max(longest, s.starts[(size_t)i] + 1);
        int decoded = 0;
        for (int q : s.q_lens) decoded += q == 1;
        const int step_keys = step_split_length(decoded, longest);
        for (int i = 0; i < s.entries; ++i) {
            const int q = s.q_lens[(size_t)i];
            for (int t = 0; t < q; t += TILE) { sec[3][b++] = i; sec[3][b++] = t; }
            if (q == 1) {
                sec[0][d] = i;
                sec[1][d] = own_length_ ? own_split_length(s.starts[(size_t)i] + 1) : step_keys;
                ++d;
                continue;
            }
            for (int t = 0; t < q; t += TILE) { sec[2][a++] = i; sec[2][a++] = t; }
            for (int t = 0; t < q; t += 2 * TILE) { sec[4][c++] = i; sec[4][c++] = t; }
        }
    }

    void advance_on_device(Ops& ops, const StepShape& s, int* const* sec, const int* context_len,
                           int entries) const override {
        // (the stream cut reads the lengths itself: no keys per split to bring up to date)
        if (stream_pays(s)) return;
        ops.decode_replan(sec[1], context_len, sec[0], entries, kv_heads_, resident_, CTA_FIXED_TILES,
                          Ops::DECODE_MAX_SPLITS, own_length_ ? 1 : 0);
    }

    // Whether the decoded tokens of a step are better cut as a stream over one wave of CTAs (see
    // attn_decode_stream_kernel) than into splits of the step's length: where the splits need
    // more than one wave or leave much of one empty (64 tokens of 2,048 keys: 5.93 against 6.26
    // ms a step; 8 tokens: 2.67 against 2.49, a run then spans two pairs and pays their set-up
    // twice, hence the margin).  Never where every token's splits are to come from its own length.
    bool stream_pays(const StepShape& s) const {
        if (own_length_) return false;
        long long tiles = 0;
        int longest = 0, decoded = 0;
        for (int i = 0; i < s.entries; ++i) {
            if (s.q_lens[(size_t)i] != 1) continue;
            const int keys = s.starts[(size_t)i] + 1;
            tiles += (keys + TILE - 1) / TILE;
            longest = std::max(longest, keys);
            ++decoded;
        }
        if (decoded == 0 || !Ops::decode_stream_ok(decoded)) return false;
        const long long pairs = (long long)decoded * kv_heads_;
        const int most = (longest + TILE - 1) / TILE;
        const int k = step_split_length(decoded, longest) / TILE;
        const long long splits = (most + k - 1) / k;
        const double split_cost = (double)((pairs * splits + resident_ - 1) / resident_) * (k + CTA_FIXED_TILES);
        const long long total = tiles * kv_heads_;
        const long long per = std::max<long long>({(total + resident_ - 1) / resident_,
                                                   (most + Ops::DECODE_MAX_SPLITS - 2) / (Ops::DECODE_MAX_SPLITS - 1), 1});
        const double pieces = 1.0 + (double)per * (double)pairs / (double)total;      // pairs a run touches
        const double stream_cost = (double)per + CTA_FIXED_TILES * pieces;
        return stream_cost * STREAM_MARGIN < split_cost;
    }

    AttentionWork work_of(const StepMeta& meta) const {
        const std::string key = this->key();
        const int stream_ctas = stream_pays(meta.shape) ? resident_ : 0;
        AttentionWork w;
        auto it = meta.work.find(key);
        if (it == meta.work.end()) fail(KIPP_E_STATE, "the step carries no work lists for " + key);
        const std::vector<int*>& sec = it->second;
        const std::vector<int>& n = meta.work_sizes.at(key);
        w.decode_rows = sec[0]; w.n_decode = n[0];
        w.split_keys = sec[1];
        w.stream_ctas = stream_ctas;
        w.prefill_work = sec[2]; w.n_prefill_items = n[2] / 2;
        w.all_work = sec[3]; w.n_all_items = n[3] / 2;
        w.prefill_work128 = sec[4]; w.n_prefill_items128 = n[4] / 2;
        for (int q : meta.shape.q_lens)
            if (q > 1) w.longest_portion = std::max(w.longest_portion, q);
        w.entries = meta.shape.entries;
        w.tokens = meta.shape.tokens;
        return w;
    }

private:
    int kv_heads_, resident_;
    bool own_length_;
};

// ---------------------------------------------------------------------------------------------
// Norms in deferred form (see NormFold, StepContext::input_scale): what a part's first product and
// its residual add pass to the kernels, and what a block runs where no residual add left the form.
inline const NormFold* fold_input(const StepContext& ctx, NormFold& f) {
    if (!ctx.input_scale.valid()) return nullptr;
    f = NormFold{};
    f.ssq_in = ctx.input_scale.ssq;
    f.ssq_in_slots = ctx.input_scale.slots;
    f.inv_n = ctx.input_scale.inv_n;
    f.eps = ctx.input_scale.eps;
    return &f;
}
inline float* fold_sums(StepContext& ctx, int hidden) {
    return ctx.workspace->get<float>("norm_ssq", (size_t)ctx.tokens() * (size_t)std::max(1, hidden / 32));
}
inline const NormFold* fold_emit(StepContext& ctx, NormFold& f, int hidden) {
    const int T = ctx.tokens();
    if (ctx.emit_for == nullptr || ctx.emit_for->size != hidden || hidden % 32 || !Ops::gemm_emit_ok(T)) return nullptr;
    f = NormFold{};
    f.norm_w = ctx.emit_for->weight;
    f.norm_w_dtype = ctx.emit_for->weight_dtype;
    f.xn = ctx.workspace->buffer("normed", (size_t)T * hidden * ctx.element());
    f.ldn = hidden;
    f.ssq_out = fold_sums(ctx, hidden);
    return &f;
}
inline RowScale deferred_norm(StepContext& ctx, const RmsNormSpec& norm, const float* x, void* h) {
    float* ssq = fold_sums(ctx, norm.size);
    ctx.ops->rmsnorm_deferred(h, ctx.dtype, ssq, x, norm.weight, norm.weight_dtype, nullptr, ctx.tokens(), norm.size);
    return RowScale{ssq, 1, 1.0f / (float)norm.size, norm.eps};
}
inline void fold_emitted(StepContext& ctx, const NormFold* f, int hidden) {
    if (f == nullptr) return;
    ctx.emitted = true;
    ctx.emitted_scale = RowScale{f->ssq_out, hidden / 32, 1.0f / (float)hidden, ctx.emit_for->eps};
}

// ---------------------------------------------------------------------------------------------
// Causal grouped-query attention over the paged cache, with optional per-head q/k RMSNorm and a
// position encoding applied to q and k.  Order of operations as the reference's block
// (docs/ARCHITECTURE.md:77-92, src/kipp.c:2950-2993): q/k/v projections (no bias) -> per-head
// norm of q and k -> rotation -> keys and values into the cache -> attention -> output
// projection added to the residual stream.
class AttentionMixer : public Mixer {
public:
    AttentionMixer(int hidden, int heads, int kv_heads, int head_dim, std::unique_ptr<PositionEncoding> position,
                   std::optional<double> qk_norm_eps, int window, std::optional<double> scale)
        : hidden_(hidden), heads_(heads), kv_heads_(kv_heads), head_dim_(head_dim), position_(std::move(position)),
          qk_norm_(qk_norm_eps.has_value()), eps_(qk_norm_eps ? (float)*qk_norm_eps : 0.f), window_(window) {
        if (hidden <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0)
            fail(KIPP_E_CONFIG, "attention: sizes must be positive");
        if (heads % kv_heads) fail(KIPP_E_CONFIG, "attention: num_heads must be a multiple of num_kv_heads");
        if (window < 0) fail(KIPP_E_CONFIG, "attention: a window must not be negative");
        if (position_->rotary_dim() > head_dim || position_->rotary_dim() % 2)
            fail(KIPP_E_CONFIG, "attention: rotary_dim must be even and at most head_dim");
        scale_ = scale ? (float)*scale : (float)(1.0 / std::sqrt((double)head_dim));
        q_dim_ = heads * head_dim;
        kv_dim_ = kv_heads * head_dim;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* n, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + n;
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        add("q_proj.weight", {q_dim_, hidden_});
        add("k_proj.weight", {kv_dim_, hidden_});
        add("v_proj.weight", {kv_dim_, hidden_});
        add("o_proj.weight", {hidden_, q_dim_});
        if (qk_norm_) {
            add("q_norm.weight", {head_dim_}, "near_one");
            add("k_norm.weight", {head_dim_}, "near_one");
        }
        position_->tensor_specs(p, out);
    }
    std::optional<PagedKVSpec> cache_spec() const override { return PagedKVSpec{kv_heads_, head_dim_, window_}; }
    std::shared_ptr<WorkPlanner> planner(const DeviceInfo& dev, bool own_length) override {
        auto p = std::make_shared<AttentionPlanner>(kv_heads_, dev.sm_count, own_length);
        planner_ = p;
        return p;
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        const int64_t rows = q_dim_ + 2 * kv_dim_;
        // one matrix for q, k and v so that one product makes all three
        w_qkv_ = b.allocate((size_t)rows * hidden_ * es, p + "qkv");
        char* base = static_cast<char*>(w_qkv_);
        b.load(p + "q_proj.weight", base, dtype_, hidden_, q_dim_, hidden_);
        b.load(p + "k_proj.weight", base + (size_t)q_dim_ * hidden_ * es, dtype_, hidden_, kv_dim_, hidden_);
        b.load(p + "v_proj.weight", base + (size_t)(q_dim_ + kv_dim_) * hidden_ * es, dtype_, hidden_, kv_dim_,
               hidden_);
        w_o_ = b.allocate((size_t)hidden_ * q_dim_ * es, p + "o_proj.weight");
        b.load(p + "o_proj.weight", w_o_, dtype_, q_dim_, hidden_, q_dim_);
        if (qk_norm_) {
            int qd = storage_dtype(b.stored_dtype(p + "q_norm.weight"));
            int kd = storage_dtype(b.stored_dtype(p + "k_norm.weight"));
            norm_dtype_ = qd == kd ? qd : F32;
            q_norm_ = b.allocate((size_t)head_dim_ * dtype_size(norm_dtype_), p + "q_norm.weight");
            k_norm_ = b.allocate((size_t)head_dim_ * dtype_size(norm_dtype_), p + "k_norm.weight");
            b.load(p + "q_norm.weight", q_norm_, norm_dtype_, head_dim_, 1, head_dim_);
            b.load(p + "k_norm.weight", k_norm_, norm_dtype_, head_dim_, 1, head_dim_);
        }
        position_->bind(b, p);
    }
    size_t weight_bytes() const override {
        size_t n = ((size_t)(q_dim_ + 2 * kv_dim_) * hidden_ + (size_t)hidden_ * q_dim_) * dtype_size(dtype_);
        if (qk_norm_) n += 2 * (size_t)head_dim_ * dtype_size(norm_dtype_);
        return n;
    }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_qkv_, hidden_, w_qkv_, hidden_); }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override;

private:
    int hidden_, heads_, kv_heads_, head_dim_;
    std::unique_ptr<PositionEncoding> position_;
    bool qk_norm_;
    float eps_;
    int window_;
    float scale_ = 1.f;
    int q_dim_ = 0, kv_dim_ = 0, dtype_ = BF16, norm_dtype_ = F32;
    void *w_qkv_ = nullptr, *w_o_ = nullptr, *q_norm_ = nullptr, *k_norm_ = nullptr;
    std::shared_ptr<AttentionPlanner> planner_;
};

// Dense SwiGLU feed-forward: x += W_down (silu(W_gate n) * (W_up n)) (src/kipp.c:2994-3010,
// silu src/kipp.c:2402-2404).
class SwiGLUFeedForward : public FeedForward {
public:
    SwiGLUFeedForward(int hidden, int intermediate) : hidden_(hidden), inter_(intermediate) {
        if (hidden <= 0 || intermediate <= 0) fail(KIPP_E_CONFIG, "swiglu: sizes must be positive");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* n, std::vector<int64_t> shape) {
            TensorSpec s;
            s.name = p + n;
            s.shape = std::move(shape);
            out.push_back(s);
        };
        add("gate_proj.weight", {inter_, hidden_});
        add("up_proj.weight", {inter_, hidden_});
        add("down_proj.weight", {hidden_, inter_});
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // rows interleaved (gate_0, up_0, gate_1, up_1, ...): one product makes both, and a gate
        // sits beside its up value in the epilogue
        w_gate_up_ = b.allocate((size_t)2 * inter_ * hidden_ * es, p + "gate_up");
        char* base = static_cast<char*>(w_gate_up_);
        b.load(p + "gate_proj.weight", base, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
        b.load(p + "up_proj.weight", base + (size_t)hidden_ * es, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
        w_down_ = b.allocate((size_t)hidden_ * inter_ * es, p + "down_proj.weight");
        b.load(p + "down_proj.weight", w_down_, dtype_, inter_, hidden_, inter_);
    }
    size_t weight_bytes() const override { return (size_t)3 * inter_ * hidden_ * dtype_size(dtype_); }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_gate_up_, hidden_, w_gate_up_, hidden_); }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        const int T = ctx.tokens();
        NormFold in, out;
        void* act = ctx.workspace->buffer("ffn_act", (size_t)T * inter_ * ctx.element());
        ctx.ops->gemm(act, ctx.dtype, inter_, h, hidden_, w_gate_up_, hidden_, dtype_, T, 2 * inter_, hidden_,
                      EPI_SWIGLU, fold_input(ctx, in));
        const NormFold* emit = fold_emit(ctx, out, hidden_);
        ctx.ops->gemm(residual, F32, hidden_, act, inter_, w_down_, inter_, dtype_, T, hidden_, inter_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_, inter_, dtype_ = BF16;
    void *w_gate_up_ = nullptr, *w_down_ = nullptr;
};

// x += mixer(norm1(x)); x += ffn(norm2(x)): the un-normed x is the residual stream
// (src/kipp.c:2948, 2994).
class PreNormBlock : public Block {
public:
    PreNormBlock(std::unique_ptr<Norm> n1, std::unique_ptr<Mixer> mixer, std::unique_ptr<Norm> n2,
                 std::unique_ptr<FeedForward> ffn, std::vector<std::string> names)
        : n1_(std::move(n1)), mixer_(std::move(mixer)), n2_(std::move(n2)), ffn_(std::move(ffn)), names_(std::move(names)) {
        if (names_.size() != 4) fail(KIPP_E_CONFIG, "pre_norm_block: four name prefixes are needed");
        if (n1_->size() != n2_->size()) fail(KIPP_E_CONFIG, "pre_norm_block: the two norms differ in size");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        n1_->tensor_specs(p + names_[0], out);
        mixer_->tensor_specs(p + names_[1], out);
        n2_->tensor_specs(p + names_[2], out);
        ffn_->tensor_specs(p + names_[3], out);
    }
    void bind(Binder& b, const std::string& p) override {
        n1_->bind(b, p + names_[0]);
        mixer_->bind(b, p + names_[1]);
        n2_->bind(b, p + names_[2]);
        ffn_->bind(b, p + names_[3]);
    }
    size_t weight_bytes() const override {
        return n1_->weight_bytes() + mixer_->weight_bytes() + n2_->weight_bytes() + ffn_->weight_bytes();
    }
    bool graph_safe() const override {
        return n1_->graph_safe() && mixer_->graph_safe() && n2_->graph_safe() && ffn_->graph_safe();
    }
    std::vector<Mixer*> mixers() override { return {mixer_.get()}; }
    const Norm* deferred_first_norm() const override {
        return mixer_->folds_rms() && n1_->rms_spec() ? n1_.get() : nullptr;
    }
    // A plain RMSNorm before a part that folds it runs in deferred form, at every size of step:
    // the part's input is bf16(x * weight), the row factor goes into its first product.  In steps
    // of few tokens the residual add BEFORE the norm leaves that form itself (two launches fewer
    // per layer, where a launch costs more than the norm's arithmetic); otherwise one kernel makes
    // it.  Both give the same bits, so the logits do not depend on which ran.
    void forward(StepContext& ctx, const LayerRun& run, float* x) override {
        const int T = ctx.tokens();
        void* h = ctx.workspace->buffer("normed", (size_t)T * n1_->size() * ctx.element());
        const std::optional<RmsNormSpec> spec1 = n1_->rms_spec(), spec2 = n2_->rms_spec();
        const bool defer1 = spec1 && mixer_->folds_rms(), defer2 = spec2 && ffn_->folds_rms();
        // -- norm 1 and the mixer
        ctx.input_scale = RowScale{};
        if (defer1 && ctx.pending_norm == n1_.get()) ctx.input_scale = ctx.pending_scale;   // h is made already
        else if (defer1) ctx.input_scale = deferred_norm(ctx, *spec1, x, h);
        else n1_->forward(ctx, x, h, nullptr, T);
        ctx.pending_norm = nullptr;
        ctx.emit_for = defer2 ? &*spec2 : nullptr;
        ctx.emitted = false;
        mixer_->forward(ctx, run, 0, h, x);
        // -- norm 2 and the feed-forward
        ctx.input_scale = RowScale{};
        if (defer2 && ctx.emitted) ctx.input_scale = ctx.emitted_scale;
        else if (defer2) ctx.input_scale = deferred_norm(ctx, *spec2, x, h);
        else n2_->forward(ctx, x, h, nullptr, T);
        const Norm* next = ctx.following_norm;
        const std::optional<RmsNormSpec> spec_next = next ? next->rms_spec() : std::nullopt;
        ctx.emit_for = spec_next && ffn_->folds_rms() && next->size() == n1_->size() ? &*spec_next : nullptr;
        ctx.emitted = false;
        ffn_->forward(ctx, h, x);
        if (ctx.emitted) {
            ctx.pending_norm = next;
            ctx.pending_scale = ctx.emitted_scale;
        }
        ctx.input_scale = RowScale{};
        ctx.emit_for = nullptr;
        ctx.emitted = false;
    }
    Norm* input_norm() { return n1_.get(); }
    Norm* post_norm() { return n2_.get(); }
    FeedForward* feed_forward() { return ffn_.get(); }

private:
    std::unique_ptr<Norm> n1_;
    std::unique_ptr<Mixer> mixer_;
    std::unique_ptr<Norm> n2_;
    std::unique_ptr<FeedForward> ffn_;
    std::vector<std::string> names_;
};

// ---------------------------------------------------------------------------------------------
// Parts whose forward pass the caller supplies (kipp_external_part).  The plan declares what
// the engine has to know without calling them: their tensors (so that a checkpoint is checked
// as a whole), a mixer's per-request state, and whether a captured graph may hold their work.
struct ExternalCommon {
    kipp_external_part hook{};
    std::vector<TensorSpec> specs;
    bool graph_safe = false;
    int size = 0;

    void read(const Json& j, const BuildContext& ctx) {
        const long long index = j.get("index").as_int();
        if (index < 0 || index >= ctx.n_external || !ctx.external || !ctx.external[index].forward)
            fail(KIPP_E_CONFIG, format("the plan names external part %lld, which the caller did not supply", index));
        hook = ctx.external[index];
        if (const Json* t = j.find("tensors"))
            for (auto& s : t->items()) specs.push_back(TensorSpec::from_json(s));
        graph_safe = j.get_bool("graph_safe", false);
        size = (int)j.get_int("size", 0);
    }
    void fill(kipp_external_call& c, StepContext& ctx, int role) const {
        const StepMeta& m = *ctx.meta;
        c = kipp_external_call{};
        c.role = role;
        c.tokens = m.shape.tokens;
        c.entries = m.shape.entries;
        c.token_ids = m.token_ids;
        c.positions = m.positions;
        c.entry_of_token = m.entry_of_token;
        c.q_start = m.q_start;
        c.context_len = m.context_len;
        c.slots = m.slots;
        c.host_q_lens = m.shape.q_lens.data();
        c.host_context_len = m.shape.starts.data();
        c.host_slots = m.shape.slots.data();
        c.input_dtype = ctx.dtype;
        c.max_requests = ctx.max_requests();
        c.stream = ctx.stream;
    }
    void call(const kipp_external_call& c, const char* what) const {
        const int rc = hook.forward(hook.user, &c);
        if (rc) fail(KIPP_E_KERNEL, format("the external %s failed with code %d", what, rc));
    }
};

class ExternalMixer : public Mixer {
public:
    ExternalMixer(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        hidden_ = j.get("hidden_size").as_int();
        if (const Json* s = j.find("state"); s && !s->is_null()) {
            StateSpec spec;
            for (auto& d : s->get("shape").items()) spec.shape.push_back(d.as_int());
            const std::string dt = s->get_string("dtype", "float32");
            spec.dtype = dt == "float32" ? F32 : dt == "bfloat16" ? BF16 : dt == "int32" ? I32 : -1;
            if (spec.dtype < 0) fail(KIPP_E_CONFIG, "external mixer: state dtype must be float32, bfloat16 or int32");
            state_ = spec;
        }
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    std::optional<StateSpec> state_spec() const override { return state_; }
    bool graph_safe() const override { return common_.graph_safe; }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        kipp_external_call c;
        common_.fill(c, ctx, 2);
        c.layer = run.layer;
        c.cache = run.cache;
        c.writes_cache = run.writes_cache ? 1 : 0;
        c.input = h;
        c.input_cols = hidden_;
        c.residual = residual;
        c.hidden = hidden_;
        if (state_) {
            size_t bytes = 0;
            c.state = ctx.state_view(run, mixer_slot, &bytes);
            c.state_bytes = (long long)bytes;
        }
        common_.call(c, "mixer");
    }

private:
    ExternalCommon common_;
    long long hidden_ = 0;
    std::optional<StateSpec> state_;
};

class ExternalFeedForward : public FeedForward {
public:
    ExternalFeedForward(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        hidden_ = j.get("hidden_size").as_int();
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    bool graph_safe() const override { return common_.graph_safe; }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        kipp_external_call c;
        common_.fill(c, ctx, 3);
        c.input = h;
        c.input_cols = hidden_;
        c.residual = residual;
        c.hidden = hidden_;
        common_.call(c, "feed-forward");
    }

private:
    ExternalCommon common_;
    long long hidden_ = 0;
};

class ExternalEmbeddingStage : public EmbeddingStage {
public:
    ExternalEmbeddingStage(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        hidden_ = j.get("hidden_size").as_int();
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    bool graph_safe() const override { return common_.graph_safe; }
    void forward(StepContext& ctx, float* x) override {
        kipp_external_call c;
        common_.fill(c, ctx, 0);
        c.residual = x;
        c.hidden = hidden_;
        common_.call(c, "embedding stage");
    }

private:
    ExternalCommon common_;
    long long hidden_ = 0;
};

class ExternalNorm : public Norm {
public:
    ExternalNorm(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        if (common_.size <= 0) fail(KIPP_E_CONFIG, "external norm: 'size' is needed");
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    bool graph_safe() const override { return common_.graph_safe; }
    int size() const override { return common_.size; }
    void forward(StepContext& ctx, const float* x, void* out, const int* rows, int n_rows) override {
        kipp_external_call c;
        common_.fill(c, ctx, 1);
        c.residual = const_cast<float*>(x);
        c.hidden = common_.size;
        c.output = out;
        c.rows = rows;
        c.n_rows = n_rows;
        common_.call(c, "norm");
    }

private:
    ExternalCommon common_;
};

// ---------------------------------------------------------------------------------------------
inline std::unique_ptr<PositionEncoding> make_position(const Json& j, const BuildContext& ctx) {
    return Registry::get().make_as<PositionEncoding>(j, ctx, "a position encoding");
}

inline void register_builtin_parts() {
    Registry& r = Registry::get();
    r.add_part_kind("token_embedding", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<TokenEmbedding>((int)j.get("vocab_size").as_int(), (int)j.get("hidden_size").as_int());
    });
    r.add_part_kind("output_head", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<OutputHead>((int)j.get("vocab_size").as_int(), (int)j.get("hidden_size").as_int(),
                                            j.get_string("tied_to", ""));
    });
    r.add_part_kind("rmsnorm", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<RMSNorm>((int)j.get("size").as_int(), j.get("eps").as_double(),
                                         j.get_string("weight_name", "weight"));
    });
    r.add_part_kind("rotary", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        const int head_dim = (int)j.get("head_dim").as_int();
        const int rot = (int)j.get_int("rotary_dim", head_dim);
        const double theta = j.get("theta").as_double();
        if (rot % 2 || rot < 0 || rot > head_dim)
            fail(KIPP_E_CONFIG, format("rotary_dim %d must be even and at most head_dim %d", rot, head_dim));
        if (!(theta > 0)) fail(KIPP_E_CONFIG, "rotary: theta must be positive");
        return std::make_unique<FrequencyTable>(rotary_frequencies(rot, theta),
                                                format("rotary/%.17g/%d", (double)(float)theta, rot));
    });
    r.add_part_kind("frequency_table", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        std::vector<float> f;
        for (auto& v : j.get("inv_freq").items()) f.push_back((float)v.as_double());
        return std::make_unique<FrequencyTable>(std::move(f), j.get("key").as_string());
    });
    r.add_part_kind("no_position", [](const Json&, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<FrequencyTable>(std::vector<float>{}, "none");
    });
    r.add_part_kind("attention", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        std::optional<double> eps, scale;
        if (const Json* e = j.find("qk_norm_eps"); e && !e->is_null()) eps = e->as_double();
        if (const Json* s = j.find("scale"); s && !s->is_null()) scale = s->as_double();
        return std::make_unique<AttentionMixer>(
            (int)j.get("hidden_size").as_int(), (int)j.get("num_heads").as_int(), (int)j.get("num_kv_heads").as_int(),
            (int)j.get("head_dim").as_int(), make_position(j.get("position"), ctx), eps, (int)j.get_int("window", 0),
            scale);
    });
    r.add_part_kind("swiglu", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<SwiGLUFeedForward>((int)j.get("hidden_size").as_int(),
                                                   (int)j.get("intermediate_size").as_int());
    });
    r.add_part_kind("pre_norm_block", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        const Registry& reg = Registry::get();
        std::vector<std::string> names;
        for (auto& n : j.get("names").items()) names.push_back(n.as_string());
        return std::make_unique<PreNormBlock>(reg.make_as<Norm>(j.get("input_norm"), ctx, "a norm"),
                                              reg.make_as<Mixer>(j.get("mixer"), ctx, "a mixer"),
                                              reg.make_as<Norm>(j.get("post_norm"), ctx, "a norm"),
                                              reg.make_as<FeedForward>(j.get("ffn"), ctx, "a feed-forward"), names);
    });
    r.add_part_kind("external", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        const std::string role = j.get("role").as_string();
        if (role == "mixer") return std::make_unique<ExternalMixer>(j, ctx);
        if (role == "feed_forward") return std::make_unique<ExternalFeedForward>(j, ctx);
        if (role == "embedding") return std::make_unique<ExternalEmbeddingStage>(j, ctx);
        if (role == "norm") return std::make_unique<ExternalNorm>(j, ctx);
        fail(KIPP_E_CONFIG, "external part: role must be mixer, feed_forward, embedding or norm, not '" + role + "'");
    });
}

}  // namespace kipp
