// The kernels as the host core calls them: typed wrappers over the `extern "C"` launchers of
// the kernel libraries, and the choice between kernels where several can do an operation
// (tensor-core or CUDA-core product; tcgen05, mma.sync or CUDA-core attention).  The Python
// package's kernel functions call the same launchers.
//
// No sizes of a model and no property of the device stand here as constants: tile sizes and
// split rules belong to the attention kernels and are kept beside them (AttentionPlanner).
#pragma once
#include <algorithm>
#include <cmath>

#include "runtime.hpp"

namespace kipp {

enum Epilogue : int { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };

// The work lists of the paged attention kernels for one step (device pointers into the
// step's metadata) and what the host needs to choose a kernel.
struct AttentionWork {
    const int* decode_rows = nullptr;      // [n_decode] entries that bring one token
    int n_decode = 0;
    const int* split_keys = nullptr;       // [n_decode] keys per split of each decoded token
    int stream_ctas = 0;                   // > 0: the decoded tokens' key tiles are dealt out in equal runs to
                                           // that many CTAs instead (split_keys is not read)
    const int* prefill_work = nullptr;     // [(entry, first token)] per 64-token tile, entries of > 1 token
    int n_prefill_items = 0;
    const int* all_work = nullptr;         // the same over every entry
    int n_all_items = 0;
    const int* prefill_work128 = nullptr;  // per 128-token tile, entries of > 1 token
    int n_prefill_items128 = 0;
    int longest_portion = 0;               // most tokens an entry of > 1 token brings
    int entries = 0, tokens = 0;
};

// Folding an RMSNorm into the products around it (kipp_gemm_tc_fold, few-token kernel): a residual
// add leaves what the NEXT norm needs (xn = bf16(new residual x norm_w), sums of squares per 32
// features in ssq_out); a store or SwiGLU product whose input lacks the norm's per-token factor
// takes it from such sums (ssq_in).  The layout is the kernel library's kipp_gemm_norm_fold.
struct NormFold {
    const void* norm_w = nullptr;
    int norm_w_dtype = 0;
    void* xn = nullptr;
    long long ldn = 0;
    float* ssq_out = nullptr;
    const float* ssq_in = nullptr;
    int ssq_in_slots = 0;
    float inv_n = 0.f, eps = 0.f;
};

// Where the rows of a fused q/k/v projection go when they skip the stored product
// (kipp_gemm_tc_heads): per-head norm, rotation, queries to q_out, keys and values into the pages.
// The layout is the kernel library's kipp_gemm_head_sink.
struct HeadSink {
    void* q_out = nullptr;
    void* k_pages = nullptr;
    void* v_pages = nullptr;
    const void* q_norm_w = nullptr;
    const void* k_norm_w = nullptr;
    int norm_dtype = 0;
    float eps = 0.f;
    const void* cos_sin = nullptr;
    const int* positions = nullptr;
    const int* entry_of_token = nullptr;
    const int* block_table = nullptr;
    int table_width = 0, page_size = 0, n_q = 0, n_kv = 0, write_cache = 0;
};

struct PagedCacheView {
    void* k_pages = nullptr;               // [pages, kv_heads, page_size, head_dim] of one run's cache
    void* v_pages = nullptr;
    int n_pages = 0;
    const int* block_table = nullptr;      // int32 [entries, table_width] of this step
    int table_width = 0;
    int page_size = 0;
};

class Ops {
public:
    cudaStream_t stream = nullptr;
    int* status = nullptr;                 // int32[4] on the device: what kernels refused or gave up
    Workspace* workspace = nullptr;
    long long launches = 0;                // kernels of this package launched through this object
    bool prefill_tensor_core = true;       // prompt portions on tcgen05 where the sizes allow

    static constexpr int DECODE_MAX_SPLITS = 32;
    static constexpr int PREFILL_TC_MIN_TOKENS = 64;   // shorter portions waste a 128-row tile

    void embed_gather(float* out, const void* table, int table_dtype, const int* ids, int tokens, int hidden,
                      int vocab) {
        using Fn = int (*)(float*, const void*, int, const int*, int, int, int, int*, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_embed_gather");
        run(f(out, table, table_dtype, ids, tokens, hidden, vocab, status, stream), "embed_gather");
    }

    // out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight, float32 arithmetic.
    void rmsnorm(void* out, int out_dtype, const float* x, const void* weight, int weight_dtype, const int* rows,
                 int n_rows, int size, float eps) {
        using Fn = int (*)(void*, int, const float*, const void*, int, const int*, int, int, float, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_rmsnorm");
        run(f(out, out_dtype, x, weight, weight_dtype, rows, n_rows, size, eps, stream), "rmsnorm");
    }

    static bool gemm_tc_ok(int dtype, const void* a, long long lda, const void* w, long long ldw) {
        return dtype == BF16 && lda % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0;
    }

    // out = a @ w^T with float32 accumulation; a [M, K] (lda), w [N, K] (ldw), both of `dtype`.
    // EPI_STORE: out[M, N]; EPI_ADD: float32 out[M, N] += product; EPI_SWIGLU: out[M, N/2] =
    // silu(p[:, 0::2]) * p[:, 1::2].  float32 runs on the CUDA cores, bfloat16 on the tensor-core
    // kernel where it takes the operands.
    // Whether a product of these operands can scale its result rows (NormFold::ssq_in): the
    // tensor-core kernels do, at every number of rows.
    static bool gemm_scale_ok(int dtype, const void* a, long long lda, const void* w, long long ldw) {
        return gemm_tc_ok(dtype, a, lda, w, ldw);
    }
    // Whether a residual add of M rows can leave what the next norm needs (NormFold::norm_w), and
    // should: measured on a 36-layer, 2,560-wide model the two launches saved per layer are 3-4 %
    // of a decode step of 1 to 8 tokens, 0.6 % at 32, and at 64 the epilogue's extra work per
    // token costs 0.4 % more than they save.
    static constexpr int EMIT_PAYS_UP_TO = 32;
    static bool gemm_emit_ok(int M) {
        using Fn = int (*)(int);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_fold_ok");
        return M <= EMIT_PAYS_UP_TO && f(M) != 0;
    }

    // x * w rounded to out's type and the rows' sums of squares: the norm with its per-row factor
    // left to the product that follows (see NormFold).
    void rmsnorm_deferred(void* out, int out_dtype, float* ssq, const float* x, const void* w, int w_dtype,
                          const int* rows, int n_rows, int size) {
        using Fn = int (*)(void*, int, float*, const float*, const void*, int, const int*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_rmsnorm_deferred");
        run(f(out, out_dtype, ssq, x, w, w_dtype, rows, n_rows, size, stream), "rmsnorm_deferred");
    }

    void gemm(void* out, int out_dtype, long long ldc, const void* a, long long lda, const void* w, long long ldw,
              int dtype, int M, int N, int K, Epilogue epilogue, const NormFold* fold = nullptr) {
        if (M <= 0 || N <= 0) return;
        if (fold != nullptr && !(gemm_scale_ok(dtype, a, lda, w, ldw) && (fold->norm_w == nullptr || gemm_emit_ok(M))))
            fail(KIPP_E_STATE, "a product was asked to fold a norm that its kernel cannot fold");   // parts ask first
        if (gemm_tc_ok(dtype, a, lda, w, ldw)) {
            using Fn = int (*)(void*, int, const void*, const void*, int, int, int, long long, long long, long long, int,
                               int, int, int, const NormFold*, int*, void*);
            static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_fold");
            run(f(out, out_dtype, a, w, M, N, K, lda, ldw, ldc, (int)epilogue, 0, 0, 0, fold, status, stream), "gemm_tc", 1,
                profiling ? format("gemm_tc %d x %d", N, K).c_str() : nullptr);
            if (fold != nullptr && fold->ssq_in != nullptr) ++folded_norms;
        } else {
            using Fn = int (*)(void*, int, const void*, const void*, int, int, int, int, int, int, int, int, void*);
            static Fn f = kernel_symbol<Fn>("gemm_simt", "kipp_gemm_simt");
            run(f(out, out_dtype, a, w, dtype, M, N, K, (int)lda, (int)ldw, (int)ldc, (int)epilogue, stream),
                "gemm_simt");
        }
    }

    // Whether the fused q/k/v projection of a step can do per-head norm, rotation and the cache
    // write in its own epilogue (projection_to_heads) instead of storing the product.
    static bool projection_to_heads_ok(int dtype, const void* a, long long lda, const void* w, long long ldw, int M,
                                       int head_dim, int rotary_dim) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_heads_ok");
        return gemm_tc_ok(dtype, a, lda, w, ldw) && f(M, head_dim, rotary_dim) != 0;
    }
    // a [M, K] x w [(n_q + 2 n_kv) head_dim, K]^T with what qk_norm_rope_write does to the product
    // in the epilogue (the same bits); `fold` may carry the row factors of a deferred norm, and
    // `cos_sin` is the step's rope_table_by_pair.
    void projection_to_heads(const void* a, long long lda, const void* w, long long ldw, int M, int N, int K,
                             const NormFold* fold, const PagedCacheView& cache, void* q_out, const void* q_norm_w,
                             const void* k_norm_w, int norm_dtype, float eps, const float* cos_sin,
                             const int* positions, const int* entry_of_token, int n_q, int n_kv, bool write_cache) {
        HeadSink sink;
        sink.q_out = q_out; sink.k_pages = cache.k_pages; sink.v_pages = cache.v_pages;
        sink.q_norm_w = q_norm_w; sink.k_norm_w = k_norm_w; sink.norm_dtype = norm_dtype; sink.eps = eps;
        sink.cos_sin = cos_sin; sink.positions = positions; sink.entry_of_token = entry_of_token;
        sink.block_table = cache.block_table; sink.table_width = cache.table_width; sink.page_size = cache.page_size;
        sink.n_q = n_q; sink.n_kv = n_kv; sink.write_cache = write_cache ? 1 : 0;
        using Fn = int (*)(const void*, const void*, int, int, int, long long, long long, const NormFold*,
                           const HeadSink*, int*, void*);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_heads");
        run(f(a, w, M, N, K, lda, ldw, fold, &sink, status, stream), "gemm_tc_heads", 1,
            profiling ? format("gemm_tc %d x %d to heads", N, K).c_str() : nullptr);
        if (fold != nullptr && fold->ssq_in != nullptr) ++folded_norms;
        ++projections_to_heads;
    }

    // float32 [tokens, half, 2]: (cos, sin) of position * inv_freq, made once per step.
    void rope_table(float* out, const int* positions, const float* inv_freq, int tokens, int half) {
        using Fn = int (*)(void*, const int*, const float*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("rope_cache", "kipp_rope_table");
        run(f(out, positions, inv_freq, tokens, half, stream), "rope_table");
    }
    // The same values as float32 [half, tokens, 2], as projection_to_heads reads them.
    void rope_table_by_pair(float* out, const int* positions, const float* inv_freq, int tokens, int half) {
        using Fn = int (*)(void*, const int*, const float*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("rope_cache", "kipp_rope_table_by_pair");
        run(f(out, positions, inv_freq, tokens, half, stream), "rope_table");
    }

    // Per-head RMSNorm of q and k, rotation, q to q_out [T, n_q, D], k and v into the pages.
    // write_cache: bit 0 write keys and values, bit 1 round them to bfloat16 first (32-bit cache).
    void qk_norm_rope_write(const void* qkv, int ld_qkv, void* q_out, const PagedCacheView& cache, int dtype,
                            const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps, const float* cos_sin,
                            int rotary_dim, const int* positions, const int* entry_of_token, int tokens, int n_q,
                            int n_kv, int head_dim, int write_cache) {
        using Fn = int (*)(const void*, int, void*, void*, void*, int, const void*, const void*, int, float, const void*,
                           int, const int*, const int*, const int*, int, int, int, int, int, int, int, int*, void*);
        static Fn f = kernel_symbol<Fn>("rope_cache", "kipp_qk_norm_rope_write");
        run(f(qkv, ld_qkv, q_out, cache.k_pages, cache.v_pages, dtype, q_norm_w, k_norm_w, norm_dtype, eps, cos_sin,
              cos_sin ? rotary_dim : 0, positions, entry_of_token, cache.block_table, cache.table_width,
              cache.page_size, tokens, n_q, n_kv, head_dim, write_cache, status, stream),
            "qk_norm_rope_write");
    }

    static bool attention_mma_supported(int head_dim, int n_q, int n_kv) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_mma_supported");
        return f(head_dim, n_q, n_kv) != 0;
    }
    static bool attention_decode_supported(int head_dim, int n_q, int n_kv) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_supported");
        return f(head_dim, n_q, n_kv) != 0;
    }
    static bool attention_tc_supported(int head_dim, int n_q, int n_kv, int page_size) {
        using Fn = int (*)(int, int, int);
        using Fp = int (*)(int);
        static Fn f = kernel_symbol<Fn>("attention_tc", "kipp_attn_prefill_tc_supported");
        static Fp g = kernel_symbol<Fp>("attention_tc", "kipp_attn_prefill_tc_page_ok");
        return f(head_dim, n_q, n_kv) != 0 && g(page_size) != 0;
    }

    // The stream cut of a step's decoded tokens, where the planner asks for it and the kernel takes the step.
    static bool decode_stream_ok(int n_decode) {
        using Fn = int (*)(int, int);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_stream_ok");
        return f(n_decode, DECODE_MAX_SPLITS) != 0;
    }
    static int decode_stream_ctas(const AttentionWork& work) {
        return work.stream_ctas > 0 && decode_stream_ok(work.n_decode) ? work.stream_ctas : 0;
    }

    float* decode_scratch(int n, int n_q, int head_dim) {
        size_t floats = (size_t)n * n_q * DECODE_MAX_SPLITS * (head_dim + 2) + (size_t)n * n_q;
        if (floats < (1u << 20)) floats = 1u << 20;
        return workspace->get<float>("attention_decode_scratch", floats);
    }
    // Causal grouped-query attention of the step's tokens over the paged cache.
    void attention(void* out, const void* q, const PagedCacheView& cache, int dtype, const AttentionWork& work,
                   const int* positions, const int* entry_of_token, const int* q_start, const int* context_len,
                   int n_q, int n_kv, int head_dim, float scale, int window) {
        if (dtype == BF16 && attention_mma_supported(head_dim, n_q, n_kv)) {
            attention_tensor_core(out, q, cache, work, q_start, context_len, n_q, n_kv, head_dim, scale, window);
            return;
        }
        using Fn = int (*)(void*, const void*, const void*, const void*, int, const int*, const int*, const int*, int,
                           int, int, int, int, int, float, int, int*, void*);
        static Fn f = kernel_symbol<Fn>("attention_simt", "kipp_paged_attention_simt");
        run(f(out, q, cache.k_pages, cache.v_pages, dtype, positions, entry_of_token, cache.block_table,
              cache.table_width, cache.page_size, work.tokens, n_q, n_kv, head_dim, scale, window, status, stream),
            "attention_simt");
    }

    // Whether a step can take attention_decode_fused: decoded tokens only, bfloat16, a head size
    // and group the split-K kernel takes, the whole head rotated or none of it.
    static bool attention_decode_fused_ok(const AttentionWork& work, int dtype, int n_q, int n_kv, int head_dim,
                                          int rotary_dim) {
        return dtype == BF16 && work.n_decode > 0 && work.n_decode == work.entries && work.entries == work.tokens &&
               (rotary_dim == 0 || rotary_dim == head_dim) && attention_mma_supported(head_dim, n_q, n_kv) &&
               attention_decode_supported(head_dim, n_q, n_kv);
    }

    // qk_norm_rope_write and attention of a step of decoded tokens in one pair of launches: the
    // attention kernel normalises and rotates the raw queries and the new key itself and writes
    // the new key and value into the pages.
    void attention_decode_fused(void* out, const void* qkv, long long ld_qkv, const PagedCacheView& cache,
                                const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps,
                                const float* cos_sin, bool write_cache, const AttentionWork& work, const int* q_start,
                                const int* context_len, int n_q, int n_kv, int head_dim, float scale, int window) {
        using Fn = int (*)(void*, const void*, long long, void*, void*, const void*, const void*, int, float, const void*,
                           int, const int*, const int*, const int*, int, int, const int*, int, int, int, int, float, int,
                           int, const int*, int, int, float*, int*, void*);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_mma_fused");
        float* scratch = decode_scratch(work.n_decode, n_q, head_dim);
        run(f(out, qkv, ld_qkv, cache.k_pages, cache.v_pages, q_norm_w, k_norm_w, norm_dtype, eps, cos_sin,
              write_cache ? 1 : 0, q_start, context_len, cache.block_table, cache.table_width, cache.page_size,
              work.decode_rows, work.n_decode, n_q, n_kv, head_dim, scale, window, DECODE_MAX_SPLITS, work.split_keys, 1,
              decode_stream_ctas(work), scratch, status, stream),
            "attn_decode_mma_fused", 2);
        ++fused_decode_launches;
        if (decode_stream_ctas(work) > 0) ++stream_decode_launches;
    }

    // The first maximum of each row; long rows are shared among blocks (two launches then).
    void argmax_rows(const float* logits, long long ld, int rows, int n, int* out) {
        using Fn = int (*)(const float*, long long, int, int, int*, void*, long long, void*);
        using Fb = long long (*)(int, int);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_argmax_rows_split");
        static Fb bytes = kernel_symbol<Fb>("sampling", "kipp_argmax_scratch_bytes");
        const long long need = bytes(rows, n);
        void* scratch = need > 0 ? workspace->buffer("argmax_parts", (size_t)need) : nullptr;
        run(f(logits, ld, rows, n, out, scratch, need, stream), "argmax_rows", need > 0 ? 2 : 1);
    }
    void sample_rows(const float* logits, long long ld, int rows, int n, const float* temperature, const int* top_k,
                     const float* top_p, const float* min_p, const double* uniform, int* out) {
        using Fn = int (*)(const float*, long long, int, int, const float*, const int*, const float*, const float*,
                           const double*, int*, void*);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_sample_rows");
        run(f(logits, ld, rows, n, temperature, top_k, top_p, min_p, uniform, out, stream), "sample_rows");
    }
    void apply_penalties(float* logits, long long ld, int rows, int n, const int* recent, int recent_width,
                         const int* recent_count, const float* repetition, const float* presence,
                         const float* frequency, const int* bias_tokens, const float* bias_values, int bias_width,
                         const int* bias_count) {
        using Fn = int (*)(float*, long long, int, int, const int*, int, const int*, const float*, const float*,
                           const float*, const int*, const float*, int, const int*, void*);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_apply_penalties");
        run(f(logits, ld, rows, n, recent, recent_width, recent_count, repetition, presence, frequency, bias_tokens,
              bias_values, bias_width, bias_count, stream),
            "apply_penalties");
    }
    // Between two greedy decode steps on the device: `next` become the step's tokens and row
    // *counter of `ring`, positions and cached lengths move on by one.
    void burst_advance(int* tokens, int* positions, int* context_len, const int* next, int* ring, int* counter, int n,
                       int ring_rows) {
        using Fn = int (*)(int*, int*, int*, const int*, int*, int*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_burst_advance");
        run(f(tokens, positions, context_len, next, ring, counter, n, ring_rows, stream), "burst_advance");
    }
    // The keys per split of every decoded token, chosen on the device for the lengths a
    // burst_advance left, by AttentionPlanner's rule.
    void decode_replan(int* split_keys, const int* context_len, const int* rows, int n, int pairs_per_entry,
                       int resident_ctas, int fixed_tiles, int max_splits, int own_length) {
        using Fn = int (*)(int*, const int*, const int*, int, int, int, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_replan");
        run(f(split_keys, context_len, rows, n, pairs_per_entry, resident_ctas, fixed_tiles, max_splits, own_length,
              stream),
            "attn_decode_replan");
    }
    void convert_rows(void* dst, int dst_dtype, long long dst_pitch, const void* src, int src_dtype,
                      long long src_pitch, long long rows, long long cols) {
        using Fn = int (*)(void*, int, long long, const void*, int, long long, long long, long long, void*);
        static Fn f = kernel_symbol<Fn>("convert", "kipp_convert_rows");
        run(f(dst, dst_dtype, dst_pitch, src, src_dtype, src_pitch, rows, cols, stream), "convert_rows");
    }

private:
    void run(int code, const char* what, int kernels = 1, const char* label = nullptr) {
        kernel_check(code, what);
        launches += kernels;
        if (profiling) mark(label ? label : what);
    }

    void attention_tensor_core(void* out, const void* q, const PagedCacheView& cache, const AttentionWork& work,
                               const int* q_start, const int* context_len, int n_q, int n_kv, int head_dim,
                               float scale, int window) {
        const bool use_decode = work.n_decode > 0 && attention_decode_supported(head_dim, n_q, n_kv);
        const int* tiles = use_decode ? work.prefill_work : work.all_work;
        const int items = use_decode ? work.n_prefill_items : work.n_all_items;
        const bool aligned = (((uintptr_t)out | (uintptr_t)q | (uintptr_t)cache.k_pages | (uintptr_t)cache.v_pages) &
                              15) == 0;
        if (prefill_tensor_core && work.n_prefill_items128 > 0 && work.longest_portion >= PREFILL_TC_MIN_TOKENS &&
            (use_decode || work.n_decode == 0) && aligned &&
            attention_tc_supported(head_dim, n_q, n_kv, cache.page_size)) {
            using Fn = int (*)(void*, const void*, int, const void*, const void*, int, const int*, const int*, const int*,
                               int, int, const int*, int, int, int, int, float, int, int*, void*);
            static Fn f = kernel_symbol<Fn>("attention_tc", "kipp_attn_prefill_tc");
            run(f(out, q, work.tokens, cache.k_pages, cache.v_pages, cache.n_pages, q_start, context_len, cache.block_table,
                  cache.table_width, cache.page_size, work.prefill_work128, work.n_prefill_items128, n_q, n_kv,
                  head_dim, scale, window, status, stream),
                "attn_prefill_tc");
            ++tc_prefill_launches;
        } else if (items > 0) {
            using Fn = int (*)(void*, const void*, const void*, const void*, const int*, const int*, const int*, int, int,
                               const int*, int, int, int, int, float, int, void*);
            static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_prefill_mma");
            run(f(out, q, cache.k_pages, cache.v_pages, q_start, context_len, cache.block_table, cache.table_width,
                  cache.page_size, tiles, items, n_q, n_kv, head_dim, scale, window, stream),
                "attn_prefill_mma");
        }
        if (use_decode) {
            using Fn = int (*)(void*, const void*, const void*, const void*, const int*, const int*, const int*, int, int,
                               const int*, int, int, int, int, float, int, int, const int*, int, int, float*, void*);
            static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_mma");
            float* scratch = decode_scratch(work.n_decode, n_q, head_dim);
            run(f(out, q, cache.k_pages, cache.v_pages, q_start, context_len, cache.block_table, cache.table_width,
                  cache.page_size, work.decode_rows, work.n_decode, n_q, n_kv, head_dim, scale, window,
                  DECODE_MAX_SPLITS, work.split_keys, 1, decode_stream_ctas(work), scratch, stream),
                "attn_decode_mma", 2);
        }
    }

public:
    // Where a step's time goes: while `profiling` is set every launch is followed by an event on
    // the stream; profile_stop() waits for them and gives the time between consecutive events
    // per kernel name in milliseconds (steps run without graphs meanwhile, so gaps between
    // launches are part of the figures: read them as shares).
    bool profiling = false;
    void profile_start() {
        profile_clear();
        profiling = true;
        mark("(start)");
    }
    std::vector<std::pair<std::string, double>> profile_stop() {
        profiling = false;
        std::vector<std::pair<std::string, double>> out;
        if (!marks_.empty()) cuda_check(cudaEventSynchronize(marks_.back().second), "profile events");
        for (size_t i = 1; i < marks_.size(); ++i) {
            float ms = 0.f;
            cuda_check(cudaEventElapsedTime(&ms, marks_[i - 1].second, marks_[i].second), "profile events");
            bool found = false;
            for (auto& kv : out)
                if (kv.first == marks_[i].first) { kv.second += ms; found = true; break; }
            if (!found) out.emplace_back(marks_[i].first, (double)ms);
        }
        profile_clear();
        return out;
    }
    ~Ops() { profile_clear(); }

private:
    std::vector<std::pair<std::string, cudaEvent_t>> marks_;
    void mark(const std::string& what) {
        cudaEvent_t ev = nullptr;
        cuda_check(cudaEventCreate(&ev), "profile event");
        cuda_check(cudaEventRecord(ev, (cudaStream_t)stream), "profile event");
        marks_.emplace_back(what, ev);
    }
    void profile_clear() {
        for (auto& m : marks_) cudaEventDestroy(m.second);
        marks_.clear();
    }

public:
    long long tc_prefill_launches = 0;      // launches of the tcgen05 prompt attention (tests look at it)
    long long fused_decode_launches = 0;
    long long folded_norms = 0;          // norms that ran inside the products around them
    long long stream_decode_launches = 0;   // decode attention dealt out as a stream
    long long projections_to_heads = 0;     // q/k/v projections with norm, rotation and cache write inside
};

}  // namespace kipp
