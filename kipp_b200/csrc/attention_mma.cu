// bfloat16 attention over the paged cache on the tensor cores: a flash-style
// kernel for prompt portions and a split-K kernel for single decoded tokens.
//
// Reference counterpart: cached_gqa_kernel (cuda/kipp_kernels.cu:160), which
// walks the keys one by one with block-wide reductions and a serial softmax;
// the formula is src/kipp.c:2882-2922 (scores (q.k)/sqrt(D) over the keys the
// token may see, softmax with the maximum subtracted, weighted sum of values,
// kv head = q head / group).  The split over keys with a final merge follows
// the idea of the reference's Metal kernels (metal/kipp_kernels.metal:517-626,
// 741-779).  The split length is a parameter of the step, read from device
// memory so that a captured graph follows it; partial results are merged in
// split order.
//
// Both kernels: keys and values are gathered page by page with cp.async into
// shared memory (16-byte chunks, XOR-swizzled rows), scores and the weighted
// sum run on mma.sync m16n8k16 (bf16 in, float32 accumulate), maxima, sums and
// the rescaling are float32.  tcgen05 is not used here: with 4 to 16 query rows
// per key (decode) the tensor memory round trip costs more than it saves, and
// the decode kernel is bound by HBM reads.
//
// Cache layout of one layer: [page][kv_head][slot][head_dim].
#include "common.cuh"
#include <math.h>

namespace {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int TILE_KEYS = 64;
#ifndef KIPP_DECODE_STAGES
#define KIPP_DECODE_STAGES 2
#endif
constexpr int DECODE_STAGES = KIPP_DECODE_STAGES;      // K/V tiles in flight per CTA

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
// 16-byte asynchronous copy; src_bytes == 0 fills the destination with zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a swizzled tile whose
// rows hold D bf16 (D * 2 bytes, at least 128).
template <int D> __device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

// Gathers TILE_KEYS rows of keys and of values, positions [j0, j0 + TILE_KEYS),
// for kv head g into swizzled tiles.  Rows outside [lo, hi] are zero-filled
// (their scores are masked; zero values keep 0 * v finite).  A thread copies
// one 16-byte column of 8 consecutive rows (or of every 8th row when a row
// holds 8 chunks); when the page size is a multiple of 8 those rows lie in
// one page and the page is looked up once.
template <int D>
__device__ __forceinline__ void load_kv_tile(uint32_t k_tile, uint32_t v_tile, const bf16* __restrict__ k_pages,
                                             const bf16* __restrict__ v_pages, const int* __restrict__ table,
                                             int table_width, int page_size, int n_kv, int g, int j0, int lo,
                                             int hi) {
    constexpr int CHUNKS = D / 8;                        // 16-byte chunks per row
    constexpr int GROUPS = THREADS / CHUNKS;             // threads along the rows
    constexpr int ROWS = TILE_KEYS / GROUPS;             // consecutive rows per thread
    const int chunk = threadIdx.x % CHUNKS, row0 = (threadIdx.x / CHUNKS) * ROWS;
    if ((page_size & 7) == 0 && ROWS <= 8) {
        const int j_first = j0 + row0;
        const int slot = j_first / page_size;
        const int within = j_first - slot * page_size;
        const int page = (slot < table_width && j_first <= hi && j_first + ROWS - 1 >= lo)
                             ? __ldg(table + slot) : -1;
        const size_t base = (((size_t)max(page, 0) * n_kv + g) * page_size + within) * D + chunk * 8;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int j = j_first + r;
            const bool ok = page >= 0 && j >= lo && j <= hi;
            const size_t src = ok ? base + (size_t)r * D : 0;
            const uint32_t off = tile_offset<D>(row0 + r, chunk);
            cp_async16(k_tile + off, k_pages + src, ok ? 16 : 0);
            cp_async16(v_tile + off, v_pages + src, ok ? 16 : 0);
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int row = row0 + r, j = j0 + row;
        size_t src = 0;
        int bytes = 0;
        if (j >= lo && j <= hi) {
            const int slot = j / page_size;
            const int page = slot < table_width ? __ldg(table + slot) : -1;
            if (page >= 0) {
                src = (((size_t)page * n_kv + g) * page_size + (j - slot * page_size)) * D + chunk * 8;
                bytes = 16;
            }
        }
        const uint32_t off = tile_offset<D>(row, chunk);
        cp_async16(k_tile + off, k_pages + src, bytes);
        cp_async16(v_tile + off, v_pages + src, bytes);
    }
}

// One warp: scores of its 16 query rows against `N_TILES * 8` keys starting at
// tile row `key0`.  q holds the A fragments of the rows (D / 16 k-steps).
template <int D, int N_TILES>
__device__ __forceinline__ void qk_scores(float (*s)[4], const uint32_t (*q)[4], uint32_t k_tile, int key0, int lane) {
#pragma unroll
    for (int nt = 0; nt < N_TILES; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
    const int m = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int nt = 0; nt < N_TILES; nt += 2) {
            uint32_t b0, b1, b2, b3;
            const int row = key0 + (nt + (m >> 1)) * 8 + r;
            ldmatrix_x4(k_tile + tile_offset<D>(row, 2 * ks + (m & 1)), b0, b1, b2, b3);
            mma_bf16(s[nt], q[ks], b0, b1);
            mma_bf16(s[nt + 1], q[ks], b2, b3);
        }
    }
}

// One warp: o += p v for `K_STEPS * 16` keys starting at tile row `key0`; p are
// the probabilities as A fragments.
template <int D, int K_STEPS>
__device__ __forceinline__ void pv_accumulate(float (*o)[4], const uint32_t (*p)[4], uint32_t v_tile, int key0,
                                              int lane) {
    const int m = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < K_STEPS; ++kk) {
#pragma unroll
        for (int dt = 0; dt < D / 8; dt += 2) {
            uint32_t b0, b1, b2, b3;
            const int row = key0 + kk * 16 + (m & 1) * 8 + r;
            ldmatrix_x4_trans(v_tile + tile_offset<D>(row, dt + (m >> 1)), b0, b1, b2, b3);
            mma_bf16(o[dt], p[kk], b0, b1);
            mma_bf16(o[dt + 1], p[kk], b2, b3);
        }
    }
}

// ----------------------------------------------------------------------------- prefill
// Work item = 64 consecutive tokens of one entry (16 per warp) x one query head.
struct PrefillParams {
    bf16* out; const bf16* q; const bf16* k_pages; const bf16* v_pages;
    const int* q_start; const int* context_len; const int* block_table;
    const int* work;            // [items][2] = (entry, first token of the tile within the entry)
    int table_width, page_size, n_q, n_kv, window;
    float scale_log2;           // scale * log2(e)
};

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const PrefillParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE_BYTES = TILE_KEYS * D * 2;
    const uint32_t k_base = smem_u32(smem), v_base = k_base + 2 * TILE_BYTES;    // [2 stages] each
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g4 = lane >> 2, t4 = lane & 3;
    const int entry = p.work[2 * blockIdx.x], tile_tok = p.work[2 * blockIdx.x + 1];
    const int h = blockIdx.y, g = h / (p.n_q / p.n_kv);
    const int qs = p.q_start[entry], q_len = p.q_start[entry + 1] - qs;
    const int ctx = p.context_len[entry];
    const int* table = p.block_table + (size_t)entry * p.table_width;

    // this thread's two rows: tokens r0 and r0 + 8 of the tile
    const int tok0 = tile_tok + warp * 16 + g4, tok1 = tok0 + 8;
    const bool live0 = tok0 < q_len, live1 = tok1 < q_len;
    const int pos0 = ctx + tok0, pos1 = ctx + tok1;
    uint32_t qf[D / 16][4];
    {
        const bf16* q0 = p.q + ((size_t)(qs + min(tok0, q_len - 1)) * p.n_q + h) * D;
        const bf16* q1 = p.q + ((size_t)(qs + min(tok1, q_len - 1)) * p.n_q + h) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qf[ks][0] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t4);
            qf[ks][1] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t4);
            qf[ks][2] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t4);
            qf[ks][3] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t4);
        }
    }
    // keys the tile may see: from the first token's window start to the last token
    const int tile_first = ctx + tile_tok, tile_last = ctx + min(tile_tok + 63, q_len - 1);
    const int lo = p.window > 0 ? max(0, tile_first - p.window + 1) : 0, hi = tile_last;
    const int first_tile = lo / TILE_KEYS, last_tile = hi / TILE_KEYS;
    const int lo0 = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int lo1 = p.window > 0 ? max(0, pos1 - p.window + 1) : 0;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    load_kv_tile<D>(k_base, v_base, p.k_pages, p.v_pages, table, p.table_width, p.page_size, p.n_kv, g,
                    first_tile * TILE_KEYS, lo, hi);
    cp_async_commit();
    for (int kt = first_tile; kt <= last_tile; ++kt) {
        const int buf = (kt - first_tile) & 1;
        if (kt < last_tile) {
            load_kv_tile<D>(k_base + (buf ^ 1) * TILE_BYTES, v_base + (buf ^ 1) * TILE_BYTES, p.k_pages, p.v_pages,
                            table, p.table_width, p.page_size, p.n_kv, g, (kt + 1) * TILE_KEYS, lo, hi);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        float s[8][4];
        qk_scores<D, 8>(s, qf, k_base + buf * TILE_BYTES, 0, lane);
        // mask, running maximum
        const int j_base = kt * TILE_KEYS + 2 * t4;
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j_base + nt * 8 + e;
                s[nt][e] = (live0 && j >= lo0 && j <= pos0) ? s[nt][e] * p.scale_log2 : -INFINITY;
                s[nt][2 + e] = (live1 && j >= lo1 && j <= pos1) ? s[nt][2 + e] * p.scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float c0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mx0);
        const float c1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mx1);
        const float b0 = (mx0 == -INFINITY) ? 0.f : mx0, b1 = (mx1 == -INFINITY) ? 0.f : mx1;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pf[4][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float p00 = exp2f(s[nt][0] - b0), p01 = exp2f(s[nt][1] - b0);
            const float p10 = exp2f(s[nt][2] - b1), p11 = exp2f(s[nt][3] - b1);
            sum0 += p00 + p01;
            sum1 += p10 + p11;
            pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p00, p01);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p10, p11);
        }
        l0 = l0 * c0 + sum0;
        l1 = l1 * c1 + sum1;
        m0 = mx0;
        m1 = mx1;
        if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {     // the maximum moved for some row
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        }
        pv_accumulate<D, 4>(o, pf, v_base + buf * TILE_BYTES, 0, lane);
        __syncthreads();
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (live0) {
        bf16* dst = p.out + ((size_t)(qs + tok0) * p.n_q + h) * D + 2 * t4;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    }
    if (live1) {
        bf16* dst = p.out + ((size_t)(qs + tok1) * p.n_q + h) * D + 2 * t4;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

// ------------------------------------------------------------------------------ decode
// CTA = (key split, kv head, decode entry).  Rows of the MMA are the query
// heads of the kv head's group (at most 16).  The four warps share each 64-key
// tile and take 16 keys each; their partial results are merged through shared
// memory, the splits through global scratch by attn_decode_merge_kernel.
struct DecodeParams {
    const bf16* q; const bf16* k_pages; const bf16* v_pages;
    const int* q_start; const int* context_len; const int* block_table;
    const int* rows;            // [n] entries that are single decoded tokens
    float* part_o;              // [n][n_q][max_splits][D]
    float* part_ml;             // [n][n_q][max_splits][2]  (max in log2 units, sum)
    bf16* out;                  // [tokens][n_q][D]: written here when a token has one split
    const int* split_keys;      // device: keys per split (a multiple of 64): one value for the step
                                // (split_stride 0) or one per decoded token (split_stride 1)
    int split_stride;
    int table_width, page_size, n_q, n_kv, window, max_splits;
    float scale_log2;
    // Fused form (qkv != nullptr): queries, the new key and the new value come raw out of
    // the q/k/v projection; the kernel does the per-head norm and the rotation itself and
    // puts the new key and value into the cache (what qk_norm_rope_write_kernel does in a
    // launch of its own, src/kipp.c:2480-2512 and 2806-2811 for the formulas).
    const bf16* qkv; int ld_qkv;
    const void* q_norm_w; const void* k_norm_w; int norm_dtype; float eps;
    const float2* cos_sin;      // [token][D / 2] (cos, sin), or nullptr: no rotation
    bf16* k_write; bf16* v_write;   // the pools, writable; nullptr: this run does not write its cache
    int* status;
    int* n_splits_out;          // stream cut: [n][n_kv] splits of each pair, written for the merge; else nullptr
    int stream_ctas;            // stream cut: the grid
};

// The per-head norm and the rotation of one head vector, one warp: lane l holds
// elements l, l + 32, ...; element e < D/2 pairs with e + D/2, which the same lane
// holds.  Returns the values in x.
template <int D>
__device__ __forceinline__ void warp_norm_rope(float (&x)[D / 32], const void* norm_w, int norm_dtype, float eps,
                                               const float2* cs_row, int lane) {
    constexpr int NE = D / 32;
    // the weights and the (cos, sin) pairs first: their loads travel while the sum is formed
    float w[NE];
    float2 cs[NE / 2];
    if (norm_w != nullptr) {
#pragma unroll
        for (int j = 0; j < NE; ++j) w[j] = load_w(norm_w, norm_dtype, lane + 32 * j);
    }
    if (cs_row != nullptr) {
#pragma unroll
        for (int j = 0; j < NE / 2; ++j) cs[j] = cs_row[lane + 32 * j];
    }
    if (norm_w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NE; ++j) ss += x[j] * x[j];
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
        for (int j = 0; j < NE; ++j) x[j] = x[j] * scale * w[j];
    }
    if (cs_row != nullptr) {
#pragma unroll
        for (int j = 0; j < NE / 2; ++j) {
            const float a = x[j], b = x[j + NE / 2];
            x[j] = a * cs[j].x - b * cs[j].y;
            x[j + NE / 2] = b * cs[j].x + a * cs[j].y;
        }
    }
}

// out[:] = sum_s o_s * 2^(m_s - m) / sum_s l_s * 2^(m_s - m) of one head, splits in order, by one
// warp.  `ml` [n_splits][2], `po` [n_splits][D]; `weight` is 64 floats of shared memory of this warp.
__device__ __forceinline__ void warp_merge_head(bf16* __restrict__ dst, const float* ml, const float* po,
                                                int n_splits, int head_dim, float* weight, int lane) {
    float m[2], l[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int s = lane + 32 * i;
        m[i] = s < n_splits ? __ldcg(ml + 2 * s) : -INFINITY;
        l[i] = s < n_splits ? __ldcg(ml + 2 * s + 1) : 0.f;
    }
    const float mx = warp_max(fmaxf(m[0], m[1]));
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float w = (m[i] == -INFINITY) ? 0.f : exp2f(m[i] - mx);
        weight[lane + 32 * i] = w;
        total += l[i] * w;
    }
    // sum in split order would need a serial loop; lanes hold splits s and s + 32,
    // a fixed tree over lanes keeps the order the same for every token
    total = warp_sum(total);
    const float inv_sum = total > 0.f ? 1.f / total : 0.f;
    __syncwarp();
    // a lane takes four neighbouring values (head sizes are multiples of 16); the loads of eight
    // splits are issued together, then added in split order
    for (int d = 4 * lane; d < head_dim; d += 128) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                // a split with no key in reach (wholly behind a window) has weight 0 and wrote no
                // partial output: what lies in the scratch there is not read (0 x garbage may be NaN)
                const bool live = s0 + i < n_splits && weight[s0 + i] != 0.f;
                v[i] = live ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)(s0 + i) * head_dim + d))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float w = s0 + i < n_splits ? weight[s0 + i] : 0.f;
                if (w != 0.f) {
                    acc[0] += v[i].x * w; acc[1] += v[i].y * w; acc[2] += v[i].z * w; acc[3] += v[i].w * w;
                }
            }
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0] * inv_sum, acc[1] * inv_sum);
        __nv_bfloat162 hi = __floats2bfloat162_rn(acc[2] * inv_sum, acc[3] * inv_sum);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst + d) = packed;
    }
    __syncwarp();
}

// Keys per split for a context of kv_len keys: the step's split length, or
// longer when max_splits of them would not cover the context.
__host__ __device__ __forceinline__ int decode_split_keys(int kv_len, int max_splits, int split_keys_min) {
    int keys = split_keys_min < TILE_KEYS ? TILE_KEYS : split_keys_min / TILE_KEYS * TILE_KEYS;
    if ((long long)keys * max_splits < kv_len) {
        keys = (kv_len + max_splits - 1) / max_splits;
        keys = (keys + TILE_KEYS - 1) / TILE_KEYS * TILE_KEYS;
    }
    return keys;
}

// One split of one (token, kv head) pair: keys lo .. hi of entry `entry` (decoded token n of the
// step), split `split` of `n_splits`.  `first`: the CTA's first piece of work (it may fetch tiles
// before the dependency wait and makes that wait); all threads of the CTA call this together.
template <int D>
__device__ __forceinline__ void decode_split(const DecodeParams& p, uint8_t* smem, int n, int entry, int g, int lo,
                                             int hi, int split, int n_splits, bool first) {
    constexpr int TILE_BYTES = TILE_KEYS * D * 2;
    constexpr int STAGES = DECODE_STAGES;
    const uint32_t k_base = smem_u32(smem), v_base = k_base + STAGES * TILE_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g4 = lane >> 2, t4 = lane & 3;
    const int group = p.n_q / p.n_kv;
    const int tok = p.q_start[entry];
    const int pos = p.context_len[entry];                  // position of the decoded token
    const int* table = p.block_table + (size_t)entry * p.table_width;
    float* my_ml = p.part_ml + (((size_t)n * p.n_q + g * group) * p.max_splits + split) * 2;
    float* my_o = p.part_o + (((size_t)n * p.n_q + g * group) * p.max_splits + split) * D;
    const size_t head_stride_ml = (size_t)p.max_splits * 2, head_stride_o = (size_t)p.max_splits * D;

    // The first tiles of the split are fetched before the wait, while the kernel before
    // this one ends, unless one of them holds the token's own position: its key and
    // value are this step's (made below, or by the kernel before this one).
    // (The CTA that makes the token's key and value itself, the fused form's last split, may
    // fetch that tile early all the same: it puts the new key and value into the tile in shared
    // memory as well as into the cache, over whatever the cache held at that slot.)
    const int first_tile = lo / TILE_KEYS, last_tile = hi / TILE_KEYS, n_tiles = last_tile - first_tile + 1;
    const int ahead_tiles = min(STAGES - 1, n_tiles);
    const bool own_in_ahead = lo <= hi && pos / TILE_KEYS - first_tile < ahead_tiles && pos <= hi;
    const bool makes_own = p.qkv != nullptr && split == n_splits - 1 && p.k_write != nullptr;
    const bool early = first && lo <= hi && (!own_in_ahead || makes_own);
    const bool patch = early && own_in_ahead;
    if (early) {
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < n_tiles)
                load_kv_tile<D>(k_base + s * TILE_BYTES, v_base + s * TILE_BYTES, p.k_pages, p.v_pages, table,
                                p.table_width, p.page_size, p.n_kv, g, (first_tile + s) * TILE_KEYS, lo, hi);
            cp_async_commit();
        }
    }
    if (first) pdl_wait();
    if (lo > hi) {                                         // split wholly behind the window
        for (int i = threadIdx.x; i < group; i += THREADS) {
            my_ml[i * head_stride_ml] = -INFINITY;
            my_ml[i * head_stride_ml + 1] = 0.f;
        }
        return;
    }
    // rows g4 and g4 + 8 = heads of the group (zero rows beyond it)
    uint32_t qf[D / 16][4];
    if (p.qkv != nullptr) {
        // Fused form: norm and rotation of the group's queries here, a warp per head, into
        // shared memory (behind the tiles); the split that holds the token's own position
        // also makes the new key and value and puts them into the cache.
        constexpr int NE = D / 32;
        if (patch) {                                     // the tiles fetched early have landed, for every thread
            cp_async_wait<0>();
            __syncthreads();
        }
        bf16* q_s = reinterpret_cast<bf16*>(smem + 2 * STAGES * TILE_BYTES);   // [16][D]
        const bf16* raw = p.qkv + (size_t)tok * p.ld_qkv;
        const float2* cs_row = p.cos_sin != nullptr ? p.cos_sin + (size_t)tok * (D / 2) : nullptr;
        for (int hh = warp; hh < group; hh += WARPS) {
            float x[NE];
#pragma unroll
            for (int j = 0; j < NE; ++j) x[j] = __bfloat162float(raw[(size_t)(g * group + hh) * D + lane + 32 * j]);
            warp_norm_rope<D>(x, p.q_norm_w, p.norm_dtype, p.eps, cs_row, lane);
#pragma unroll
            for (int j = 0; j < NE; ++j) q_s[hh * D + lane + 32 * j] = __float2bfloat16_rn(x[j]);
        }
        if (split == n_splits - 1 && p.k_write != nullptr && warp < 2) {
            const int slot = pos / p.page_size;
            const int page = slot < p.table_width ? table[slot] : -1;
            if (page < 0) {                                        // unmapped page: refuse, never write
                if (lane == 0) atomicExch(p.status, 2);
            } else {
                const size_t at = (((size_t)page * p.n_kv + g) * p.page_size + (pos - slot * p.page_size)) * D;
                float x[NE];
                const bf16* src = raw + (size_t)(p.n_q + (warp == 0 ? 0 : p.n_kv) + g) * D;
#pragma unroll
                for (int j = 0; j < NE; ++j) x[j] = __bfloat162float(src[lane + 32 * j]);
                if (warp == 0) warp_norm_rope<D>(x, p.k_norm_w, p.norm_dtype, p.eps, cs_row, lane);
                bf16* dst = (warp == 0 ? p.k_write : p.v_write) + at;
#pragma unroll
                for (int j = 0; j < NE; ++j) dst[lane + 32 * j] = __float2bfloat16_rn(cache_value(x[j]));
                if (patch) {
                    const int ti = pos / TILE_KEYS - first_tile, row = pos - (first_tile + ti) * TILE_KEYS;
                    uint8_t* tile = smem + (warp == 0 ? 0 : STAGES * TILE_BYTES) + ti * TILE_BYTES;
#pragma unroll
                    for (int j = 0; j < NE; ++j) {
                        const int e = lane + 32 * j;
                        *reinterpret_cast<bf16*>(tile + tile_offset<D>(row, e >> 3) + (e & 7) * 2) =
                            __float2bfloat16_rn(cache_value(x[j]));
                    }
                }
            }
            __threadfence();                                       // before this CTA gathers that page
        }
        __syncthreads();
        const bool v0 = g4 < group, v1 = g4 + 8 < group;
        const bf16* q0 = q_s + min(g4, group - 1) * D;
        const bf16* q1 = q_s + min(g4 + 8, group - 1) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t4) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t4) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t4) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t4) : 0u;
        }
    } else {
        const bf16* q0 = p.q + ((size_t)tok * p.n_q + g * group + min(g4, group - 1)) * D;
        const bf16* q1 = p.q + ((size_t)tok * p.n_q + g * group + min(g4 + 8, group - 1)) * D;
        const bool v0 = g4 < group, v1 = g4 + 8 < group;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t4) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t4) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t4) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t4) : 0u;
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    if (!early) {
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < n_tiles)
                load_kv_tile<D>(k_base + s * TILE_BYTES, v_base + s * TILE_BYTES, p.k_pages, p.v_pages, table,
                                p.table_width, p.page_size, p.n_kv, g, (first_tile + s) * TILE_KEYS, lo, hi);
            cp_async_commit();
        }
    }
    for (int i = 0; i < n_tiles; ++i) {
        const int buf = i % STAGES;
        if (i + STAGES - 1 < n_tiles) {
            const int nb = (i + STAGES - 1) % STAGES;
            load_kv_tile<D>(k_base + nb * TILE_BYTES, v_base + nb * TILE_BYTES, p.k_pages, p.v_pages, table,
                            p.table_width, p.page_size, p.n_kv, g, (first_tile + i + STAGES - 1) * TILE_KEYS, lo, hi);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        float s[2][4];
        qk_scores<D, 2>(s, qf, k_base + buf * TILE_BYTES, warp * 16, lane);
        const int j_base = (first_tile + i) * TILE_KEYS + warp * 16 + 2 * t4;
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j_base + nt * 8 + e;
                const bool ok = j >= lo && j <= hi;
                s[nt][e] = ok ? s[nt][e] * p.scale_log2 : -INFINITY;
                s[nt][2 + e] = ok ? s[nt][2 + e] * p.scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float c0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mx0);
        const float c1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mx1);
        const float b0 = (mx0 == -INFINITY) ? 0.f : mx0, b1 = (mx1 == -INFINITY) ? 0.f : mx1;
        uint32_t pf[1][4];
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float p00 = exp2f(s[nt][0] - b0), p01 = exp2f(s[nt][1] - b0);
            const float p10 = exp2f(s[nt][2] - b1), p11 = exp2f(s[nt][3] - b1);
            sum0 += p00 + p01;
            sum1 += p10 + p11;
            pf[0][nt * 2 + 0] = pack_bf16(p00, p01);
            pf[0][nt * 2 + 1] = pack_bf16(p10, p11);
        }
        l0 = l0 * c0 + sum0;
        l1 = l1 * c1 + sum1;
        m0 = mx0;
        m1 = mx1;
        if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {     // the maximum moved for some row
#pragma unroll
            for (int d = 0; d < D / 8; ++d) { o[d][0] *= c0; o[d][1] *= c0; o[d][2] *= c1; o[d][3] *= c1; }
        }
        pv_accumulate<D, 1>(o, pf, v_base + buf * TILE_BYTES, warp * 16, lane);
        __syncthreads();
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // merge the four warps: [warp][row 0..15] max and sum, [warp][row][D] values
    __syncthreads();
    float* w_m = reinterpret_cast<float*>(smem);                  // [WARPS][16]
    float* w_l = w_m + WARPS * 16;                                // [WARPS][16]
    float* w_o = w_l + WARPS * 16;                                // [WARPS][16][D + 8]
    // (rows 8 floats longer than a head: the eight rows a warp's lanes write at once then fall on
    // four groups of banks instead of one)
    constexpr int WO = D + 8;
    if (t4 == 0) {
        w_m[warp * 16 + g4] = m0; w_m[warp * 16 + g4 + 8] = m1;
        w_l[warp * 16 + g4] = l0; w_l[warp * 16 + g4 + 8] = l1;
    }
#pragma unroll
    for (int d = 0; d < D / 8; ++d) {
        float* r0 = w_o + ((size_t)warp * 16 + g4) * WO + d * 8 + 2 * t4;
        float* r1 = w_o + ((size_t)warp * 16 + g4 + 8) * WO + d * 8 + 2 * t4;
        r0[0] = o[d][0]; r0[1] = o[d][1];
        r1[0] = o[d][2]; r1[1] = o[d][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * D; i += THREADS) {
        const int row = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, w_m[w * 16 + row]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {                          // fixed order
            const float wm = w_m[w * 16 + row];
            const float c = (wm == -INFINITY) ? 0.f : exp2f(wm - m);
            l += w_l[w * 16 + row] * c;
            acc += w_o[((size_t)w * 16 + row) * WO + d] * c;
        }
        if (n_splits == 1) {
            // nothing to merge: this is the token's result
            p.out[((size_t)tok * p.n_q + g * group + row) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
            continue;
        }
        my_o[row * head_stride_o + d] = acc;
        if (d == 0) {
            my_ml[row * head_stride_ml] = m;
            my_ml[row * head_stride_ml + 1] = l;
        }
    }
}


template <int D>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    // (What is read before the dependency wait comes with the step's lists, which a
    // copy brought before any kernel of the step started, or lies in the cache since
    // earlier steps.)
    // Grid (kv heads, tokens, splits): the splits are the slowest dimension, so the CTAs
    // that have work come first in launch order and all start at once; those of
    // splits a step does not use come after and leave at once.  (With the splits as
    // x, 1,664 of 2,048 CTAs of a batch-8 step were empty ones interleaved with the
    // working ones, and the last working CTA started microseconds late.)
    const int n = blockIdx.y, entry = p.rows[n], g = blockIdx.x, split = blockIdx.z;
    const int pos = p.context_len[entry];
    const int kv_len = pos + 1;
    const int first_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int split_keys = decode_split_keys(kv_len, p.max_splits, __ldg(p.split_keys + n * p.split_stride));
    const int n_splits = (kv_len + split_keys - 1) / split_keys;
    if (split >= n_splits) return;
    decode_split<D>(p, smem, n, entry, g, max(first_key, split * split_keys), min(pos, (split + 1) * split_keys - 1),
                    split, n_splits, true);
}

// The same work cut differently (DecodeParams::stream): the 64-key tiles of all (token, kv head)
// pairs of the step, pair after pair, are dealt out in equal runs to the CTAs of ONE wave, so a
// CTA's set-up and the merge of its four warps are paid once per run instead of once per short
// split, and all CTAs end together however the pairs and lengths fall (a step of 64 tokens with
// 2,048 keys each: 434 CTAs of 39 tiles instead of 1,536 of 11, four waves).  A run may end one
// pair and begin the next; each piece is a split of its pair, numbered in key order, and the
// pair's first piece notes the number of splits for the merge.  Tiles per run: the total over
// the grid, rounded up, but at least what keeps a pair within max_splits pieces.
constexpr int STREAM_MAX_TOKENS = 1024;
struct StreamCut { int per, total; };
// cum[i] = key tiles of the decoded tokens before i (of one kv head); returns the tiles per run
__device__ __forceinline__ StreamCut stream_cut(const DecodeParams& p, int n_tokens, int runs, int* cum, int* scratch) {
    int most = 0;
    for (int i = threadIdx.x; i < n_tokens; i += blockDim.x) {
        const int pos = p.context_len[p.rows[i]];
        const int first_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const int tiles = pos / TILE_KEYS - first_key / TILE_KEYS + 1;
        cum[i + 1] = tiles;
        most = max(most, tiles);
    }
    if (threadIdx.x == 0) { cum[0] = 0; *scratch = 0; }
    __syncthreads();
    atomicMax(scratch, most);
    if (threadIdx.x == 0)
        for (int i = 0; i < n_tokens; ++i) cum[i + 1] += cum[i];           // few hundred entries at most
    __syncthreads();
    StreamCut c;
    c.total = cum[n_tokens] * p.n_kv;
    const int longest = *scratch;
    c.per = max(max((c.total + runs - 1) / runs, (longest + p.max_splits - 2) / max(p.max_splits - 1, 1)), 1);
    return c;
}

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_decode_stream_kernel(const DecodeParams p, int n_tokens) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int cum[STREAM_MAX_TOKENS + 1];
    __shared__ int longest_s;
    pdl_launch_dependents();
    const StreamCut cut = stream_cut(p, n_tokens, (int)gridDim.x, cum, &longest_s);
    int idx = (int)blockIdx.x * cut.per;
    const int end = min(cut.total, idx + cut.per);
    bool first = true;
    while (idx < end) {
        // the pair the run's next tile belongs to: tokens in order, their kv heads in order
        int lo_n = 0, hi_n = n_tokens - 1;
        while (lo_n < hi_n) {
            const int mid = (lo_n + hi_n + 1) >> 1;
            if (cum[mid] * p.n_kv <= idx) lo_n = mid; else hi_n = mid - 1;
        }
        const int n = lo_n, tiles = cum[n + 1] - cum[n];
        const int within = idx - cum[n] * p.n_kv, g = within / tiles, t_in = within - g * tiles;
        const int take = min(tiles - t_in, end - idx);
        const int pair_first = cum[n] * p.n_kv + g * tiles;
        const int run_first = pair_first / cut.per, run_last = (pair_first + tiles - 1) / cut.per;
        const int n_splits = run_last - run_first + 1, split = (int)blockIdx.x - run_first;
        const int entry = p.rows[n];
        const int pos = p.context_len[entry];
        const int first_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const int tile0 = first_key / TILE_KEYS + t_in;
        if (t_in == 0 && threadIdx.x == 0) p.n_splits_out[n * p.n_kv + g] = n_splits;
        decode_split<D>(p, smem, n, entry, g, max(first_key, tile0 * TILE_KEYS),
                        min(pos, (tile0 + take) * TILE_KEYS - 1), split, n_splits, first);
        first = false;
        idx += take;
        __syncthreads();                                   // the merge's shared memory before the next piece's tiles
    }
    // (a CTA without a run leaves without the dependency wait: it touched nothing but the lists)
}

// The merge of a token's splits: a warp per head, WARPS heads per block.  (Merging inside the
// split kernel, by the CTA that finishes a token's last split, was measured and is no faster:
// one CTA then does behind a fence what this launch spreads over many while the next kernel
// already prefetches its weights.)
__global__ void __launch_bounds__(THREADS)
attn_decode_merge_kernel(bf16* __restrict__ out, const float* __restrict__ part_o,
                         const float* __restrict__ part_ml, const int* __restrict__ rows,
                         const int* __restrict__ q_start, const int* __restrict__ context_len,
                         int n_q, int head_dim, int max_splits,
                         const int* __restrict__ split_keys_ptr, int split_stride,
                         const int* __restrict__ n_splits_info, int n_kv) {
    __shared__ float weight[WARPS * 64];           // max_splits <= 64 checked by the launcher
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.y, h = blockIdx.x * WARPS + warp;
    if (h >= n_q) return;
    const int entry = rows[n];
    int n_splits;
    if (n_splits_info != nullptr) {                // the stream cut noted the pair's splits
        n_splits = n_splits_info[n * n_kv + h / (n_q / n_kv)];
    } else {
        const int kv_len = context_len[entry] + 1;
        const int split_keys = decode_split_keys(kv_len, max_splits, __ldg(split_keys_ptr + n * split_stride));
        n_splits = (kv_len + split_keys - 1) / split_keys;
    }
    if (n_splits == 1) return;                     // the split kernel wrote the result itself
    const size_t head = (size_t)n * n_q + h;
    warp_merge_head(out + ((size_t)q_start[entry] * n_q + h) * head_dim, part_ml + head * max_splits * 2,
                    part_o + head * max_splits * head_dim, n_splits, head_dim, weight + warp * 64, lane);
}

template <int D> int launch_prefill(const PrefillParams& p, int items, cudaStream_t s) {
    constexpr int SMEM = 4 * TILE_KEYS * D * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return kipp_launch(attn_prefill_kernel<D>, dim3(items, p.n_q), dim3(THREADS), SMEM, s, 1, p);
}

inline int launch_merge(const DecodeParams& p, void* out, int n, int head_dim, cudaStream_t s) {
    return kipp_launch(attn_decode_merge_kernel, dim3((p.n_q + WARPS - 1) / WARPS, n), dim3(THREADS), 0, s, 1,
                       (bf16*)out, (const float*)p.part_o, (const float*)p.part_ml, p.rows, p.q_start, p.context_len,
                       p.n_q, head_dim, p.max_splits, p.split_keys, p.split_stride, (const int*)p.n_splits_out, p.n_kv);
}

template <int D> int launch_decode(const DecodeParams& p, int n, cudaStream_t s) {
    constexpr int PIPE = 2 * DECODE_STAGES * TILE_KEYS * D * 2 + 16 * D * 2;   // tiles, and the group's queries
    constexpr int MERGE = (2 * WARPS * 16 + WARPS * 16 * (D + 8)) * 4;
    constexpr int SMEM = PIPE > MERGE ? PIPE : MERGE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (p.n_splits_out != nullptr) {
        static bool configured_stream = false;
        if (!configured_stream) {
            cudaError_t e = cudaFuncSetAttribute(attn_decode_stream_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
            if (e != cudaSuccess) return (int)e;
            configured_stream = true;
        }
        return kipp_launch(attn_decode_stream_kernel<D>, dim3(p.stream_ctas), dim3(THREADS), SMEM, s, 1, p, n);
    }
    if (n > 65535) return KIPP_ERR_ARG;
    return kipp_launch(attn_decode_kernel<D>, dim3(p.n_kv, n, p.max_splits), dim3(THREADS), SMEM, s, 1, p);
}
}  // namespace

// Whether these kernels take a head size / group.
extern "C" int kipp_attn_mma_supported(int head_dim, int n_q, int n_kv) {
    if (head_dim != 64 && head_dim != 128) return 0;
    if (n_kv <= 0 || n_q % n_kv) return 0;
    return 1;
}
extern "C" int kipp_attn_decode_supported(int head_dim, int n_q, int n_kv) {
    return kipp_attn_mma_supported(head_dim, n_q, n_kv) && n_q / n_kv <= 16;
}

// Prompt portions: `work` lists (entry, first token) of every 64-token tile.
extern "C" int kipp_attn_prefill_mma(void* out, const void* q, const void* k_pages, const void* v_pages,
                                     const int* q_start, const int* context_len, const int* block_table,
                                     int table_width, int page_size, const int* work, int items, int n_q,
                                     int n_kv, int head_dim, float scale, int window, void* stream) {
    if (items <= 0) return 0;
    if (!kipp_attn_mma_supported(head_dim, n_q, n_kv) || page_size <= 0 || window < 0) return KIPP_ERR_ARG;
    PrefillParams p;
    p.out = (bf16*)out; p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.q_start = q_start; p.context_len = context_len; p.block_table = block_table; p.work = work;
    p.table_width = table_width; p.page_size = page_size; p.n_q = n_q; p.n_kv = n_kv; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
    return head_dim == 64 ? launch_prefill<64>(p, items, s) : launch_prefill<128>(p, items, s);
}

// Bytes of scratch for n decode entries: partial outputs and (max, sum) pairs.
extern "C" long long kipp_attn_decode_scratch_bytes(int n, int n_q, int head_dim, int max_splits) {
    return (long long)n * n_q * max_splits * (head_dim + 2) * 4 + (long long)n * n_q * 4;   // and the pairs' split counts
}

// Whether a step of n decoded tokens can be cut as a stream (kipp_attn_decode_mma, stream_ctas > 0).
extern "C" int kipp_attn_decode_stream_ok(int n, int max_splits) { return n > 0 && n <= STREAM_MAX_TOKENS && max_splits >= 2; }

// Single decoded tokens: `rows` lists the n entries; scratch as sized above
// (part_o first, then part_ml, then the split counts), 16-byte aligned.  stream_ctas > 0: the
// step's key tiles are dealt out in equal runs to that many CTAs (attn_decode_stream_kernel;
// split_keys is not read); 0: every token is cut into splits of split_keys keys.
extern "C" int kipp_attn_decode_mma(void* out, const void* q, const void* k_pages, const void* v_pages,
                                    const int* q_start, const int* context_len, const int* block_table,
                                    int table_width, int page_size, const int* rows, int n, int n_q, int n_kv,
                                    int head_dim, float scale, int window, int max_splits,
                                    const int* split_keys, int split_stride, int stream_ctas, float* scratch,
                                    void* stream) {
    if (n <= 0) return 0;
    if (!kipp_attn_decode_supported(head_dim, n_q, n_kv) || page_size <= 0 || window < 0 || max_splits <= 0 ||
        max_splits > 64 || scratch == nullptr || ((uintptr_t)scratch & 15) || ((uintptr_t)out & 7) || stream_ctas < 0 ||
        (stream_ctas > 0 ? !kipp_attn_decode_stream_ok(n, max_splits) : split_keys == nullptr))
        return KIPP_ERR_ARG;
    DecodeParams p;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.q_start = q_start; p.context_len = context_len; p.block_table = block_table; p.rows = rows;
    p.part_o = scratch;
    p.out = (bf16*)out;
    p.part_ml = scratch + (size_t)n * n_q * max_splits * head_dim;
    p.table_width = table_width; p.page_size = page_size; p.n_q = n_q; p.n_kv = n_kv; p.window = window;
    p.max_splits = max_splits; p.split_keys = split_keys; p.split_stride = split_stride ? 1 : 0;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.qkv = nullptr; p.ld_qkv = 0; p.q_norm_w = p.k_norm_w = nullptr; p.norm_dtype = 0; p.eps = 0.f;
    p.cos_sin = nullptr; p.k_write = p.v_write = nullptr; p.status = nullptr;
    p.stream_ctas = stream_ctas;
    p.n_splits_out = stream_ctas > 0 ? reinterpret_cast<int*>(p.part_ml + (size_t)n * n_q * max_splits * 2) : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    int rc = head_dim == 64 ? launch_decode<64>(p, n, s) : launch_decode<128>(p, n, s);
    if (rc) return rc;
    return launch_merge(p, out, n, head_dim, s);
}

// The keys per split of each decoded token, chosen on the device from the cached lengths
// (context_len[rows[i]] + 1 keys), by the rule the host uses when it packs a step
// (AttentionPlanner in csrc/host/parts.hpp): with own_length, an eighth of the token's own
// context (so a token's result does not depend on its neighbours); else, for the whole step,
// the number of 64-key tiles per split k with the least (waves of resident CTAs) x (k + a CTA's
// fixed cost in tiles), on a tie the fewer splits.  One block; used between the steps of a
// burst that runs without the host.
namespace {
struct SplitRule { int pairs_per_entry, resident_ctas, fixed_tiles, max_splits, own_length; };
__global__ void attn_decode_replan_kernel(int* split_keys, const int* context_len, const int* rows, int n,
                                          SplitRule rule) {
    __shared__ int shared_s;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) shared_s = 0;
    __syncthreads();
    int longest = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) longest = max(longest, context_len[rows[i]] + 1);
    atomicMax(&shared_s, longest);
    __syncthreads();
    longest = shared_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        const long long pairs = (long long)n * rule.pairs_per_entry;
        const int total = (longest + TILE_KEYS - 1) / TILE_KEYS;
        int best = total;
        long long best_cost = -1;
        for (int k = total; k >= 1; --k) {
            const int splits = (total + k - 1) / k;
            if (splits > rule.max_splits) break;
            const long long waves = (pairs * splits + rule.resident_ctas - 1) / rule.resident_ctas;
            const long long cost = waves * (k + rule.fixed_tiles);
            if (best_cost < 0 || cost < best_cost) { best = k; best_cost = cost; }
        }
        shared_s = best * TILE_KEYS;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (rule.own_length) {
            const int own = (context_len[rows[i]] + 1 + 7) / 8;
            split_keys[i] = max(TILE_KEYS, (own + TILE_KEYS - 1) / TILE_KEYS * TILE_KEYS);
        } else {
            split_keys[i] = shared_s;
        }
    }
}
}  // namespace

extern "C" int kipp_attn_decode_replan(int* split_keys, const int* context_len, const int* rows, int n,
                                       int pairs_per_entry, int resident_ctas, int fixed_tiles, int max_splits,
                                       int own_length, void* stream) {
    if (n <= 0) return 0;
    if (pairs_per_entry <= 0 || resident_ctas <= 0 || max_splits <= 0) return KIPP_ERR_ARG;
    SplitRule rule{pairs_per_entry, resident_ctas, fixed_tiles, max_splits, own_length ? 1 : 0};
    return kipp_launch(attn_decode_replan_kernel, dim3(1), dim3(128), 0, (cudaStream_t)stream, 1, split_keys,
                       context_len, rows, n, rule);
}

// The same for a step of decoded tokens only, taking the raw output of the q/k/v
// projection [tokens, (n_q + 2 n_kv) * head_dim]: per-head norm (weights or nullptr),
// rotation by the step's (cos, sin) table (or nullptr) and the write of the new key and
// value into the pools (write_cache) happen inside the attention kernel.
extern "C" int kipp_attn_decode_mma_fused(void* out, const void* qkv, long long ld_qkv, void* k_pages,
                                          void* v_pages, const void* q_norm_w, const void* k_norm_w,
                                          int norm_dtype, float eps, const void* cos_sin, int write_cache,
                                          const int* q_start, const int* context_len, const int* block_table,
                                          int table_width, int page_size, const int* rows, int n, int n_q,
                                          int n_kv, int head_dim, float scale, int window, int max_splits,
                                          const int* split_keys, int split_stride, int stream_ctas, float* scratch,
                                          int* status, void* stream) {
    if (n <= 0) return 0;
    if (!kipp_attn_decode_supported(head_dim, n_q, n_kv) || page_size <= 0 || window < 0 || max_splits <= 0 ||
        max_splits > 64 || scratch == nullptr || ((uintptr_t)scratch & 15) || stream_ctas < 0 ||
        (stream_ctas > 0 ? !kipp_attn_decode_stream_ok(n, max_splits) : split_keys == nullptr) ||
        ((uintptr_t)out & 7) || status == nullptr || qkv == nullptr ||
        ld_qkv < (long long)(n_q + 2 * n_kv) * head_dim || ld_qkv > 0x7fffffffLL ||
        (q_norm_w == nullptr) != (k_norm_w == nullptr))
        return KIPP_ERR_ARG;
    if (q_norm_w != nullptr && norm_dtype != KIPP_DT_F32 && norm_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    DecodeParams p;
    p.q = nullptr; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.q_start = q_start; p.context_len = context_len; p.block_table = block_table; p.rows = rows;
    p.part_o = scratch;
    p.out = (bf16*)out;
    p.part_ml = scratch + (size_t)n * n_q * max_splits * head_dim;
    p.table_width = table_width; p.page_size = page_size; p.n_q = n_q; p.n_kv = n_kv; p.window = window;
    p.max_splits = max_splits; p.split_keys = split_keys; p.split_stride = split_stride ? 1 : 0;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.qkv = (const bf16*)qkv; p.ld_qkv = (int)ld_qkv;
    p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.norm_dtype = norm_dtype; p.eps = eps;
    p.cos_sin = (const float2*)cos_sin;
    p.k_write = write_cache ? (bf16*)k_pages : nullptr;
    p.v_write = write_cache ? (bf16*)v_pages : nullptr;
    p.status = status;
    p.stream_ctas = stream_ctas;
    p.n_splits_out = stream_ctas > 0 ? reinterpret_cast<int*>(p.part_ml + (size_t)n * n_q * max_splits * 2) : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    int rc = head_dim == 64 ? launch_decode<64>(p, n, s) : launch_decode<128>(p, n, s);
    if (rc) return rc;
    return launch_merge(p, out, n, head_dim, s);
}
