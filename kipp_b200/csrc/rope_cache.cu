// Per-head RMSNorm of queries and keys, rotary position encoding, and the
// write of keys and values into the paged cache, in one pass over the fused
// q/k/v projection output.
//
// Reference counterparts, one launch each per token: head_norm_kernel
// (cuda/kipp_kernels.cu:67), rope_kernel (:121), kv_write_kernel (:143);
// formulas src/kipp.c:2480-2500 (norm over head_dim with one weight vector for
// all heads, before the rotation), src/kipp.c:2368-2382 (half-split pairs
// (i, i + rot/2), angle = position * theta^(-2i/rot)), and the cache row
// src/kipp.c:2806-2811 (keys stored after norm and rotation).
//
// The cosines and sines do not depend on the head or the layer: rope_table_kernel
// makes them once per step, [token][pair] -> (cos, sin), and every layer's
// launch reads them (full-range cosf/sinf for 40 heads x 36 layers per token
// were most of this kernel's instructions).
//
// One warp handles one (token, head).  Heads [0, Nq) are queries, [Nq, Nq+Nkv)
// keys, the rest values.  All arithmetic is float32; cosf/sinf are the full
// range-reduced versions.
//
// Cache layout of one layer: [page][kv_head][slot][head_dim]; a token at
// position p of entry e lives in page table[e][p / page_size], slot
// p % page_size.
#include "common.cuh"
#include "head_math.cuh"

namespace {
constexpr int MAX_PER_LANE = 8;   // head_dim <= 512 (pairs: 256 per half / 32 lanes)

__device__ __forceinline__ void load2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
}
__device__ __forceinline__ void load2(const bf16* p, float& a, float& b) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
    a = __low2float(v); b = __high2float(v);
}
__device__ __forceinline__ void store2(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
__device__ __forceinline__ void store2(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
// The reference's storage contract on a 32-bit cache: keys and values are rounded to
// bfloat16 when they are stored (src/kipp.c:2806-2811, 2614-2615).  Bit 1 of the
// launchers' write_cache argument asks for it.
__device__ __forceinline__ float stored(float v, bool round_bf16) {
    return round_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
}
// what a key or value element becomes in the cache: rounded if asked for, never an infinity or NaN
__device__ __forceinline__ float stored(float v, bool round_bf16, bool into_cache) {
    return into_cache ? cache_value(stored(v, round_bf16)) : v;
}

// V = elements a lane handles side by side (2 when head_dim is a multiple of 4:
// 4- or 8-byte loads and stores; else 1).
template <typename T, int V>
__global__ void qk_norm_rope_write_kernel(
    const T* __restrict__ qkv, int ld_qkv, T* __restrict__ q_out,
    T* __restrict__ k_pages, T* __restrict__ v_pages,
    const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_dtype, float eps,
    const float2* __restrict__ cos_sin, int rotary_dim,
    const int* __restrict__ positions, const int* __restrict__ entry_of_token,
    const int* __restrict__ block_table, int table_width, int page_size,
    int tokens, int n_q, int n_kv, int head_dim, int write_cache, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int heads_total = n_q + 2 * n_kv;
    if (warp_global >= tokens * heads_total) return;
    const int t = warp_global / heads_total;
    const int h = warp_global % heads_total;
    const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
    if (!is_q && !(write_cache & 1)) return;
    const bool rnd = !is_q && (write_cache & 2), kv = !is_q;
    const T* src = qkv + (size_t)t * ld_qkv + (size_t)h * head_dim;
    const int pos = positions[t];

    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * n_q + h) * head_dim;
    } else {
        const int e = entry_of_token[t];
        const int slot = pos / page_size;
        const int page = slot < table_width ? block_table[(size_t)e * table_width + slot] : -1;
        if (page < 0) {                       // unmapped page: refuse, never write
            if (lane == 0) atomicExch(status, 2);
            return;
        }
        const int g = is_k ? h - n_q : h - n_q - n_kv;
        T* base = is_k ? k_pages : v_pages;
        dst = base + (((size_t)page * n_kv + g) * page_size + (pos % page_size)) * head_dim;
    }

    if (!is_q && !is_k) {                     // values: copy
        if constexpr (V == 2) {
            for (int i = 2 * lane; i < head_dim; i += 64) {
                float a, b;
                load2(src + i, a, b);
                store2(dst + i, stored(a, rnd, true), stored(b, rnd, true));
            }
        } else {
            for (int i = lane; i < head_dim; i += 32) dst[i] = from_f32<T>(stored(to_f32(src[i]), rnd, true));
        }
        return;
    }

    const int half = head_dim / 2;
    // Lane owns pairs (i, i + half) for i = V * (lane + 32 j) + v.
    constexpr int STEPS = MAX_PER_LANE / V;
    float lo[STEPS][V], hi[STEPS][V];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < STEPS; ++j) {
        const int i = V * (lane + 32 * j);
        if (i < half) {
            if constexpr (V == 2) {
                load2(src + i, lo[j][0], lo[j][1]);
                load2(src + i + half, hi[j][0], hi[j][1]);
            } else {
                lo[j][0] = to_f32(src[i]);
                hi[j][0] = to_f32(src[i + half]);
            }
#pragma unroll
            for (int v = 0; v < V; ++v) ss += lo[j][v] * lo[j][v] + hi[j][v] * hi[j][v];
        }
    }
    const void* nw = is_q ? q_norm_w : k_norm_w;
    if (nw != nullptr) {
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)head_dim + eps);
#pragma unroll
        for (int j = 0; j < STEPS; ++j) {
            const int i = V * (lane + 32 * j);
            if (i < half) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    lo[j][v] = lo[j][v] * scale * load_w(nw, norm_dtype, i + v);
                    hi[j][v] = hi[j][v] * scale * load_w(nw, norm_dtype, i + v + half);
                }
            }
        }
    }
    // Rotation of the first rotary_dim dims, pairs (i, i + rotary_dim/2).
    // With rotary_dim == head_dim a pair is exactly this lane's (lo, hi).
    if (cos_sin != nullptr && rotary_dim == head_dim) {
        const float2* cs_row = cos_sin + (size_t)t * half;
#pragma unroll
        for (int j = 0; j < STEPS; ++j) {
            const int i = V * (lane + 32 * j);
            if (i < half) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const float2 cs = cs_row[i + v];
                    const float c = cs.x, s = cs.y;
                    const float a = lo[j][v], b = hi[j][v];
                    lo[j][v] = a * c - b * s;
                    hi[j][v] = b * c + a * s;
                }
            }
        }
    }
    if (cos_sin == nullptr || rotary_dim == head_dim || rotary_dim == 0) {
#pragma unroll
        for (int j = 0; j < STEPS; ++j) {
            const int i = V * (lane + 32 * j);
            if (i < half) {
                if constexpr (V == 2) {
                    store2(dst + i, stored(lo[j][0], rnd, kv), stored(lo[j][1], rnd, kv));
                    store2(dst + i + half, stored(hi[j][0], rnd, kv), stored(hi[j][1], rnd, kv));
                } else {
                    dst[i] = from_f32<T>(stored(lo[j][0], rnd, kv));
                    dst[i + half] = from_f32<T>(stored(hi[j][0], rnd, kv));
                }
            }
        }
        return;
    }
    // Partial rotation (rotary_dim < head_dim): pairs (i, i + rotary_dim/2)
    // cross lanes, so the normalised head goes through shared memory in float32.
    __shared__ float stage[4][64 * MAX_PER_LANE];
    float* row = stage[threadIdx.x >> 5];
#pragma unroll
    for (int j = 0; j < STEPS; ++j) {
        const int i = V * (lane + 32 * j);
        if (i < half) {
#pragma unroll
            for (int v = 0; v < V; ++v) {
                row[i + v] = lo[j][v];
                row[i + v + half] = hi[j][v];
            }
        }
    }
    __syncwarp();
    const int rh = rotary_dim / 2;
    for (int i = lane; i < head_dim; i += 32) {
        float v = row[i];
        if (i < rotary_dim) {
            const int p = i < rh ? i : i - rh;
            const float2 cs = cos_sin[(size_t)t * rh + p];
            const float c = cs.x, s = cs.y;
            v = i < rh ? row[i] * c - row[i + rh] * s : row[i] * c + row[i - rh] * s;
        }
        dst[i] = from_f32<T>(stored(v, rnd, kv));
    }
}

template <typename T>
int launch_rope(const void* qkv, int ld_qkv, void* q_out, void* k_pages, void* v_pages, const void* q_norm_w,
                const void* k_norm_w, int norm_dtype, float eps, const float2* cos_sin, int rotary_dim,
                const int* positions, const int* entry_of_token, const int* block_table, int table_width,
                int page_size, int tokens, int n_q, int n_kv, int head_dim, int write_cache, int* status,
                unsigned blocks, int threads, cudaStream_t s) {
    // adjacent elements side by side only when pairs of them stay inside one half
    const bool two = head_dim % 4 == 0 && ld_qkv % 2 == 0 && ((uintptr_t)qkv & 7) == 0 &&
                     ((uintptr_t)q_out & 7) == 0 && ((uintptr_t)k_pages & 7) == 0 && ((uintptr_t)v_pages & 7) == 0;
    auto kernel = two ? qk_norm_rope_write_kernel<T, 2> : qk_norm_rope_write_kernel<T, 1>;
    return kipp_launch(kernel, dim3(blocks), dim3(threads), 0, s, 1, (const T*)qkv, ld_qkv, (T*)q_out, (T*)k_pages,
                       (T*)v_pages, q_norm_w, k_norm_w, norm_dtype, eps, cos_sin, rotary_dim, positions,
                       entry_of_token, block_table, table_width, page_size, tokens, n_q, n_kv, head_dim,
                       write_cache, status);
}
// Fast path for bfloat16 with head_dim 64, 128 or 256 and a rotation over the
// whole head (or none): HEAD_DIM / 16 neighbouring lanes share a (token, head); a
// lane holds 8 consecutive elements of the head's first half and the 8 elements
// half a head further, which are the partners of its rotated pairs (two 16-byte
// loads and stores, no exchange between lanes but the norm's sum).  Grid (blocks of
// heads, tokens): no division per thread but the page lookup.  (The kernel is bound
// by the instructions it issues, not by memory: the version with 8 elements per
// lane and one shuffle per rotated element took 276 instructions per warp and
// 23 us for a 2,048-token portion of 48 heads.)
constexpr int ROPE_THREADS = 128;    // a block per 128 / (HEAD_DIM / 16) heads of a token: few idle lanes in the last block
template <int HEAD_DIM>
__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_write_bf16_kernel(
    const bf16* __restrict__ qkv, int ld_qkv, bf16* __restrict__ q_out,
    bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
    const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_dtype, float eps,
    const float2* __restrict__ cos_sin, const int* __restrict__ positions,
    const int* __restrict__ entry_of_token, const int* __restrict__ block_table, int table_width,
    int page_size, int n_q, int n_kv, int write_cache, int* __restrict__ status) {
    constexpr int LPH = HEAD_DIM / 16;           // lanes per head
    constexpr int HALF = HEAD_DIM / 2;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    const int h = blockIdx.x * (ROPE_THREADS / LPH) + (threadIdx.x / LPH);
    const int sub = threadIdx.x % LPH;
    const bool valid = h < n_q + 2 * n_kv;
    const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
    const bool active = valid && (is_q || (write_cache & 1));

    bf16* dst = nullptr;                         // of the lane's first 8 elements; the others HALF further
    if (active) {
        if (is_q) {
            dst = q_out + ((size_t)t * n_q + h) * HEAD_DIM + sub * 8;
        } else {
            const int pos = positions[t];
            const int slot = pos / page_size;
            const int page = slot < table_width ? block_table[(size_t)entry_of_token[t] * table_width + slot] : -1;
            if (page < 0) {                       // unmapped page: refuse, never write
                if (sub == 0) atomicExch(status, 2);
            } else {
                const int g = is_k ? h - n_q : h - n_q - n_kv;
                dst = (is_k ? k_pages : v_pages) +
                      (((size_t)page * n_kv + g) * page_size + (pos - slot * page_size)) * HEAD_DIM + sub * 8;
            }
        }
    }
    uint4 raw_lo = make_uint4(0u, 0u, 0u, 0u), raw_hi = raw_lo;
    if (dst) {
        const bf16* src = qkv + (size_t)t * ld_qkv + (size_t)h * HEAD_DIM + sub * 8;
        raw_lo = *reinterpret_cast<const uint4*>(src);
        raw_hi = *reinterpret_cast<const uint4*>(src + HALF);
    }
    if (valid && !is_q && !is_k) {                // values: copy
        if (dst) {
            *reinterpret_cast<uint4*>(dst) = cache_values_bf16x8(raw_lo);
            *reinterpret_cast<uint4*>(dst + HALF) = cache_values_bf16x8(raw_hi);
        }
        dst = nullptr;
    }
    // queries and keys.  No lane leaves early: a warp holds several heads, and
    // the lanes of value heads or beyond the last head take part in the shuffles.
    float a[8], b[8];
    unpack8(a, raw_lo);
    unpack8(b, raw_hi);
    if (q_norm_w != nullptr) {                    // both weights or neither (checked by the host)
        float ss = head_ssq8(a, b);
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
        const float scale = head_rstd(ss, HEAD_DIM, eps);
        if (dst) {
            const void* nw = is_q ? q_norm_w : k_norm_w;
            float wa[8], wb[8];
            load_w8(wa, nw, norm_dtype, sub * 8);
            load_w8(wb, nw, norm_dtype, HALF + sub * 8);
            head_scale8(a, scale, wa);
            head_scale8(b, scale, wb);
        }
    }
    if (cos_sin != nullptr && dst) head_rotate8(a, b, cos_sin + (size_t)t * HALF + sub * 8);
    if (dst) {
        const uint4 lo = pack8(a), hi = pack8(b);
        *reinterpret_cast<uint4*>(dst) = is_q ? lo : cache_values_bf16x8(lo);
        *reinterpret_cast<uint4*>(dst + HALF) = is_q ? hi : cache_values_bf16x8(hi);
    }
}

template <int HEAD_DIM>
int launch_rope_bf16(const void* qkv, int ld_qkv, void* q_out, void* k_pages, void* v_pages, const void* q_norm_w,
                     const void* k_norm_w, int norm_dtype, float eps, const float2* cos_sin, const int* positions,
                     const int* entry_of_token, const int* block_table, int table_width, int page_size, int tokens,
                     int n_q, int n_kv, int write_cache, int* status, cudaStream_t s) {
    constexpr int HEADS_PER_BLOCK = ROPE_THREADS / (HEAD_DIM / 16);
    const unsigned bx = (unsigned)((n_q + 2 * n_kv + HEADS_PER_BLOCK - 1) / HEADS_PER_BLOCK);
    return kipp_launch(qk_norm_rope_write_bf16_kernel<HEAD_DIM>, dim3(bx, (unsigned)tokens), dim3(ROPE_THREADS), 0, s, 1,
                       (const bf16*)qkv, ld_qkv, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, q_norm_w, k_norm_w,
                       norm_dtype, eps, cos_sin, positions, entry_of_token, block_table, table_width, page_size,
                       n_q, n_kv, write_cache, status);
}

// (cos, sin) of position * inv_freq[i] for every token of the step and every
// rotated pair: float32 angle as the reference forms it ((float)position *
// frequency, src/kipp.c:2374), full-range cosf/sinf.
__global__ void rope_table_kernel(float2* __restrict__ out, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int tokens, int half, int by_pair) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= tokens * half) return;
    // by_pair: out[pair][token], and a warp's threads are neighbouring tokens of one pair
    const int t = by_pair ? i % tokens : i / half, k = by_pair ? i / tokens : i - t * half;
    const float angle = (float)positions[t] * inv_freq[k];
    float s, c;
    sincosf(angle, &s, &c);
    out[i] = make_float2(c, s);
}
}  // namespace

extern "C" int kipp_rope_table(void* out, const int* positions, const float* inv_freq, int tokens, int half,
                               void* stream) {
    if (tokens <= 0 || half <= 0) return 0;
    const long long n = (long long)tokens * half;
    if (n > 0x7fffffffLL) return KIPP_ERR_ARG;
    return kipp_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, 1,
                       (float2*)out, positions, inv_freq, tokens, half, 0);
}

// The same values laid out [half, tokens]: for readers whose neighbouring threads hold
// neighbouring tokens (the projection epilogue that rotates its own heads).
extern "C" int kipp_rope_table_by_pair(void* out, const int* positions, const float* inv_freq, int tokens, int half,
                                       void* stream) {
    if (tokens <= 0 || half <= 0) return 0;
    const long long n = (long long)tokens * half;
    if (n > 0x7fffffffLL) return KIPP_ERR_ARG;
    return kipp_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, 1,
                       (float2*)out, positions, inv_freq, tokens, half, 1);
}

extern "C" int kipp_qk_norm_rope_write(
    const void* qkv, int ld_qkv, void* q_out, void* k_pages, void* v_pages, int dtype,
    const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps,
    const void* cos_sin, int rotary_dim, const int* positions, const int* entry_of_token,
    const int* block_table, int table_width, int page_size, int tokens, int n_q, int n_kv,
    int head_dim, int write_cache, int* status, void* stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || (head_dim & 1) || head_dim > 64 * MAX_PER_LANE) return KIPP_ERR_ARG;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return KIPP_ERR_ARG;
    if (page_size <= 0 || n_q <= 0 || n_kv <= 0) return KIPP_ERR_ARG;
    if (norm_dtype != KIPP_DT_F32 && norm_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    const long long warps = (long long)tokens * (n_q + 2 * n_kv);
    const int threads = 128;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages |
                           (uintptr_t)q_norm_w | (uintptr_t)k_norm_w | (uintptr_t)cos_sin) & 15) == 0;
    if (dtype == KIPP_DT_BF16 && aligned && ld_qkv % 8 == 0 && tokens <= 65535 &&
        (cos_sin == nullptr || rotary_dim == head_dim) && (q_norm_w == nullptr) == (k_norm_w == nullptr) &&
        (head_dim == 64 || head_dim == 128 || head_dim == 256)) {
        const float2* cs = rotary_dim == 0 ? nullptr : (const float2*)cos_sin;
        if (head_dim == 64)
            return launch_rope_bf16<64>(qkv, ld_qkv, q_out, k_pages, v_pages, q_norm_w, k_norm_w, norm_dtype, eps, cs,
                                        positions, entry_of_token, block_table, table_width, page_size, tokens, n_q,
                                        n_kv, write_cache, status, s);
        if (head_dim == 128)
            return launch_rope_bf16<128>(qkv, ld_qkv, q_out, k_pages, v_pages, q_norm_w, k_norm_w, norm_dtype, eps, cs,
                                         positions, entry_of_token, block_table, table_width, page_size, tokens, n_q,
                                         n_kv, write_cache, status, s);
        return launch_rope_bf16<256>(qkv, ld_qkv, q_out, k_pages, v_pages, q_norm_w, k_norm_w, norm_dtype, eps, cs,
                                     positions, entry_of_token, block_table, table_width, page_size, tokens, n_q,
                                     n_kv, write_cache, status, s);
    }
    if (dtype == KIPP_DT_F32)
        return launch_rope<float>(qkv, ld_qkv, q_out, k_pages, v_pages, q_norm_w, k_norm_w, norm_dtype, eps,
                                  (const float2*)cos_sin, rotary_dim, positions, entry_of_token, block_table, table_width,
                                  page_size, tokens, n_q, n_kv, head_dim, write_cache, status, (unsigned)blocks,
                                  threads, s);
    if (dtype == KIPP_DT_BF16)
        return launch_rope<bf16>(qkv, ld_qkv, q_out, k_pages, v_pages, q_norm_w, k_norm_w, norm_dtype, eps,
                                 (const float2*)cos_sin, rotary_dim, positions, entry_of_token, block_table, table_width,
                                 page_size, tokens, n_q, n_kv, head_dim, write_cache, status, (unsigned)blocks,
                                 threads, s);
    return KIPP_ERR_DTYPE;
}
