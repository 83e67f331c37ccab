// Causal grouped-query attention of prompt portions over the paged cache on the
// 5th-generation tensor cores: both products (scores = Q K^T and output = P V)
// are tcgen05.mma with their accumulators in tensor memory.
//
// Reference counterpart: cached_gqa_kernel (cuda/kipp_kernels.cu:160), formula
// src/kipp.c:2882-2922 (scores (q.k)/sqrt(D) over the keys a token may see,
// softmax with the maximum subtracted, weighted sum of values).
//
// One CTA = 128 consecutive tokens of one entry x one query head, 128 threads;
// thread r owns query row r: it reads the row's 64 scores of a key tile from
// tensor memory, so maximum, exponentials and sum need no exchange between
// threads.  Per tile of 64 keys:
//   1. keys and values are gathered page by page with cp.async into swizzled
//      shared-memory tiles (double-buffered: the next tile is in flight);
//   2. one thread issues S = Q K^T (128 x 64 x D) into tensor memory;
//   3. every thread: scale, mask, running maximum, p = 2^(s - m) -> bfloat16
//      into the shared-memory P tile; if some row's maximum moved, the output
//      accumulator in tensor memory is rescaled (tcgen05.ld / st);
//   4. one thread issues O += P V (128 x D x 64), V as an MN-major operand.
// Two CTAs fit an SM (112 KB shared memory, 256 tensor-memory columns each),
// so one's softmax runs under the other's MMAs.  All arithmetic outside the
// MMAs is float32.  Every mbarrier wait is bounded; on a time-out status[1] is
// set and the CTA drains and frees its tensor memory.
//
// Sizes: head_dim 64 or 128.  Cache layout of a layer: [page][kv_head][slot][D].
#include "common.cuh"
#include <math.h>

namespace {
constexpr int BM = 128;            // query rows per CTA = MMA M
constexpr int BN = 64;             // keys per tile
constexpr int THREADS = 128;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;   // ~1 s: a wait that long has failed

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    // Bounded by time, not by polls (a poll may itself block for a while): about
    // a second of SM clocks, or at once when another thread of the CTA gave up.
    const long long t0 = clock64();
    for (unsigned i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) break;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
          "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
          "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
          "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
          "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
          "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
// 2^x, single instruction (flushes denormals to zero: such weights do not matter in a sum of weights <= 1)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor (sm_100), 128-byte swizzle.  K-major tiles:
// rows of 128 bytes, 8-row groups `sbo` bytes apart.  MN-major tiles (values):
// `lbo` and `sbo` as the launcher passes them.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}
// bf16 x bf16 -> f32, A K-major, B K-major (b_mn = 0) or MN-major (b_mn = 1).
__host__ __device__ constexpr uint32_t idesc(int m, int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// Tiles are halves of 64 columns: half h, row r, 16-byte chunk c (0..7):
template <int ROWS> __device__ __forceinline__ uint32_t tile_off(int half, int row, int chunk) {
    return (uint32_t)(half * (ROWS * 128) + row * 128 + ((chunk ^ (row & 7)) << 4));
}

struct Params {
    bf16* out; const bf16* q; const bf16* k_pages; const bf16* v_pages;
    const int* q_start; const int* context_len; const int* block_table;
    const int* work;            // [items][2] = (entry, first token of the tile within the entry)
    int table_width, page_size, n_q, n_kv, window;
    float scale_log2;
    uint32_t v_lbo, v_sbo;      // descriptor strides of the MN-major value tile
    int* status;
};

template <int D> struct Cfg {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = BM * D * 2;
    static constexpr int KV_BYTES = BN * D * 2;       // one of K or V, one stage
    static constexpr int P_BYTES = BM * BN * 2;
    static constexpr int TMEM_COLS = D == 128 ? 256 : 128;      // S (64) + O (D), power of two
    // 114,816 bytes at head_dim 128: two CTAs (plus the 1 KB the system keeps per CTA) fit in 227 KB
    static constexpr size_t SMEM = Q_BYTES + 4 * KV_BYTES + P_BYTES + 128;
};

// Gathers BN rows of keys and of values, positions [j0, j0 + BN), kv head g.
template <int D>
__device__ __forceinline__ void load_kv(uint32_t k_tile, uint32_t v_tile, const bf16* __restrict__ k_pages,
                                        const bf16* __restrict__ v_pages, const int* __restrict__ table,
                                        int table_width, int page_size, int n_kv, int g, int j0, int lo, int hi) {
    constexpr int CHUNKS = D / 8;                        // 16-byte chunks per row
    constexpr int GROUPS = THREADS / CHUNKS;
    constexpr int ROWS = BN / GROUPS;                    // consecutive rows per thread
    const int chunk = threadIdx.x % CHUNKS, row0 = (threadIdx.x / CHUNKS) * ROWS;
    if ((page_size & 7) == 0 && ROWS <= 8) {
        // the thread's rows are consecutive and start at a multiple of ROWS: one page
        const int j_first = j0 + row0;
        const int slot = j_first / page_size;
        const int page = (slot < table_width && j_first <= hi && j_first + ROWS - 1 >= lo) ? __ldg(table + slot) : -1;
        const size_t base = (((size_t)max(page, 0) * n_kv + g) * page_size + (j_first - slot * page_size)) * D +
                            chunk * 8;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int j = j_first + r;
            const bool in = page >= 0 && j >= lo && j <= hi;
            const uint32_t off = tile_off<BN>(chunk >> 3, row0 + r, chunk & 7);
            cp_async16(k_tile + off, k_pages + (in ? base + (size_t)r * D : 0), in ? 16 : 0);
            cp_async16(v_tile + off, v_pages + (in ? base + (size_t)r * D : 0), in ? 16 : 0);
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
        const uint32_t off = tile_off<BN>(chunk >> 3, row, chunk & 7);
        cp_async16(k_tile + off, k_pages + src, bytes);
        cp_async16(v_tile + off, v_pages + src, bytes);
    }
}

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_tc_kernel(const Params p) {
    using C = Cfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];     // swizzled tiles need 1024-byte alignment
    const uint32_t q_tile = smem_u32(smem);
    const uint32_t k_tiles = q_tile + C::Q_BYTES;                  // [2 stages]
    const uint32_t v_tiles = k_tiles + 2 * C::KV_BYTES;            // [2 stages]
    const uint32_t p_tile = v_tiles + 2 * C::KV_BYTES;
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + C::Q_BYTES + 4 * C::KV_BYTES + C::P_BYTES);
    uint64_t* bar_o = bar_s + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        *abort_flag = (q_tile & 1023u) ? 1 : 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + BN;      // columns [0, 64) and [64, 64 + D)
    pdl_wait();

    const int entry = p.work[2 * blockIdx.x], tile_tok = p.work[2 * blockIdx.x + 1];
    const int h = blockIdx.y, g = h / (p.n_q / p.n_kv);
    const int qs = p.q_start[entry], q_len = p.q_start[entry + 1] - qs;
    const int ctx = p.context_len[entry];
    const int* table = p.block_table + (size_t)entry * p.table_width;

    // ---- the query tile: rows beyond the entry are zero
    {
        constexpr int CHUNKS = D / 8;
        for (int i = threadIdx.x; i < BM * CHUNKS; i += THREADS) {
            const int row = i / CHUNKS, chunk = i % CHUNKS;
            const int tok = tile_tok + row;
            const bool live = tok < q_len;
            const bf16* src = p.q + ((size_t)(qs + (live ? tok : 0)) * p.n_q + h) * D + chunk * 8;
            cp_async16(q_tile + tile_off<BM>(chunk >> 3, row, chunk & 7), src, live ? 16 : 0);
        }
    }
    // keys the tile may see: from the first token's window start to the last token
    const int row = threadIdx.x;                           // this thread's query row
    const int tok = tile_tok + row;
    const bool live = tok < q_len;
    const int pos = ctx + tok;
    const int lo_row = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int tile_first = ctx + tile_tok, tile_last = ctx + min(tile_tok + BM - 1, q_len - 1);
    const int lo = p.window > 0 ? max(0, tile_first - p.window + 1) : 0, hi = tile_last;
    const int first_tile = lo / BN, last_tile = hi / BN;

    load_kv<D>(k_tiles, v_tiles, p.k_pages, p.v_pages, table, p.table_width, p.page_size, p.n_kv, g,
               first_tile * BN, lo, hi);
    cp_async_commit();

    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    uint32_t phase = 0;
    constexpr uint32_t IDESC_S = idesc(BM, BN, 0);
    constexpr uint32_t IDESC_O = idesc(BM, D, 1);
    const uint32_t t_lane = (uint32_t)(warp * 32) << 16;   // this warp's tensor-memory lanes

    // (a failed wait does not leave the loop: every thread must meet every barrier;
    // once the abort flag is up the remaining waits return at once)
    for (int kt = first_tile; kt <= last_tile; ++kt) {
        const int buf = (kt - first_tile) & 1;
        const uint32_t k_tile = k_tiles + buf * C::KV_BYTES, v_tile = v_tiles + buf * C::KV_BYTES;
        // 1. this tile's keys and values (and, the first time, the queries) have landed
        cp_async_wait<0>();
        fence_async_proxy();                               // cp.async wrote; the tensor core reads
        __syncthreads();
        // 2. S = Q K^T
        if (threadIdx.x == 0) {
            tc_fence_after();
#pragma unroll
            for (int hh = 0; hh < C::HALVES; ++hh) {
                const uint64_t qd = smem_desc(q_tile + hh * (BM * 128), 0, 1024);
                const uint64_t kd = smem_desc(k_tile + hh * (BN * 128), 0, 1024);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem_s, qd + 2 * k, kd + 2 * k, IDESC_S, (hh | k) ? 1u : 0u);
            }
            umma_commit(bar_s);
        }
        // the next tile's keys and values travel meanwhile
        if (kt < last_tile) {
            load_kv<D>(k_tiles + (buf ^ 1) * C::KV_BYTES, v_tiles + (buf ^ 1) * C::KV_BYTES, p.k_pages, p.v_pages,
                       table, p.table_width, p.page_size, p.n_kv, g, (kt + 1) * BN, lo, hi);
        }
        cp_async_commit();
        // 3. softmax of this thread's row
        if (!mbar_wait(bar_s, phase, abort_flag)) { if (ok) atomicMax(&p.status[2], 1); ok = false; }
        tc_fence_after();
        float s[BN];
        tmem_ld32(tmem_s + t_lane, s);
        tmem_ld32(tmem_s + t_lane + 32, s + 32);
        const int j0 = kt * BN;
        // Masking only where the tile crosses a row's limits (the diagonal, a
        // window's edge, rows beyond the entry): decided per warp.
        if (!__all_sync(0xffffffffu, live && j0 + BN - 1 <= pos && j0 >= lo_row)) {
#pragma unroll
            for (int j = 0; j < BN; ++j) {
                const int key = j0 + j;
                if (!(live && key >= lo_row && key <= pos)) s[j] = -INFINITY;
            }
        }
        float raw = -INFINITY;
#pragma unroll
        for (int j = 0; j < BN; ++j) raw = fmaxf(raw, s[j]);
        const float mx = fmaxf(m_run, raw * p.scale_log2);          // scale > 0: the maximum commutes
        const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - mx);
        const float neg_base = (mx == -INFINITY) ? 0.f : -mx;
        float sum = 0.f;
        uint32_t packed[BN / 2];
#pragma unroll
        for (int j = 0; j < BN; j += 2) {
            const float p0 = fast_exp2(fmaf(s[j], p.scale_log2, neg_base));
            const float p1 = fast_exp2(fmaf(s[j + 1], p.scale_log2, neg_base));
            sum += p0 + p1;
            __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
            packed[j / 2] = *reinterpret_cast<uint32_t*>(&pk);
        }
        l_run = l_run * corr + sum;
        m_run = mx;
        // P tile: this thread's row, 8 chunks of 8 keys
        {
            uint8_t* p_row = smem + (p_tile - q_tile);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint4 v4 = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
                *reinterpret_cast<uint4*>(p_row + tile_off<BM>(0, row, c)) = v4;
            }
        }
        // rescale the output accumulator when some row of the warp moved its maximum
        if (kt > first_tile && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                float o[32];
                tmem_ld32(tmem_o + t_lane + c, o);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] *= corr;
                tmem_st32(tmem_o + t_lane + c, o);
            }
            tmem_st_wait();
        }
        fence_async_proxy();                               // P was written with ordinary stores
        tc_fence_before();
        __syncthreads();
        // 4. O += P V
        if (threadIdx.x == 0) {
            tc_fence_after();
            const uint64_t pd = smem_desc(p_tile, 0, 1024);
            const uint64_t vd = smem_desc(v_tile, p.v_lbo, p.v_sbo);
#pragma unroll
            for (int k = 0; k < BN / 16; ++k)
                // 16 keys further: 32 bytes in a P row; 16 rows = 2048 bytes in the value tile
                umma_bf16(tmem_o, pd + 2 * k, vd + 128 * k, IDESC_O, (kt > first_tile || k > 0) ? 1u : 0u);
            umma_commit(bar_o);
        }
        if (!mbar_wait(bar_o, phase, abort_flag)) { if (ok) atomicMax(&p.status[2], 2); ok = false; }
        tc_fence_after();
        phase ^= 1;
    }
    cp_async_wait<0>();

    // ---- result: o / l, this thread's row.  The tensor-memory loads are warp-wide
    // (.sync.aligned): every thread of the warp runs them, whether its row exists or not.
    {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        bf16* dst = p.out + ((size_t)(qs + (live ? tok : 0)) * p.n_q + h) * D;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
            float o[32];
            tmem_ld32(tmem_o + t_lane + c, o);
            if (ok && live) {
                uint4 pk[4];
                uint32_t* w = reinterpret_cast<uint32_t*>(pk);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
                    w[i] = *reinterpret_cast<uint32_t*>(&h2);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(dst + c)[i] = pk[i];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(&p.status[1], 1);
    if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D> int launch(const Params& p, int items, cudaStream_t s) {
    using C = Cfg<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return kipp_launch(attn_prefill_tc_kernel<D>, dim3(items, p.n_q), dim3(THREADS), C::SMEM, s, 1, p);
}
}  // namespace

extern "C" int kipp_attn_prefill_tc_supported(int head_dim, int n_q, int n_kv) {
    return (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0;
}

// Prompt portions: `work` lists (entry, first token) of every 128-token tile.
extern "C" int kipp_attn_prefill_tc(void* out, const void* q, const void* k_pages, const void* v_pages,
                                    const int* q_start, const int* context_len, const int* block_table,
                                    int table_width, int page_size, const int* work, int items, int n_q,
                                    int n_kv, int head_dim, float scale, int window, int* status,
                                    void* stream) {
    if (items <= 0) return 0;
    if (!kipp_attn_prefill_tc_supported(head_dim, n_q, n_kv) || page_size <= 0 || window < 0 || status == nullptr)
        return KIPP_ERR_ARG;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 15))
        return -3;
    Params p;
    p.out = (bf16*)out; p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.q_start = q_start; p.context_len = context_len; p.block_table = block_table; p.work = work;
    p.table_width = table_width; p.page_size = page_size; p.n_q = n_q; p.n_kv = n_kv; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    // The value tile is the MN-major operand of O += P V: leading offset = the next
    // 64-column half of the tile, stride offset = the next 8 keys (checked against
    // the other assignment on the device: that one gives wrong sums).
    p.v_lbo = (uint32_t)(BN * 128);
    p.v_sbo = 1024u;
    p.status = status;
    cudaStream_t s = (cudaStream_t)stream;
    return head_dim == 64 ? launch<64>(p, items, s) : launch<128>(p, items, s);
}
