// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
// TMA -> shared memory -> tcgen05.mma -> tensor memory -> epilogue.
//
//   C[t, f] (+)= sum_k X[t, k] * W[f, k]        X [tokens, K], W [features, K]
//
// The reference computes these products one output row per block and one token
// per launch on the CUDA cores (matvec_kernel, cuda/kipp_kernels.cu:93); this
// kernel is the replacement for all seven projections and the output head.
//
// Orientation.  The WEIGHT tile is the M operand of the MMA (128 features per
// CTA) and the TOKENS are its N operand (16 to 256 per CTA).  So the same
// kernel serves a 2,048-token prompt (N tile 256, tensor-core bound) and a
// single decoded token (N tile 16, weight-streaming, HBM bound): a narrow token
// tile wastes no MMA rows on padding.  The accumulator of a CTA is D[feature
// lane, token column] in tensor memory; in the epilogue a warp's 32 lanes hold
// 32 neighbouring features of one token, so stores are contiguous.
//
// Work split.  grid = (token tiles, feature tiles, K splits).  With few tokens
// there are too few tiles to pull the whole HBM bandwidth, so K is split over
// the CTAs of one thread-block cluster (up to 8, along grid z).  Each CTA puts
// its partial accumulator into its own shared memory; after a cluster barrier
// CTA r adds, in split order, the partial sums of its share of the tokens out
// of all the CTAs' shared memory (distributed shared memory) and runs the
// epilogue for them.  No global scratch, no atomics, and the order of the sum
// is fixed.
//
// Warp roles (320 threads): warp 0 issues TMA loads, warp 1 allocates tensor
// memory and issues the MMAs, warps 2-9 run the epilogue (warp w reads the
// tensor-memory lanes 32*(w%4) .. +31, half of the columns each).  Every
// mbarrier wait gives up after about a second, records it in `status[1]` and
// lets the CTA drain and free its tensor memory.
//
// Prompt-sized batches (512 tokens and more) take a second kernel with the
// operands the other way round: 128 TOKENS are the M operand and 128 to 256
// features the N operand, one persistent CTA per SM walks over the tiles with
// two accumulators in tensor memory (the epilogue of a tile runs under the MMAs
// of the next), and the residual add leaves as reducing TMA stores.  The
// feature tile is chosen so that the rounds of tiles over the SMs are full.
// From 1,024 tokens on, store and SwiGLU products take a third kernel of the
// same build in which a PAIR of CTAs shares one MMA (cta_group::2, 256 tokens
// per tile, each CTA holding half of the weight tile).
//
// No multicast: every CTA fetches its own tiles.
#include "common.cuh"
#include "head_math.cuh"
#include "mbarrier.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>

#define EPI_STORE 0
#define EPI_ADD 1
#define EPI_SWIGLU 2

// Where the rows of a fused q/k/v projection go when they skip the stored product: the rows are
// [n_q query heads | n_kv key heads | n_kv value heads] of 128 features; queries and keys get their
// per-head RMSNorm (both weights or neither) and the half-split rotation, queries land in q_out,
// keys and values in the pages of the token's request.  The arithmetic is that of
// kipp_qk_norm_rope_write on the product rounded to bfloat16, bit for bit.
struct kipp_gemm_head_sink {
    void* q_out;                       // bf16 [tokens, n_q, 128]
    void* k_pages; void* v_pages;      // bf16 [page][kv head][slot][128]
    const void* q_norm_w; const void* k_norm_w; int norm_dtype; float eps;
    const void* cos_sin;               // float2 [64, tokens] (kipp_rope_table_by_pair), or NULL: no rotation
    const int* positions; const int* entry_of_token; const int* block_table;
    int table_width, page_size, n_q, n_kv;
    int write_cache;                   // bit 0: write keys and values
};

namespace {

constexpr int UMMA_M = 128;          // features per accumulator = MMA M (a CTA holds 1 or 2)
constexpr int TILE_K = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 320;         // TMA warp, MMA warp, 8 epilogue warps

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) { return kipp_mbar_try_wait(bar, parity); }
// bounded in time (mbarrier.cuh): false when the wait ran out or another thread of the CTA gave up
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return kipp_mbar_wait_limited(bar, parity, abort_flag, KIPP_WAIT_LIMIT_CYCLES);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// Adds a float32 box from shared memory into global memory (the adds happen at
// the L2; nothing is read back).  Tracked by the thread's bulk-group.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the sources of all earlier bulk-groups of this thread have been read
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all earlier bulk-groups of this thread are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// makes this thread's ordinary shared-memory writes visible to the TMA unit
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on `bar` when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
// ---- a pair of CTAs (a cluster of two) on one MMA: cta_group::2 forms
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Arrives on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// The address, in the cluster's shared window, of `bar` at the same offset in CTA `rank`.
__device__ __forceinline__ uint32_t mbar_in_cta(uint64_t* bar, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
    return remote;
}
// TMA load into this CTA's shared memory whose bytes are counted on a barrier of either
// CTA of the pair (`bar_cluster_addr` from mbar_in_cta).  No multicast: every CTA
// fetches what it holds.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
// Both CTAs of the pair run these (one warp each): the columns are taken in both.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[256 x N] (+)= A[256 x 16] B[N x 16]^T: 128 rows of A and D and N/2 rows of B live
// in each CTA, at the same shared- and tensor-memory addresses.  Issued by one thread
// of the pair's first CTA.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on `bar` (same offset) in both CTAs when all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"((uint16_t)3)
        : "memory");
}
// true in one lane of the (converged) warp.  The warps that issue copies and products walk
// their loops and wait as whole warps and let one elected lane issue: with a single lane in a
// branch of its own the operands of every product come out of that lane's registers, and a
// product was measured to take 60 to 80 cycles to issue instead of about 40.
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
    return chosen != 0;
}
__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// 16 consecutive float32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte
// swizzle, 8-row groups 1024 bytes apart (tile base 1024-byte aligned).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);          // start address, bits 0-13
    d |= (uint64_t)0 << 16;                            // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024u >> 4) << 32;                 // stride byte offset: next 8-row group
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4)                 // D format f32
           | (1u << 7)               // A format bf16
           | (1u << 10)              // B format bf16
           | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Ring of a narrow token tile (two CTAs per SM): as deep as two CTAs allow.  The weight
// matrices of a decode step are 20-100 MB, and the rings of all CTAs together hold
// about a quarter of the smallest: the deeper the ring, the more of the matrix is
// asked for before the kernel's dependency wait (measured: 96 KB -> 110 KB is 0.9 % of
// a decode step; 72, 56 and 40 KB, which would let the next kernel's CTAs move in
// beside this one's, cost 3, 8 and 29 %).
constexpr int NARROW_RING_BYTES = 110 * 1024;
template <int TILE_T, int TILE_F> struct Cfg {
    static constexpr int HALVES = TILE_F / UMMA_M;               // accumulators (128 features each)
    static constexpr int W_BYTES = TILE_F * TILE_K * 2;
    static constexpr int X_BYTES = TILE_T * TILE_K * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    // stages: as many as fit in NARROW_RING_BYTES for narrow token tiles (two CTAs
    // per SM), ~192 KB for wide ones
    static constexpr int STAGES = (TILE_T >= 128 || TILE_F > 128)
                                      ? (192 * 1024) / STAGE_BYTES
                                      : (NARROW_RING_BYTES / STAGE_BYTES > 8 ? 8 : NARROW_RING_BYTES / STAGE_BYTES);
    static constexpr int ACC_COLS = TILE_T * HALVES;
    static constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;   // 32, 64, 128, 256 or 512
    // epilogue warp groups: two groups of four warps split the token columns
    static constexpr int COL_GROUPS = TILE_T >= 32 ? 2 : 1;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ +
                                   TILE_T * 4 /*per-token factors*/;
};

constexpr int SINK_HEAD = 128;

struct Params {
    void* C;
    int out_dtype;          // KIPP_DT_*
    int epilogue;
    int tokens, features, K;
    long long ldc;
    int k_blocks_per_split; // TILE_K blocks each split handles
    int splits;
    int* status;
    // Folding an RMSNorm into the products around it (few-token kernel only; all optional):
    // a residual add can leave, beside the new residual r, what the NEXT norm needs:
    // xn[t, f] = bf16(r * norm_w[f]) and the sum of r^2 over each 32 features of a token
    // (ssq_out[t, f / 32]); a store or SwiGLU product whose input lacks the norm's factor
    // rsqrt(mean(r^2) + eps) per token gets it from those sums (ssq_in) and scales its rows.
    const void* norm_w; int norm_w_dtype;
    bf16* xn; long long ldn;
    float* ssq_out; int ssq_slots;
    const float* ssq_in; int ssq_in_slots;
    float inv_n, eps;
    kipp_gemm_head_sink heads;   // the HEADS form of the pair kernel only
};

// What the next norm needs of a new residual value r of token t, feature f (see Params): called
// by whole warps whose lanes hold 32 neighbouring features of one token.
__device__ __forceinline__ void emit_for_next_norm(const Params& p, float r, bool valid, int t, int f, int lane,
                                                   float w) {
    if (valid) p.xn[(size_t)t * p.ldn + f] = __float2bfloat16_rn(r * w);
    const float s = warp_sum(valid ? r * r : 0.f);
    const int slot = (f - lane) >> 5;
    if (lane == 0 && t < p.tokens && slot < p.ssq_slots) p.ssq_out[(size_t)t * p.ssq_slots + slot] = s;
}

// Epilogue of 16 tokens (t_first .. + 15) of this thread's feature f; `rstd` (or nullptr) holds
// the factor of each of these tokens that the product's input lacks.
__device__ __forceinline__ void epilogue_chunk(const Params& p, float* v, int t_first, int f, int lane,
                                               const float* rstd) {
    if (rstd != nullptr) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= rstd[j];
    }
    if (p.epilogue == EPI_ADD) {
        // all loads of the residual first, then the stores: the loads overlap
        float* cbase = reinterpret_cast<float*>(p.C) + f;
        float old[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = t_first + j;
            old[j] = (t < p.tokens && f < p.features) ? cbase[(size_t)t * p.ldc] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = t_first + j;
            if (t < p.tokens && f < p.features) cbase[(size_t)t * p.ldc] = old[j] + v[j];
        }
        if (p.xn != nullptr) {
            const bool f_ok = f < p.features;
            const float w = f_ok ? load_w(p.norm_w, p.norm_w_dtype, f) : 0.f;
            float sq[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int t = t_first + j;
                const float r = old[j] + v[j];
                const bool valid = t < p.tokens && f_ok;
                if (valid) p.xn[(size_t)t * p.ldn + f] = __float2bfloat16_rn(r * w);
                sq[j] = valid ? r * r : 0.f;
            }
            // Sums over the warp's 32 features of all 16 tokens at once: each exchange halves
            // the tokens a lane carries (16 shuffles instead of 5 per token); lane bits 4..1
            // then spell the token whose sum the lane holds.
#define KIPP_FOLD_STEP(n, bit)                                                    \
            _Pragma("unroll") for (int j = 0; j < n; ++j) {                       \
                const bool up = (lane & bit) != 0;                                \
                const float send = up ? sq[j] : sq[j + n];                        \
                const float keep = up ? sq[j + n] : sq[j];                        \
                sq[j] = keep + __shfl_xor_sync(0xffffffffu, send, bit);           \
            }
            KIPP_FOLD_STEP(8, 16) KIPP_FOLD_STEP(4, 8) KIPP_FOLD_STEP(2, 4) KIPP_FOLD_STEP(1, 2)
#undef KIPP_FOLD_STEP
            sq[0] += __shfl_xor_sync(0xffffffffu, sq[0], 1);
            const int t = t_first + (lane >> 1);        // bits 4..1 of the lane: 8, 4, 2, 1
            const int slot = (f - lane) >> 5;
            if ((lane & 1) == 0 && t < p.tokens && slot < p.ssq_slots) p.ssq_out[(size_t)t * p.ssq_slots + slot] = sq[0];
        }
    } else if (p.epilogue == EPI_SWIGLU) {
        // gate rows are even, up rows odd: the even lane takes its neighbour's
        // up value and writes silu(gate) * up
        const bool writer = (lane & 1) == 0 && f + 1 < p.features;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float u = __shfl_xor_sync(0xffffffffu, v[j], 1);
            const int t = t_first + j;
            if (writer && t < p.tokens) {
                const float r = __fdividef(v[j], 1.0f + __expf(-v[j])) * u;
                if (p.out_dtype == KIPP_DT_F32) reinterpret_cast<float*>(p.C)[(size_t)t * p.ldc + (f >> 1)] = r;
                else reinterpret_cast<bf16*>(p.C)[(size_t)t * p.ldc + (f >> 1)] = __float2bfloat16_rn(r);
            }
        }
    } else if (f < p.features) {
        if (p.out_dtype == KIPP_DT_F32) {
            float* c = reinterpret_cast<float*>(p.C) + f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (t_first + j < p.tokens) c[(size_t)(t_first + j) * p.ldc] = v[j];
        } else {
            bf16* c = reinterpret_cast<bf16*>(p.C) + f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (t_first + j < p.tokens) c[(size_t)(t_first + j) * p.ldc] = __float2bfloat16_rn(v[j]);
        }
    }
}

template <int TILE_T, int TILE_F>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const Params p) {
    using C = Cfg<TILE_T, TILE_F>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(tiles + (size_t)C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_ready = empty + C::STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* rstd_s = (float*)(tiles + (size_t)C::STAGES * C::STAGE_BYTES + 256);   // [TILE_T], see Params::ssq_in

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // token tiles vary fastest: CTAs that run together share a weight tile (L2)
    const int t0 = blockIdx.x * TILE_T;
    const int f0 = blockIdx.y * TILE_F;
    const int split = blockIdx.z;
    const int total_kb = (p.K + TILE_K - 1) / TILE_K;
    const int kb_begin = split * p.k_blocks_per_split;
    const int kb_end = min(total_kb, kb_begin + p.k_blocks_per_split);
    const int n_kb = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_ready, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        {
            // Weights do not depend on the kernels before this one: the first
            // ring of weight tiles is on its way before the dependency wait; the
            // activation tiles follow after it.
            const int ahead = min(n_kb, C::STAGES);
            if (elect_one()) {
                for (int i = 0; i < ahead; ++i) {
                    uint8_t* wt = tiles + (size_t)i * C::STAGE_BYTES;
                    mbar_expect_tx(&full[i], C::STAGE_BYTES);
                    tma_load_2d(wt, &map_w, &full[i], (kb_begin + i) * TILE_K, f0);
                }
            }
            __syncwarp();
            pdl_wait();
            if (elect_one()) {
                for (int i = 0; i < ahead; ++i) {
                    uint8_t* xt = tiles + (size_t)i * C::STAGE_BYTES + C::W_BYTES;
                    tma_load_2d(xt, &map_x, &full[i], (kb_begin + i) * TILE_K, t0);
                }
            }
            __syncwarp();
            for (int i = ahead; i < n_kb; ++i) {
                const int s = i % C::STAGES;
                const uint32_t ph = (i / C::STAGES) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1, abort_flag))) break;
                uint8_t* wt = tiles + (size_t)s * C::STAGE_BYTES;
                uint8_t* xt = wt + C::W_BYTES;
                const int k = (kb_begin + i) * TILE_K;
                if (elect_one()) {
                    mbar_expect_tx(&full[s], C::STAGE_BYTES);
                    tma_load_2d(wt, &map_w, &full[s], k, f0);
                    tma_load_2d(xt, &map_x, &full[s], k, t0);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        {
            constexpr uint32_t idesc = umma_idesc(UMMA_M, TILE_T);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % C::STAGES;
                const uint32_t ph = (i / C::STAGES) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(&full[s], ph, abort_flag))) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t wa = smem_u32(tiles + (size_t)s * C::STAGE_BYTES);
                const uint64_t wd = umma_smem_desc(wa), xd = umma_smem_desc(wa + C::W_BYTES);
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k) {
#pragma unroll
                        for (int h = 0; h < C::HALVES; ++h) {
                            // advance 16 elements = 32 bytes inside the swizzled row: +2 in the address
                            // field; the second 128 features start 128 rows = 16 KB further: +1024
                            umma_bf16(tmem_base + h * TILE_T, wd + 2 * k + h * 1024, xd + 2 * k, idesc,
                                      (i | k) ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty[s]);            // stage reusable when these MMAs are done
                }
                __syncwarp();
            }
            if (ok && elect_one()) umma_commit(acc_ready);
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps 2..9
        const int q = warp & 3;                    // tensor-memory lane quarter of this warp
        const int cg = (warp - 2) >> 2;            // which share of the token columns
        pdl_wait();                                // the epilogue reads and writes what earlier kernels made
        if (p.ssq_in != nullptr) {
            // the factor each token's row still lacks, while the products run: thread i of the
            // 256 epilogue threads sums token t0 + i's partial sums in slot order
            for (int j = threadIdx.x - 64; j < TILE_T; j += 256) {
                float sum = 0.f;
                if (t0 + j < p.tokens) {
                    const float* row = p.ssq_in + (size_t)(t0 + j) * p.ssq_in_slots;
#pragma unroll 8
                    for (int i = 0; i < p.ssq_in_slots; ++i) sum += row[i];
                }
                rstd_s[j] = 1.0f / sqrtf(sum * p.inv_n + p.eps);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        const float* rstd_tile = p.ssq_in != nullptr ? rstd_s : nullptr;
        bool ok = n_kb > 0 ? mbar_wait(acc_ready, 0, abort_flag) : true;
        tcgen05_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        constexpr int COLS_PER_GROUP = TILE_T / C::COL_GROUPS;
        if (ok && cg < C::COL_GROUPS) {
            if (p.splits == 1) {
#pragma unroll 1
                for (int h = 0; h < C::HALVES; ++h) {
                    const int f = f0 + h * UMMA_M + q * 32 + lane;
#pragma unroll 1
                    for (int c = cg * COLS_PER_GROUP; c < (cg + 1) * COLS_PER_GROUP; c += 16) {
                        float v[16];
                        if (n_kb > 0) tmem_ld16(taddr + h * TILE_T + c, v);
                        else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = 0.f;
                        }
                        epilogue_chunk(p, v, t0 + c, f, lane, rstd_tile ? rstd_tile + c : nullptr);
                    }
                }
            } else {
                // partial sums of this split into this CTA's shared memory, [token][feature]
                // (the pipeline stages are idle once the accumulator is complete)
                float* red = reinterpret_cast<float*>(tiles) + q * 32 + lane;
#pragma unroll 1
                for (int c = cg * COLS_PER_GROUP; c < (cg + 1) * COLS_PER_GROUP; c += 16) {
                    float v[16];
                    tmem_ld16(taddr + c, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) red[(size_t)(c + j) * UMMA_M] = v[j];
                }
            }
        }
    }

    // ------------------------------------------------------------------- split-K fix-up
    if (p.splits > 1) {
        // The residual values (and the norm weight) this thread adds to below are asked for before
        // the barrier and arrive under it: behind it they cost a trip to the L2 and back on a
        // path that is all latency (measured: 1,500 cycles from the barrier to the last store).
        constexpr int PRE = 4;
        float old_c[PRE] = {0.f, 0.f, 0.f, 0.f};
        float next_norm_w = 0.f;
        if (warp >= 2 && p.epilogue == EPI_ADD) {
            const int f = f0 + (warp & 3) * 32 + lane;
            const int per = (TILE_T + p.splits - 1) / p.splits;
            const int j0 = split * per, j1 = min(TILE_T, j0 + per);
            if (f < p.features) {
#pragma unroll
                for (int k = 0; k < PRE; ++k) {
                    const int j = j0 + ((warp - 2) >> 2) + 2 * k;
                    if (j < j1 && t0 + j < p.tokens) old_c[k] = reinterpret_cast<const float*>(p.C)[(size_t)(t0 + j) * p.ldc + f];
                }
                if (p.xn != nullptr) next_norm_w = load_w(p.norm_w, p.norm_w_dtype, f);
            }
        }
        // all threads of all CTAs of the cluster: partial sums are visible afterwards
        asm volatile("barrier.cluster.arrive.release.aligned;\n"
                     "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        if (warp >= 2 && !*abort_flag) {
            const int q = warp & 3;
            const int cg = (warp - 2) >> 2;                             // two warp groups share the tokens
            const int f = f0 + q * 32 + lane;
            const int per = (TILE_T + p.splits - 1) / p.splits;       // tokens this CTA finishes
            const int j0 = split * per, j1 = min(TILE_T, j0 + per);
            const uint32_t local = smem_u32(reinterpret_cast<float*>(tiles) + q * 32 + lane);
            // this CTA's view of every split's partial tile (at most 8 splits)
            uint32_t remote[8];
#pragma unroll
            for (int s = 0; s < 8; ++s)
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[s]) : "r"(local),
                             "r"(s < p.splits ? s : 0));
            // all loads of a token at once (they overlap), and a token ahead: the partial sums of
            // the next token travel while this one is finished (a trip through the cluster's
            // shared memory per token, one after the other, took 5,000 cycles for 7 tokens)
            auto load_parts = [&](float (&part)[8], int j) {
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    part[s] = 0.f;
                    if (s < p.splits)
                        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part[s])
                                     : "r"(remote[s] + (uint32_t)(j * UMMA_M * 4)) : "memory");
                }
            };
            float ahead[8];
            if (j0 + cg < j1) load_parts(ahead, j0 + cg);
            int k = -1;
            for (int j = j0 + cg; j < j1; j += 2) {
                ++k;
                const float old_pre = k == 0 ? old_c[0] : (k == 1 ? old_c[1] : (k == 2 ? old_c[2] : old_c[3]));
                float part[8];
#pragma unroll
                for (int s = 0; s < 8; ++s) part[s] = ahead[s];
                if (j + 2 < j1) load_parts(ahead, j + 2);
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < 8; ++s) v += part[s];              // in split order; absent splits add zero
                if (p.ssq_in != nullptr) v *= rstd_s[j];
                const int t = t0 + j;
                // one value per thread: the epilogue of a 16-token chunk with one live token
                if (p.epilogue == EPI_SWIGLU) {
                    const float u = __shfl_xor_sync(0xffffffffu, v, 1);
                    if ((lane & 1) == 0 && f + 1 < p.features && t < p.tokens) {
                        const float r = __fdividef(v, 1.0f + __expf(-v)) * u;
                        if (p.out_dtype == KIPP_DT_F32) reinterpret_cast<float*>(p.C)[(size_t)t * p.ldc + (f >> 1)] = r;
                        else reinterpret_cast<bf16*>(p.C)[(size_t)t * p.ldc + (f >> 1)] = __float2bfloat16_rn(r);
                    }
                } else if (p.epilogue == EPI_ADD && p.xn != nullptr) {
                    const bool valid = t < p.tokens && f < p.features;
                    float r = 0.f;
                    if (valid) {
                        float* c = reinterpret_cast<float*>(p.C) + (size_t)t * p.ldc + f;
                        r = (k < PRE ? old_pre : *c) + v;
                        *c = r;
                    }
                    emit_for_next_norm(p, r, valid, t, f, lane, next_norm_w);
                } else if (t < p.tokens && f < p.features) {
                    if (p.out_dtype == KIPP_DT_F32) {
                        float* c = reinterpret_cast<float*>(p.C) + (size_t)t * p.ldc + f;
                        *c = p.epilogue == EPI_ADD ? (k < PRE ? old_pre : *c) + v : v;
                    } else {
                        reinterpret_cast<bf16*>(p.C)[(size_t)t * p.ldc + f] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
        // nobody's shared memory may go away while a neighbour still reads it
        asm volatile("barrier.cluster.arrive.release.aligned;\n"
                     "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    }

    tcgen05_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(&p.status[1], 1);
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------
// Many tokens (prompt portions): the TOKENS are the M operand (128 per CTA) and
// the features the N operand (TILE_N per CTA).  A thread of the epilogue then
// owns one token row and gets consecutive features in consecutive registers,
// so it writes 16-byte vectors and SwiGLU pairs sit in one thread: an eighth of
// the instructions of the feature-per-thread epilogue above, which matters
// because the epilogue is not hidden behind the next tile's MMAs.
constexpr int TOKM_TILE_FIXED = 96;              // fixed part of a tile's time, in feature columns
constexpr int RED_BOX = 32;                     // the residual add goes out in boxes of 32 tokens x 32 features
constexpr int RED_BYTES = RED_BOX * RED_BOX * 4;
template <int TILE_N, bool REDUCE> struct CfgTok {
    static constexpr int X_BYTES = UMMA_M * TILE_K * 2;          // 128 tokens
    static constexpr int W_BYTES = TILE_N * TILE_K * 2;
    static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
    static constexpr int STAGING = REDUCE ? 8 * RED_BYTES : 0;   // one box per epilogue warp
    // persistent kernel, one CTA per SM: the ring takes what shared memory there is
    static constexpr int BUDGET = 227 * 1024 - 1024 - 256 - STAGING;
    static constexpr int STAGES = BUDGET / STAGE_BYTES > 8 ? 8 : BUDGET / STAGE_BYTES;
    static constexpr int TMEM_COLS = TILE_N <= 128 ? 128 : 256;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + STAGING + 1024 + 256;
};

// 16 consecutive features [f, f + 16) of token t held by one thread.
__device__ __forceinline__ void epilogue_row16(const Params& p, const float* v, int t, int f) {
    if (t >= p.tokens || f >= p.features) return;
    const bool full = f + 16 <= p.features;
    if (p.epilogue == EPI_ADD) {
        float* c = reinterpret_cast<float*>(p.C) + (size_t)t * p.ldc + f;
        if (full && ((uintptr_t)c & 15) == 0) {
            float4 old[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) old[i] = reinterpret_cast<float4*>(c)[i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                reinterpret_cast<float4*>(c)[i] = make_float4(old[i].x + v[4 * i], old[i].y + v[4 * i + 1],
                                                              old[i].z + v[4 * i + 2], old[i].w + v[4 * i + 3]);
        } else {
            for (int i = 0; i < 16 && f + i < p.features; ++i) c[i] += v[i];
        }
    } else if (p.epilogue == EPI_SWIGLU) {
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = __fdividef(v[2 * i], 1.0f + __expf(-v[2 * i])) * v[2 * i + 1];
        const size_t at = (size_t)t * p.ldc + (f >> 1);
        if (p.out_dtype == KIPP_DT_F32) {
            float* c = reinterpret_cast<float*>(p.C) + at;
            for (int i = 0; i < 8 && f + 2 * i + 1 < p.features; ++i) c[i] = r[i];
        } else {
            bf16* c = reinterpret_cast<bf16*>(p.C) + at;
            if (full && ((uintptr_t)c & 15) == 0) {
                uint4 pk;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(r[0], r[1]), h1 = __floats2bfloat162_rn(r[2], r[3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(r[4], r[5]), h3 = __floats2bfloat162_rn(r[6], r[7]);
                pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(c) = pk;
            } else {
                for (int i = 0; i < 8 && f + 2 * i + 1 < p.features; ++i) c[i] = __float2bfloat16_rn(r[i]);
            }
        }
    } else if (p.out_dtype == KIPP_DT_F32) {
        float* c = reinterpret_cast<float*>(p.C) + (size_t)t * p.ldc + f;
        if (full && ((uintptr_t)c & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                reinterpret_cast<float4*>(c)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
            for (int i = 0; i < 16 && f + i < p.features; ++i) c[i] = v[i];
        }
    } else {
        bf16* c = reinterpret_cast<bf16*>(p.C) + (size_t)t * p.ldc + f;
        if (full && ((uintptr_t)c & 15) == 0) {
            uint4 pk[2];
            uint32_t* w = reinterpret_cast<uint32_t*>(pk);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(c)[0] = pk[0];
            reinterpret_cast<uint4*>(c)[1] = pk[1];
        } else {
            for (int i = 0; i < 16 && f + i < p.features; ++i) c[i] = __float2bfloat16_rn(v[i]);
        }
    }
}

// 16 columns of a head's first half (from column 16 j) and their partners half a head further, as
// the stored product would hold them: times the row's factor (if the product's input lacks one),
// rounded to bfloat16, in pairs (words 0-7 the first half's values, 8-15 their partners).
__device__ __forceinline__ void sink_load(uint32_t taddr_head, int j, bool scaled, float rstd, uint32_t* words) {
    uint32_t r0[16], r1[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r0[0]), "=r"(r0[1]), "=r"(r0[2]), "=r"(r0[3]), "=r"(r0[4]), "=r"(r0[5]), "=r"(r0[6]), "=r"(r0[7]),
          "=r"(r0[8]), "=r"(r0[9]), "=r"(r0[10]), "=r"(r0[11]), "=r"(r0[12]), "=r"(r0[13]), "=r"(r0[14]), "=r"(r0[15])
        : "r"(taddr_head + 16 * j));
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r1[0]), "=r"(r1[1]), "=r"(r1[2]), "=r"(r1[3]), "=r"(r1[4]), "=r"(r1[5]), "=r"(r1[6]), "=r"(r1[7]),
          "=r"(r1[8]), "=r"(r1[9]), "=r"(r1[10]), "=r"(r1[11]), "=r"(r1[12]), "=r"(r1[13]), "=r"(r1[14]), "=r"(r1[15])
        : "r"(taddr_head + SINK_HEAD / 2 + 16 * j));
    // the registers of both loads are inputs of the wait, so nothing reads them before it
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r0[0]), "+r"(r0[1]), "+r"(r0[2]), "+r"(r0[3]), "+r"(r0[4]), "+r"(r0[5]), "+r"(r0[6]), "+r"(r0[7]),
                   "+r"(r0[8]), "+r"(r0[9]), "+r"(r0[10]), "+r"(r0[11]), "+r"(r0[12]), "+r"(r0[13]), "+r"(r0[14]),
                   "+r"(r0[15]), "+r"(r1[0]), "+r"(r1[1]), "+r"(r1[2]), "+r"(r1[3]), "+r"(r1[4]), "+r"(r1[5]),
                   "+r"(r1[6]), "+r"(r1[7]), "+r"(r1[8]), "+r"(r1[9]), "+r"(r1[10]), "+r"(r1[11]), "+r"(r1[12]),
                   "+r"(r1[13]), "+r"(r1[14]), "+r"(r1[15]));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float a0 = __uint_as_float(r0[2 * i]), a1 = __uint_as_float(r0[2 * i + 1]);
        float b0 = __uint_as_float(r1[2 * i]), b1 = __uint_as_float(r1[2 * i + 1]);
        if (scaled) {
            a0 = __fmul_rn(a0, rstd); a1 = __fmul_rn(a1, rstd);
            b0 = __fmul_rn(b0, rstd); b1 = __fmul_rn(b1, rstd);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1), hi = __floats2bfloat162_rn(b0, b1);
        words[i] = *reinterpret_cast<const uint32_t*>(&lo);
        words[8 + i] = *reinterpret_cast<const uint32_t*>(&hi);
    }
}
// Values 8 u .. 8 u + 7 of a block of sink_load's words (u = 0, 1) and their partners.
__device__ __forceinline__ void sink_unpack(const uint32_t* words, int u, float (&a)[8], float (&b)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = words[4 * u + i], hi = words[8 + 4 * u + i];
        a[2 * i] = __uint_as_float(lo << 16); a[2 * i + 1] = __uint_as_float(lo & 0xffff0000u);
        b[2 * i] = __uint_as_float(hi << 16); b[2 * i + 1] = __uint_as_float(hi & 0xffff0000u);
    }
}

// Where head h of token t goes (see kipp_gemm_head_sink), or nullptr: nothing to write.  Needs
// nothing of the product, so it is looked up while the tile's MMAs still run.
__device__ __forceinline__ bf16* sink_dst(const Params& p, int t, int h) {
    const kipp_gemm_head_sink& s = p.heads;
    if (t >= p.tokens || h >= s.n_q + 2 * s.n_kv) return nullptr;
    if (h < s.n_q) return reinterpret_cast<bf16*>(s.q_out) + ((size_t)t * s.n_q + h) * SINK_HEAD;
    if (!(s.write_cache & 1)) return nullptr;
    const int pos = s.positions[t];
    const int slot = pos / s.page_size;
    const int page = slot < s.table_width ? s.block_table[(size_t)s.entry_of_token[t] * s.table_width + slot] : -1;
    if (page < 0) {                               // unmapped page: refuse, never write
        atomicExch(p.status, 2);
        return nullptr;
    }
    const bool is_k = h < s.n_q + s.n_kv;
    const int g = is_k ? h - s.n_q : h - s.n_q - s.n_kv;
    return reinterpret_cast<bf16*>(is_k ? s.k_pages : s.v_pages) +
           (((size_t)page * s.n_kv + g) * s.page_size + (pos - slot * s.page_size)) * SINK_HEAD;
}

// The (cos, sin) of token t's pairs first .. first + 7 from the table laid out by pair.
__device__ __forceinline__ void sink_angles(const Params& p, int t, int first, bool wanted, float2 (&cs)[8]) {
    const float2* at = reinterpret_cast<const float2*>(p.heads.cos_sin) + (size_t)first * p.tokens + t;
#pragma unroll
    for (int i = 0; i < 8; ++i) cs[i] = wanted ? at[(size_t)i * p.tokens] : make_float2(1.f, 0.f);
}

// One head (SINK_HEAD accumulator columns from `taddr_head`) of token t, held by one thread, on its
// way to `dst` (sink_dst).  Called by whole warps: the head h is the same for all lanes, the
// tokens differ.  The head is read once and kept as bfloat16 pairs (the rounding of the stored
// product) while its sum of squares forms; the angles of 8 pairs are fetched 8 pairs ahead.
__device__ __forceinline__ void sink_head(const Params& p, uint32_t taddr_head, int t, int h, float rstd, bf16* dst) {
    const kipp_gemm_head_sink& s = p.heads;
    constexpr int BLOCKS = SINK_HEAD / 32;        // of 16 values and their 16 partners
    const bool is_q = h < s.n_q;
    const bool turns = h < s.n_q + s.n_kv;        // values are copied
    const bool normed = turns && s.q_norm_w != nullptr;
    const bool rotates = turns && s.cos_sin != nullptr;
    const bool scaled = p.ssq_in != nullptr;
    float2 cs[8];
    if (rotates) sink_angles(p, t, 0, dst != nullptr, cs);
    uint32_t words[BLOCKS * 16];
    float part[2 * BLOCKS];
#pragma unroll
    for (int j = 0; j < BLOCKS; ++j) {
        sink_load(taddr_head, j, scaled, rstd, words + 16 * j);
        if (normed) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                float a[8], b[8];
                sink_unpack(words + 16 * j, u, a, b);
                part[2 * j + u] = head_ssq8(a, b);
            }
        }
    }
    const float scale = normed ? head_rstd(head_ssq_tree(part), SINK_HEAD, s.eps) : 1.0f;
    const void* nw = is_q ? s.q_norm_w : s.k_norm_w;
#pragma unroll
    for (int j = 0; j < BLOCKS; ++j) {
        uint4 out_lo[2], out_hi[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int first = 16 * j + 8 * u;      // of the 8 values in the head's first half
            float2 cs_next[8];
            if (rotates && first + 8 < SINK_HEAD / 2) sink_angles(p, t, first + 8, dst != nullptr, cs_next);
            float a[8], b[8];
            sink_unpack(words + 16 * j, u, a, b);
            if (normed) {
                float wa[8], wb[8];
                load_w8(wa, nw, s.norm_dtype, first);
                load_w8(wb, nw, s.norm_dtype, SINK_HEAD / 2 + first);
                head_scale8(a, scale, wa);
                head_scale8(b, scale, wb);
            }
            if (rotates) {
#pragma unroll
                for (int i = 0; i < 8; ++i) head_rotate(a[i], b[i], cs[i]);
                if (first + 8 < SINK_HEAD / 2) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) cs[i] = cs_next[i];
                }
            }
            out_lo[u] = pack8(a);
            out_hi[u] = pack8(b);
            if (!is_q) { out_lo[u] = cache_values_bf16x8(out_lo[u]); out_hi[u] = cache_values_bf16x8(out_hi[u]); }
        }
        if (dst != nullptr) {                      // 32 bytes of each half of the head side by side
            uint4* lo = reinterpret_cast<uint4*>(dst + 16 * j);
            uint4* hi = reinterpret_cast<uint4*>(dst + SINK_HEAD / 2 + 16 * j);
            lo[0] = out_lo[0]; lo[1] = out_lo[1];
            hi[0] = out_hi[0]; hi[1] = out_hi[1];
        }
    }
}

// Epilogue of one 128-token x TILE_N tile by one warp: its 32 tokens (tensor-memory
// lanes of `taddr`), its share `cg` (0 or 1) of the feature columns.
template <int TILE_N, bool REDUCE, bool HEADS = false>
__device__ __forceinline__ void tokm_epilogue_tile(const Params& p, const CUtensorMap* map_c, uint32_t taddr,
                                                   uint8_t* box, int t_warp, int f0, int cg, int lane, bool ok,
                                                   bf16* head_dst = nullptr) {
    constexpr int HALF = (TILE_N / 2 + 15) / 16 * 16;
    const int t = t_warp + lane;
    if constexpr (REDUCE) {
#pragma unroll 1
        for (int c = cg * RED_BOX; c < TILE_N; c += 2 * RED_BOX) {
            float v[32];
            tmem_ld16(taddr + c, v);
            tmem_ld16(taddr + c + 16, v + 16);
            if (lane == 0) bulk_wait_read();        // the unit has read the previous box
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                    make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && ok && t_warp < p.tokens && f0 + c < p.features) {
                tma_reduce_add_2d(map_c, box, f0 + c, t_warp);
                bulk_commit();
            }
        }
    } else {
        // the factor this thread's token still lacks (see Params::ssq_in), summed in slot order
        float rstd = 1.0f;
        if (p.ssq_in != nullptr && t < p.tokens) {
            const float* row = p.ssq_in + (size_t)t * p.ssq_in_slots;
            float sum = 0.f;
            for (int i = 0; i < p.ssq_in_slots; ++i) sum += row[i];
            rstd = 1.0f / sqrtf(sum * p.inv_n + p.eps);
        }
        if constexpr (HEADS) {
            static_assert(TILE_N == 2 * SINK_HEAD, "a head per half of the tile's columns");
            sink_head(p, taddr + cg * SINK_HEAD, t, f0 / SINK_HEAD + cg, rstd, ok ? head_dst : nullptr);
            return;
        }
#pragma unroll 1
        for (int c = cg * HALF; c < min(TILE_N, (cg + 1) * HALF); c += 16) {
            float v[16];
            tmem_ld16(taddr + c, v);
            if (p.ssq_in != nullptr) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] *= rstd;
            }
            if (ok) epilogue_row16(p, v, t, f0 + c);
        }
    }
}

// Persistent: one CTA per SM walks over the tiles (token tiles fastest, so CTAs
// that run together share a weight tile in L2).  Two accumulators in tensor
// memory: while the epilogue warps drain tile i, the MMA warp already works on
// tile i + 1, and the TMA warp streams on without a break between tiles.
//
// REDUCE (the float32 residual add): a thread per token would touch 16 bytes of
// 32 different lines per store.  Instead each epilogue warp puts 32 tokens x 32
// features of the product into shared memory (128-byte swizzle, so the row-wise
// writes spread over the banks) and hands the box to the TMA unit as a reducing
// store: the sum is formed at the L2, whole lines at a time, and the old value
// never travels to the SM.  One add per element, so the result does not depend
// on timing.  `map_c` covers exactly [tokens, features]: what lies outside is
// dropped by the unit.
template <int TILE_N, bool REDUCE>
__global__ void __launch_bounds__(THREADS)
gemm_tc_tokm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_c, const Params p) {
    using C = CfgTok<TILE_N, REDUCE>;
    static_assert(TILE_N % RED_BOX == 0 && TILE_N >= 2 * RED_BOX && TILE_N <= 256, "feature tile");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = tiles + (size_t)C::STAGES * C::STAGE_BYTES;        // 1024-byte aligned
    uint64_t* full = (uint64_t*)(staging + C::STAGING);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;        // [2]
    uint64_t* acc_empty = acc_full + 2;            // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (p.K + TILE_K - 1) / TILE_K;
    const int m_tiles = (p.tokens + UMMA_M - 1) / UMMA_M;
    const int n_tiles = (p.features + TILE_N - 1) / TILE_N;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, 2 * C::TMEM_COLS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0 && (int)blockIdx.x < total_tiles) {
            // Weights depend on no earlier kernel: the first ring of weight tiles of
            // this CTA's first tile is requested before the dependency wait, the
            // activations after it.
            const int first = blockIdx.x;
            const int ahead = min(n_kb, C::STAGES);
            {
                const int t0 = (first % m_tiles) * UMMA_M, f0 = (first / m_tiles) * TILE_N;
                for (int i = 0; i < ahead; ++i) {
                    mbar_expect_tx(&full[i], C::STAGE_BYTES);
                    tma_load_2d(tiles + (size_t)i * C::STAGE_BYTES + C::X_BYTES, &map_w, &full[i], i * TILE_K, f0);
                }
                pdl_wait();
                for (int i = 0; i < ahead; ++i)
                    tma_load_2d(tiles + (size_t)i * C::STAGE_BYTES, &map_x, &full[i], i * TILE_K, t0);
            }
            int it = ahead;                                 // K blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = first; tile < total_tiles && ok; tile += gridDim.x) {
                const int t0 = (tile % m_tiles) * UMMA_M, f0 = (tile / m_tiles) * TILE_N;
                for (int i = (tile == first ? ahead : 0); i < n_kb; ++i, ++it) {
                    const int s = it % C::STAGES;
                    if (it >= C::STAGES && !mbar_wait(&empty[s], ((it / C::STAGES) & 1) ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* xt = tiles + (size_t)s * C::STAGE_BYTES;
                    mbar_expect_tx(&full[s], C::STAGE_BYTES);
                    tma_load_2d(xt, &map_x, &full[s], i * TILE_K, t0);
                    tma_load_2d(xt + C::X_BYTES, &map_w, &full[s], i * TILE_K, f0);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(UMMA_M, TILE_N);
            int it = 0, tile_iter = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_iter) {
                const int b = tile_iter & 1, use = tile_iter >> 1;
                if (tile_iter >= 2 && !mbar_wait(&acc_empty[b], (use & 1) ^ 1, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + b * C::TMEM_COLS;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % C::STAGES;
                    if (!mbar_wait(&full[s], (it / C::STAGES) & 1, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t xa = smem_u32(tiles + (size_t)s * C::STAGE_BYTES);
                    const uint64_t xd = umma_smem_desc(xa), wd = umma_smem_desc(xa + C::X_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k)
                        umma_bf16(acc, xd + 2 * k, wd + 2 * k, idesc, (i | k) ? 1u : 0u);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[b]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps 2..9
        const int q = warp & 3;                    // tensor-memory lane quarter = 32 tokens
        const int cg = (warp - 2) >> 2;            // half of the feature columns
        pdl_wait();
        uint8_t* box = staging + (size_t)(warp - 2) * RED_BYTES;
        int tile_iter = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tile_iter) {
            const int b = tile_iter & 1, use = tile_iter >> 1;
            const int t_warp = (tile % m_tiles) * UMMA_M + q * 32, f0 = (tile / m_tiles) * TILE_N;
            if (ok && !mbar_wait(&acc_full[b], use & 1, abort_flag)) ok = false;
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + b * C::TMEM_COLS + ((uint32_t)(q * 32) << 16);
            tokm_epilogue_tile<TILE_N, REDUCE>(p, &map_c, taddr, box, t_warp, f0, cg, lane, ok);
            // this warp has read its part of the accumulator: hand it back
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
        if (REDUCE && lane == 0) bulk_wait_all();
    }
    tcgen05_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(&p.status[1], 1);
    if (warp == 1) tmem_dealloc(tmem_base, 2 * C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------
// The same work with a PAIR of CTAs on one MMA (cta_group::2): a tile is 256 tokens x
// TILE_N features; CTA r of the pair holds tokens [128 r, 128 r + 128) and the
// weight rows [r TILE_N/2, (r + 1) TILE_N/2) of the tile, and gets the accumulator
// of its 128 tokens in its own tensor memory.  Each SM then writes and reads half
// of the weight tile instead of all of it: a 128 x 256 x 64 block costs 64 KB of
// shared-memory traffic per 512 tensor cycles instead of 96 KB, under the 128 B/cycle
// the shared memory gives (the one-CTA kernel is capped near 68 % by that).
//
// Hand-overs.  Every CTA fills its own ring by TMA, but the bytes of both are counted
// on full[s] of the first CTA (armed there with twice a stage's bytes): its MMA
// thread waits for that one barrier, issues the MMAs and commits to empty[s] in
// both CTAs; after a tile it commits to acc_full[b] in both.  The epilogue warps of
// both CTAs arrive on acc_empty[b] of the first CTA (16 arrivals).  A cluster
// barrier stands after the barrier set-up and before the tensor memory is given
// back.  (A first version let a thread of the second CTA relay "my stage is full"
// to the first: one relay per K block took about a microsecond, three times the
// MMAs of the block.)
//
// Tiles wider than the 256 features one MMA takes (288, 320) are made of two MMAs of half the
// width per K step, side by side in ONE accumulator (288 or 320 of the 512 tensor-memory
// columns, so no second accumulator: the next tile's MMAs wait for this tile's epilogue).
// They are for shapes whose narrower tiles leave a second, nearly empty round: 2,048 tokens x
// 2,560 features are 8 x 9 tiles of 288 = 72 pairs = one round on 74 pairs of SMs.  A CTA's
// share of the weight tile then lies in two blocks of SUB_N / 2 rows, one per MMA.
template <int TILE_N, bool REDUCE> struct CfgPair {
    static constexpr int SUBS = TILE_N > 256 ? 2 : 1;            // MMAs per K step
    static constexpr int SUB_N = TILE_N / SUBS;                  // features of one MMA
    static constexpr int SUB_ROWS = SUB_N / 2;                   // its weight rows in one CTA
    static constexpr int SUB_BYTES = SUB_ROWS * TILE_K * 2;
    static constexpr int HALF_N = TILE_N / 2;                    // weight rows per CTA
    static constexpr int X_BYTES = UMMA_M * TILE_K * 2;
    static constexpr int W_BYTES = HALF_N * TILE_K * 2;
    static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
    static constexpr int STAGING = REDUCE ? 8 * RED_BYTES : 0;
    static constexpr int BUDGET = 227 * 1024 - 1024 - 512 - STAGING;
    static constexpr int STAGES = BUDGET / STAGE_BYTES > 8 ? 8 : BUDGET / STAGE_BYTES;
    static constexpr int TMEM_COLS = TILE_N <= 128 ? 128 : (TILE_N <= 256 ? 256 : 512);
    static constexpr int ACCS = TILE_N <= 256 ? 2 : 1;           // accumulators in tensor memory
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + STAGING + 1024 + 512;
    static_assert(SUB_N % 16 == 0 && SUB_ROWS % 8 == 0 && SUB_N <= 256, "one MMA of the pair");
    static_assert(STAGE_BYTES % 1024 == 0 && SUB_BYTES % 1024 == 0, "swizzled tiles start on 1,024 bytes");
};

template <int TILE_N, bool REDUCE, bool HEADS = false>
__global__ void __launch_bounds__(THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_c, const Params p) {
    using C = CfgPair<TILE_N, REDUCE>;
    static_assert(TILE_N % RED_BOX == 0 && TILE_N >= 2 * RED_BOX && TILE_N <= 320, "feature tile");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = tiles + (size_t)C::STAGES * C::STAGE_BYTES;        // 1024-byte aligned
    uint64_t* full = (uint64_t*)(staging + C::STAGING);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;        // [2] (one in use with a single accumulator)
    uint64_t* acc_empty = acc_full + 2;            // [2], used in the first CTA only
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_kb = (p.K + TILE_K - 1) / TILE_K;
    const int m_tiles = (p.tokens + 2 * UMMA_M - 1) / (2 * UMMA_M);
    const int n_tiles = (p.features + TILE_N - 1) / TILE_N;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(&full[s], 1); mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 16); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, C::ACCS * C::TMEM_COLS);
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                             // the other CTA's barriers exist before anyone arrives on them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0 && pair < total_tiles) {
            const int ahead = min(n_kb, C::STAGES);
            {
                const int f0 = (pair / m_tiles) * TILE_N + (int)rank * C::SUB_ROWS;
                const int t0 = (pair % m_tiles) * (2 * UMMA_M) + (int)rank * UMMA_M;
                for (int i = 0; i < ahead; ++i) {
                    if (rank == 0) mbar_expect_tx(&full[i], 2 * C::STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < C::SUBS; ++j)
                        tma_load_2d_pair(tiles + (size_t)i * C::STAGE_BYTES + C::X_BYTES + j * C::SUB_BYTES, &map_w,
                                         mbar_in_cta(&full[i], 0), i * TILE_K, f0 + j * C::SUB_N);
                }
                pdl_wait();
                for (int i = 0; i < ahead; ++i)
                    tma_load_2d_pair(tiles + (size_t)i * C::STAGE_BYTES, &map_x, mbar_in_cta(&full[i], 0), i * TILE_K,
                                     t0);
            }
            int it = ahead;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
                const int f0 = (tile / m_tiles) * TILE_N + (int)rank * C::SUB_ROWS;
                const int t0 = (tile % m_tiles) * (2 * UMMA_M) + (int)rank * UMMA_M;
                for (int i = (tile == pair ? ahead : 0); i < n_kb; ++i, ++it) {
                    const int s = it % C::STAGES;
                    if (it >= C::STAGES && !mbar_wait(&empty[s], ((it / C::STAGES) & 1) ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* xt = tiles + (size_t)s * C::STAGE_BYTES;
                    const uint32_t bar = mbar_in_cta(&full[s], 0);
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * C::STAGE_BYTES);
                    tma_load_2d_pair(xt, &map_x, bar, i * TILE_K, t0);
#pragma unroll
                    for (int j = 0; j < C::SUBS; ++j)
                        tma_load_2d_pair(xt + C::X_BYTES + j * C::SUB_BYTES, &map_w, bar, i * TILE_K, f0 + j * C::SUB_N);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ------------------------------------------------------------ MMA issuer (first CTA)
            constexpr uint32_t idesc = umma_idesc(2 * UMMA_M, C::SUB_N);
            int it = 0, tile_iter = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++tile_iter) {
                const int b = tile_iter % C::ACCS, use = tile_iter / C::ACCS;
                if (tile_iter >= C::ACCS && !mbar_wait(&acc_empty[b], (use & 1) ^ 1, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + b * C::TMEM_COLS;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1;
                    if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t xa = smem_u32(tiles + (size_t)s * C::STAGE_BYTES);
                    const uint64_t xd = umma_smem_desc(xa), wd = umma_smem_desc(xa + C::X_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k) {
#pragma unroll
                        for (int j = 0; j < C::SUBS; ++j)
                            umma_bf16_pair(acc + j * C::SUB_N, xd + 2 * k, wd + j * (C::SUB_BYTES >> 4) + 2 * k, idesc,
                                           (i | k) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[b]);
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue warps 2..9 (both CTAs)
        const int q = warp & 3;                    // tensor-memory lane quarter = 32 tokens
        const int cg = (warp - 2) >> 2;            // half of the feature columns
        pdl_wait();
        uint8_t* box = staging + (size_t)(warp - 2) * RED_BYTES;
        int tile_iter = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles; tile += n_pairs, ++tile_iter) {
            const int b = tile_iter % C::ACCS, use = tile_iter / C::ACCS;
            const int t_warp = (tile % m_tiles) * (2 * UMMA_M) + (int)rank * UMMA_M + q * 32;
            const int f0 = (tile / m_tiles) * TILE_N;
            bf16* head_dst = nullptr;
            if constexpr (HEADS) head_dst = sink_dst(p, t_warp + lane, f0 / SINK_HEAD + cg);
            if (ok && !mbar_wait(&acc_full[b], use & 1, abort_flag)) ok = false;
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + b * C::TMEM_COLS + ((uint32_t)(q * 32) << 16);
            tokm_epilogue_tile<TILE_N, REDUCE, HEADS>(p, &map_c, taddr, box, t_warp, f0, cg, lane, ok, head_dst);
            // this warp has read its part of the accumulator: hand it back to the first CTA
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(&acc_empty[b]);
                else mbar_arrive_remote(&acc_empty[b], 0);
            }
        }
        if (REDUCE && lane == 0) bulk_wait_all();
    }
    tcgen05_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(&p.status[1], 1);
    cluster_sync_all();                             // no MMA of the pair is in flight, no arrival under way
    if (warp == 1) tmem_dealloc_pair(tmem_base, C::ACCS * C::TMEM_COLS);
}

// ------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)ptr;
    });
    return fn;
}

struct MapKey {
    const void* ptr; int rows, cols; long long ld; int box_rows;   // box_rows < 0: float32 box for the reducing store
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld;   h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// Row-major bf16 [rows, cols] with leading dimension ld; box = [box_rows, 64].
// f32_box: row-major float32 instead, box = [RED_BOX, RED_BOX].
int make_map(CUtensorMap* out, const void* ptr, int rows, int cols, long long ld, int box_rows,
             bool f32_box = false) {
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, ld, f32_box ? -RED_BOX : box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiled fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (f32_box ? 4 : 2)};
    cuuint32_t box[2] = {(cuuint32_t)(f32_box ? RED_BOX : TILE_K), (cuuint32_t)(f32_box ? RED_BOX : box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, f32_box ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

template <int TILE_T, int TILE_F>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid, cudaStream_t s) {
    using C = Cfg<TILE_T, TILE_F>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TILE_T, TILE_F>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return kipp_launch(gemm_tc_kernel<TILE_T, TILE_F>, grid, dim3(THREADS), C::SMEM, s, p.splits, mw, mx, p);
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

template <int TILE_N, bool REDUCE>
int launch_tokm(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mc, const Params& p, int total,
                cudaStream_t s) {
    using C = CfgTok<TILE_N, REDUCE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_tokm_kernel<TILE_N, REDUCE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // persistent: at most one CTA per SM
    const int sms = sm_count();
    return kipp_launch(gemm_tc_tokm_kernel<TILE_N, REDUCE>, dim3(total < sms ? total : sms), dim3(THREADS), C::SMEM,
                       s, 1, mw, mx, mc, p);
}
template <bool REDUCE>
int launch_tokm_n(int tile_n, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mc, const Params& p,
                  int total, cudaStream_t s) {
    switch (tile_n) {
    case 128: return launch_tokm<128, REDUCE>(mw, mx, mc, p, total, s);
    case 160: return launch_tokm<160, REDUCE>(mw, mx, mc, p, total, s);
    case 192: return launch_tokm<192, REDUCE>(mw, mx, mc, p, total, s);
    case 224: return launch_tokm<224, REDUCE>(mw, mx, mc, p, total, s);
    case 256: return launch_tokm<256, REDUCE>(mw, mx, mc, p, total, s);
    }
    return KIPP_ERR_ARG;
}

template <int TILE_N, bool REDUCE, bool HEADS = false>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mc, const Params& p, int total,
                cudaStream_t s) {
    using C = CfgPair<TILE_N, REDUCE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<TILE_N, REDUCE, HEADS>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // persistent: at most one pair of CTAs per pair of SMs
    const int pairs = sm_count() / 2;
    // the two CTAs of an MMA pair are neighbours along x
    return kipp_launch_cluster(gemm_tc_pair_kernel<TILE_N, REDUCE, HEADS>, dim3(2 * (total < pairs ? total : pairs)),
                               dim3(THREADS), C::SMEM, s, dim3(2, 1, 1), mw, mx, mc, p);
}
template <bool REDUCE>
int launch_pair_n(int tile_n, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mc, const Params& p,
                  int total, cudaStream_t s) {
    switch (tile_n) {
    case 128: return launch_pair<128, REDUCE>(mw, mx, mc, p, total, s);
    case 160: return launch_pair<160, REDUCE>(mw, mx, mc, p, total, s);
    case 192: return launch_pair<192, REDUCE>(mw, mx, mc, p, total, s);
    case 224: return launch_pair<224, REDUCE>(mw, mx, mc, p, total, s);
    case 256: return launch_pair<256, REDUCE>(mw, mx, mc, p, total, s);
    case 288: return launch_pair<288, REDUCE>(mw, mx, mc, p, total, s);
    case 320: return launch_pair<320, REDUCE>(mw, mx, mc, p, total, s);
    }
    return KIPP_ERR_ARG;
}

// Feature tile of the persistent kernel: the CTAs take the tiles in rounds, so
// the cost is rounds x (time of a tile); a tile's time grows with its width
// plus a fixed part.  For 2,048 tokens x 2,560 features, 256 wide gives 160
// tiles = two rounds of which the second is nearly empty; 160 wide gives 256
// tiles = two well-filled rounds of shorter tiles.
// `pair`: tiles of 256 tokens, taken in rounds by the pairs of SMs.
// Tiles wider than 256 (pairs only) have one accumulator, so their epilogue is not hidden
// behind the next tile's MMAs: they are taken only where they make the whole product one round.
int pick_tile_n(int tokens, int features, bool pair = false, long long* cost_out = nullptr) {
    const int units = pair ? sm_count() / 2 : sm_count();
    const int rows = pair ? 2 * UMMA_M : UMMA_M;
    const int m_tiles = (tokens + rows - 1) / rows;
    int best = 256;
    long long best_cost = -1;
    for (int n = pair ? 320 : 256; n >= 128; n -= 32) {
        const long long tiles = (long long)m_tiles * ((features + n - 1) / n);
        const long long rounds = (tiles + units - 1) / units;
        if (n > 256 && rounds > 1) continue;
        const long long cost = rounds * (n + TOKM_TILE_FIXED);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = n; }
    }
    if (cost_out) *cost_out = best_cost;
    return best;
}

// Tile choice, from measurements on B200: 128 features with a token tile of 16,
// 32 or 64 (two CTAs per SM, one's epilogue under the other's MMAs), 256 tokens
// from 1,024 tokens on.  256 features x 256 tokens per CTA (two accumulators,
// all 512 tensor-memory columns) is built and selectable but measured no faster
// than 128 x 256 here, so it is not chosen by default.
void pick_tiles(int tokens, int features, int* tile_t, int* tile_f) {
    *tile_f = 128;
    if (tokens <= 16) *tile_t = 16;
    else if (tokens <= 32) *tile_t = 32;
    else if (tokens >= 1024) *tile_t = 256;
    else *tile_t = 64;
}
}  // namespace

// The token tile, feature tile and number of K splits (= cluster size, at most
// 8) the kernel uses for a shape; a want_* of 0 lets it choose.
extern "C" int kipp_gemm_tc_plan(int tokens, int features, int K, int want_splits, int want_tile,
                                 int want_tile_f, int* tile_t_out, int* tile_f_out, int* splits_out) {
    int tile_t, tile_f;
    pick_tiles(tokens, features, &tile_t, &tile_f);
    if (want_tile == 16 || want_tile == 32 || want_tile == 64 || want_tile == 128 || want_tile == 256) {
        tile_t = want_tile;
        if (tile_t != 256) tile_f = 128;
    }
    if (want_tile_f == 128) tile_f = 128;
    if (want_tile_f == 256 && tile_t == 256) tile_f = 256;
    const int f_tiles = (features + tile_f - 1) / tile_f;
    const int t_tiles = (tokens + tile_t - 1) / tile_t;
    const int kb = (K + TILE_K - 1) / TILE_K;
    int splits = want_splits;
    if (splits <= 0) {
        // Few tiles: split K so that tiles x splits comes close to, but stays
        // under, what is resident at once with clusters (measured: 48 tiles run
        // fastest with 5 splits = 240 CTAs, slower with 6 = 288; 20 tiles with 8).
        // Every split keeps at least 4 K blocks.
        const int tiles = f_tiles * t_tiles;
        splits = 1;
        if (tiles <= 128) {
            splits = 256 / tiles;
            if (splits > kb / 4) splits = kb / 4;
        }
    }
    if (tile_f != 128) splits = 1;                     // the cluster reduction holds one accumulator
    if (splits > 8) splits = 8;
    if (splits > kb) splits = kb;
    if (splits < 1) splits = 1;
    const int per = (kb + splits - 1) / splits;
    splits = (kb + per - 1) / per;                     // no empty split
    if (splits < 1) splits = 1;
    *tile_t_out = tile_t;
    *tile_f_out = tile_f;
    *splits_out = splits;
    return 0;
}

// C (+)= X W^T.  X [tokens, K] bf16 (ldx), W [features, K] bf16 (ldw), C float32
// or bf16 (ldc).  Pointers 16-byte aligned, ldx and ldw multiples of 8.
// What folds an RMSNorm into the products around it (the few-token kernel only; see Params).
struct kipp_gemm_norm_fold {
    const void* norm_w;       // EPI_ADD: weight of the norm that follows the add, or NULL
    int norm_w_dtype;
    void* xn;                 //   bf16 [tokens, ldn]: new residual x that weight, without the per-token factor
    long long ldn;
    float* ssq_out;           //   float32 [tokens, features / 32]: sums of squares of the new residual
    const float* ssq_in;      // store / SwiGLU: such sums for this product's input rows, or NULL
    int ssq_in_slots;
    float inv_n, eps;         //   the factor is 1 / sqrt(sum * inv_n + eps)
};

// Whether a residual add of this many tokens can leave what the next norm needs (norm_w; prompt-
// sized batches run the other kernels, whose add goes out as reducing stores that never see the
// new value).  Row factors (ssq_in) are taken at every size.
extern "C" int kipp_gemm_tc_fold_ok(int tokens) { return tokens > 0 && tokens < 512; }

extern "C" int kipp_gemm_tc_fold(void* C, int out_dtype, const void* X, const void* W, int tokens, int features,
                                 int K, long long ldx, long long ldw, long long ldc, int epilogue, int splits,
                                 int want_tile, int want_tile_f, const kipp_gemm_norm_fold* fold, int* status,
                                 void* stream);

// Whether a fused q/k/v projection of this many tokens can hand its heads straight to attention
// (kipp_gemm_tc_heads): the kernel that does it is the one for prompt-sized batches, its tile holds
// two heads of 128, and the rotation covers the whole head or nothing.
extern "C" int kipp_gemm_tc_heads_ok(int tokens, int head_dim, int rotary_dim) {
    return tokens >= 1024 && head_dim == SINK_HEAD && (rotary_dim == 0 || rotary_dim == head_dim);
}

namespace {
int gemm_tc_run(void* C, int out_dtype, const void* X, const void* W, int tokens, int features, int K, long long ldx,
                long long ldw, long long ldc, int epilogue, int splits, int want_tile, int want_tile_f,
                const kipp_gemm_norm_fold* fold, const kipp_gemm_head_sink* sink, int* status, void* stream);
}

// X W^T of a fused q/k/v projection whose rows go on as `sink` says; nothing is stored as a
// product.  `fold` may carry the row factors of a deferred norm (ssq_in), as in kipp_gemm_tc_fold.
extern "C" int kipp_gemm_tc_heads(const void* X, const void* W, int tokens, int features, int K, long long ldx,
                                  long long ldw, const kipp_gemm_norm_fold* fold, const kipp_gemm_head_sink* sink,
                                  int* status, void* stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (sink == nullptr || !kipp_gemm_tc_heads_ok(tokens, SINK_HEAD, 0)) return KIPP_ERR_ARG;
    if (sink->n_q <= 0 || sink->n_kv <= 0 || features != (sink->n_q + 2 * sink->n_kv) * SINK_HEAD) return KIPP_ERR_ARG;
    if (sink->page_size <= 0 || sink->table_width < 0) return KIPP_ERR_ARG;
    if ((sink->q_norm_w == nullptr) != (sink->k_norm_w == nullptr)) return KIPP_ERR_ARG;
    if (sink->norm_dtype != KIPP_DT_F32 && sink->norm_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    if (((uintptr_t)sink->q_out | (uintptr_t)sink->k_pages | (uintptr_t)sink->v_pages | (uintptr_t)sink->q_norm_w |
         (uintptr_t)sink->k_norm_w | (uintptr_t)sink->cos_sin) & 15)
        return -3;
    if (fold != nullptr && fold->norm_w != nullptr) return KIPP_ERR_ARG;
    return gemm_tc_run(nullptr, KIPP_DT_BF16, X, W, tokens, features, K, ldx, ldw, features, EPI_STORE, 0, 0, 0, fold,
                       sink, status, stream);
}

extern "C" int kipp_gemm_tc(void* C, int out_dtype, const void* X, const void* W, int tokens, int features,
                            int K, long long ldx, long long ldw, long long ldc, int epilogue, int splits,
                            int want_tile, int want_tile_f, int* status, void* stream) {
    return kipp_gemm_tc_fold(C, out_dtype, X, W, tokens, features, K, ldx, ldw, ldc, epilogue, splits, want_tile,
                             want_tile_f, nullptr, status, stream);
}

extern "C" int kipp_gemm_tc_fold(void* C, int out_dtype, const void* X, const void* W, int tokens, int features,
                                 int K, long long ldx, long long ldw, long long ldc, int epilogue, int splits,
                                 int want_tile, int want_tile_f, const kipp_gemm_norm_fold* fold, int* status,
                                 void* stream) {
    return gemm_tc_run(C, out_dtype, X, W, tokens, features, K, ldx, ldw, ldc, epilogue, splits, want_tile,
                       want_tile_f, fold, nullptr, status, stream);
}

namespace {
int gemm_tc_run(void* C, int out_dtype, const void* X, const void* W, int tokens, int features, int K, long long ldx,
                long long ldw, long long ldc, int epilogue, int splits, int want_tile, int want_tile_f,
                const kipp_gemm_norm_fold* fold, const kipp_gemm_head_sink* sink, int* status, void* stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (fold != nullptr) {
        if (fold->norm_w != nullptr &&
            (!kipp_gemm_tc_fold_ok(tokens) || want_tile_f < 0 || epilogue != EPI_ADD || fold->xn == nullptr || fold->ssq_out == nullptr || (features % 32) ||
             (fold->norm_w_dtype != KIPP_DT_F32 && fold->norm_w_dtype != KIPP_DT_BF16)))
            return KIPP_ERR_ARG;
        if (fold->ssq_in != nullptr && (epilogue == EPI_ADD || fold->ssq_in_slots <= 0)) return KIPP_ERR_ARG;
    }
    if (K <= 0) return KIPP_ERR_ARG;
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return -3;
    if (epilogue == EPI_ADD && out_dtype != KIPP_DT_F32) return KIPP_ERR_DTYPE;
    if (epilogue == EPI_SWIGLU && (features & 1)) return KIPP_ERR_ARG;
    if (out_dtype != KIPP_DT_F32 && out_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    // Prompt-sized batches: tokens as the M operand (want_tile_f < 0 forces it with
    // the feature tile -want_tile_f).  The residual add needs a tensor map over C.
    const bool c_map_ok = epilogue != EPI_ADD || (ldc % 4 == 0 && ((uintptr_t)C & 15) == 0);
    // Between 33 and 511 tokens a store or SwiGLU product also goes this way where its tiles of 128
    // tokens fill most of the SMs: the few-token kernel streams the weights once per 64 tokens, and
    // even at one pass its 128-feature tiles lose against one round of wider tiles here (gate/up
    // 19,456 x 2,560: 19.3 against 22.6 us at 64 tokens, 19.7 against 36.4 at 128, 45.7 against 85.2
    // at 511; the head 151,936 x 2,560: 120 against 129 us at 64 tokens, 200 against 292 at 256;
    // q/k/v 6,144 x 2,560, 39 to 48 tiles: 14.3 against 10.9 us, so it stays).  The residual add stays
    // with the few-token kernel up to 511 tokens (9.8 against 21 us at 64 tokens, even at 511).
    bool mid_fills = false;
    if (splits == 0 && want_tile == 0 && want_tile_f == 0 && tokens > 32 && tokens < 512 && epilogue != EPI_ADD) {
        const int n = pick_tile_n(tokens, features, false);
        const long long tiles = (long long)((tokens + UMMA_M - 1) / UMMA_M) * ((features + n - 1) / n);
        mid_fills = 4 * tiles >= 3LL * sm_count();
    }
    if ((want_tile == 0 && want_tile_f == 0 && tokens >= 512 && c_map_ok) || want_tile_f < 0 || mid_fills) {
        const bool reduce = epilogue == EPI_ADD && c_map_ok;     // else a thread per token adds in place
        // want_tile_f: -N = one CTA per tile, -(1000 + N) = a pair of CTAs per 256-token tile
        // By default: the pair kernel from 1,024 tokens on, except for the residual
        // add (measured 8-12 % faster for store and SwiGLU at 1,024 and 2,048 tokens,
        // no faster for the add, whose 2,560-feature shapes are bound by the rounds).
        // The residual add (2,560-feature shapes here) is bound by the rounds, so there the pair
        // is taken only where its tiles make fewer of them: 2,048 x 2,560 as 8 x 9 tiles of 288
        // features is one round of 72 pairs (measured 34.9 against 42.5 us at K = 4,096 and 77.0
        // against 94.8 us at K = 9,728).
        long long cost_pair = 0, cost_one = 0;
        const int n_pair = pick_tile_n(tokens, features, true, &cost_pair);
        const int n_one = pick_tile_n(tokens, features, false, &cost_one);
        // (From 1,536 tokens on the pair also takes the add where the rounds tie: sweeps over 768 to
        // 4,096 tokens at 2,560, 6,144 and 19,456 features, K 2,560 to 9,728: the pair's tiles of 224
        // or 256 features 6 to 13 % ahead at 1,536, 3,072 and 4,096 tokens, one CTA per tile 4 to 7 %
        // ahead at 1,024.)
        const bool add_pair = tokens >= 1536 ? cost_pair <= cost_one : cost_pair < cost_one;
        const bool pair = sink != nullptr || (want_tile_f < 0 ? want_tile_f <= -1000
                                                              : (tokens >= 1024 && (epilogue != EPI_ADD || add_pair)));
        const int tile_n = sink != nullptr        ? 2 * SINK_HEAD
                           : want_tile_f <= -1000 ? -want_tile_f - 1000
                           : want_tile_f < 0      ? -want_tile_f
                                                  : (pair ? n_pair : n_one);
        if (tile_n < 128 || tile_n > (pair ? 320 : 256) || tile_n % 32) return KIPP_ERR_ARG;
        CUtensorMap mw, mx, mc;
        // a CTA of a pair loads its half of the weight rows of each MMA (two MMAs above 256 features)
        int rc = make_map(&mw, W, features, K, ldw, pair ? (tile_n > 256 ? tile_n / 4 : tile_n / 2) : tile_n);
        if (rc) return rc;
        rc = make_map(&mx, X, tokens, K, ldx, UMMA_M);
        if (rc) return rc;
        if (reduce) {
            rc = make_map(&mc, C, tokens, features, ldc, RED_BOX, true);
            if (rc) return rc;
        } else {
            mc = mw;                                    // unused
        }
        Params p = {};
        p.C = C; p.out_dtype = out_dtype; p.epilogue = epilogue;
        p.tokens = tokens; p.features = features; p.K = K; p.ldc = ldc;
        p.k_blocks_per_split = (K + TILE_K - 1) / TILE_K; p.splits = 1; p.status = status;
        if (fold != nullptr && fold->ssq_in != nullptr) {
            p.ssq_in = fold->ssq_in; p.ssq_in_slots = fold->ssq_in_slots;
            p.inv_n = fold->inv_n; p.eps = fold->eps;
        }
        const int rows = pair ? 2 * UMMA_M : UMMA_M;
        const long long total = (long long)((tokens + rows - 1) / rows) * ((features + tile_n - 1) / tile_n);
        if (total > 0x7fffffffLL) return KIPP_ERR_ARG;
        cudaStream_t s = (cudaStream_t)stream;
        if (sink != nullptr) {
            p.heads = *sink;
            return launch_pair<2 * SINK_HEAD, false, true>(mw, mx, mc, p, (int)total, s);
        }
        if (pair)
            return reduce ? launch_pair_n<true>(tile_n, mw, mx, mc, p, (int)total, s)
                          : launch_pair_n<false>(tile_n, mw, mx, mc, p, (int)total, s);
        return reduce ? launch_tokm_n<true>(tile_n, mw, mx, mc, p, (int)total, s)
                      : launch_tokm_n<false>(tile_n, mw, mx, mc, p, (int)total, s);
    }
    int tile_t, tile_f, planned;
    kipp_gemm_tc_plan(tokens, features, K, splits, want_tile, want_tile_f, &tile_t, &tile_f, &planned);
    splits = planned;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, features, K, ldw, tile_f);
    if (rc) return rc;
    rc = make_map(&mx, X, tokens, K, ldx, tile_t);
    if (rc) return rc;
    Params p = {};
    p.C = C; p.out_dtype = out_dtype; p.epilogue = epilogue;
    p.tokens = tokens; p.features = features; p.K = K; p.ldc = ldc;
    const int kb = (K + TILE_K - 1) / TILE_K;
    p.k_blocks_per_split = (kb + splits - 1) / splits;
    p.splits = splits; p.status = status;
    if (fold != nullptr) {
        if (fold->norm_w != nullptr) {
            p.norm_w = fold->norm_w; p.norm_w_dtype = fold->norm_w_dtype;
            p.xn = (bf16*)fold->xn; p.ldn = fold->ldn;
            p.ssq_out = fold->ssq_out; p.ssq_slots = features / 32;
        }
        if (fold->ssq_in != nullptr) {
            p.ssq_in = fold->ssq_in; p.ssq_in_slots = fold->ssq_in_slots;
            p.inv_n = fold->inv_n; p.eps = fold->eps;
        }
    }
    dim3 grid((tokens + tile_t - 1) / tile_t, (features + tile_f - 1) / tile_f, splits);
    if (grid.y > 65535) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (tile_f == 256) return launch<256, 256>(mw, mx, p, grid, s);
    switch (tile_t) {
    case 16: return launch<16, 128>(mw, mx, p, grid, s);
    case 32: return launch<32, 128>(mw, mx, p, grid, s);
    case 64: return launch<64, 128>(mw, mx, p, grid, s);
    case 128: return launch<128, 128>(mw, mx, p, grid, s);
    default: return launch<256, 128>(mw, mx, p, grid, s);
    }
}
}  // namespace
