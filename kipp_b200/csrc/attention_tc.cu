// Causal grouped-query attention of prompt portions over the paged cache on the
// 5th-generation tensor cores: both products (scores = Q K^T and output = P V)
// are tcgen05.mma with their accumulators in tensor memory.
//
// Reference counterpart: cached_gqa_kernel (cuda/kipp_kernels.cu:160), formula
// src/kipp.c:2882-2922 (scores (q.k)/sqrt(D) over the keys a token may see,
// softmax with the maximum subtracted, weighted sum of values).
//
// One CTA = 128 consecutive tokens of one entry x one query head, 10 warps:
//   warps 0-7  softmax: threads r and r + 128 share query row r, each takes 32 of
//              a tile's 64 keys (scores straight from tensor memory, lane = row)
//              and half of the output columns;
//   warp 8     gathers the key and value tiles page by page with TMA (one box
//              per lane, 128-byte swizzle) into a two-stage ring;
//   warp 9     one thread issues the score products S = Q K^T;
//   warp 10    one thread issues the output products O += P V.
// (Two issuing threads: one thread that waited for four barriers and issued twelve
// products and five commits per tile took 1,700 cycles for that, sharing its scheduler
// with busy softmax warps, while the tensor pipe needs 512 per tile and the softmax
// warps 900: the issuing thread was the kernel's bottleneck.  The two chains, scores
// and outputs, meet only through the softmax warps.)
// Per tile of 64 keys: S = Q K^T (128 x 64 x D) into one of two score buffers in
// tensor memory, up to two tiles ahead of the softmax threads; these take their scores
// into registers, scale, mask, take the running maximum (exchanged between the two
// threads of a row through shared memory) and form p = 2^(s - m), which goes as
// bfloat16 over the first half of the tile's own score buffer (the buffer is free for
// the scores of tile i + 2 when O += P V of tile i has read it).  The running maximum
// moves only when a tile exceeds
// it by more than 2^8 (numerator and denominator carry the same reference), so the
// output accumulator in tensor memory is rescaled rarely.  O += P V (128 x D x 64)
// takes P from tensor memory and V as an MN-major shared-memory operand; it runs
// while the next tile is in the softmax.  Everything is handed over through
// mbarriers; every wait is bounded in time, and on a time-out status[1] is set
// and the CTA drains and frees its tensor memory.  Two CTAs fit an SM (98 KB
// shared memory, 256 tensor-memory columns each: 2 x 64 scores with the weights
// inside, 128 output).  All arithmetic outside the MMAs is float32.
//
// The gather costs one TMA box per page and 64-column half (with 16-slot pages 16
// boxes of 2 KB a tile; the kernel is then 3 % slower than with pages of 64 slots,
// with 8-slot pages 40 %), unless the pages of a tile follow one another in the pool,
// as those of a request that grew without interruption do: then the tile comes as
// one box per half, from a 4-dimensional map [page][kv head][slot][column].
//
// Keys beyond a row's limits are masked after the product, so whole pages are
// fetched; rows of a tile without a page are fetched from beyond the end of the
// pool, where the TMA unit fills zeros.  A masked value row is multiplied by a
// weight of exactly zero: the pool must hold finite numbers everywhere (it is
// created zeroed and only ever holds keys and values).
//
// Sizes: head_dim 64 or 128; page size 8, 16, 32 or a multiple of 64.  Cache
// layout of a layer: [page][kv_head][slot][D].
#include "common.cuh"
#include "mbarrier.cuh"
#include <cuda.h>
#include <math.h>
#include <mutex>
#include <unordered_map>

namespace {
constexpr int BM = 128;            // query rows per CTA = MMA M
constexpr int BN = 64;             // keys per tile
constexpr float RESCALE_SLACK = 8.f;   // log2 of the largest weight a stale running maximum may give
constexpr int SOFTMAX_THREADS = 256;  // two threads per query row: each half of a tile's keys
constexpr int THREADS = 352;          // + the TMA warp and the two MMA warps

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) { return kipp_mbar_try_wait(bar, parity); }
// bounded in time (mbarrier.cuh): false when the wait ran out or another thread of the CTA gave up
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return kipp_mbar_wait_limited(bar, parity, abort_flag, KIPP_WAIT_LIMIT_CYCLES);
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// A box from shared memory to a 2-dimensional map (what lies outside the tensor is dropped).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the sources of all earlier bulk-groups of this thread have been read
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Box of a 4-dimensional map: columns x, slot y, kv head z, page w.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                            int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
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
// 16 columns of raw 32-bit words (pairs of bfloat16) into this thread's lane.
__device__ __forceinline__ void tmem_st16_words(uint32_t taddr, const uint32_t* w) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]),
          "r"(w[8]), "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15])
        : "memory");
}
// Barrier among `count` threads (whole warps) that all name `id` (1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// D (+)= A B with A in tensor memory (lane = row, a column = two bfloat16 of K) and B in shared memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 2^x, single instruction (flushes denormals to zero: such weights do not matter in a sum of weights <= 1)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// true in one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
    return chosen != 0;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Two float32 operations in one instruction, a maximum of three (sm_100): the softmax warps
// stand in the chain from a tile's scores to the next but one's, instruction by instruction.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)),
        "l"(*reinterpret_cast<unsigned long long*>(&b)), "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long*>(&a)),
        "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

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
    bf16* out; const bf16* q;   // keys and values come through the tensor maps
    const int* q_start; const int* context_len; const int* block_table;
    const int* work;            // [items][2] = (entry, first token of the tile within the entry)
    int table_width, page_size, n_q, n_kv, window;
    int box_rows;               // rows of one TMA box = min(page_size, 64)
    int pages_per_box;          // > 1: pages of fewer than 64 slots; a tile whose pages follow one another
                                // in the pool comes as one box per 64-column half (the 4-dimensional maps)
    int rows_total;             // pages x kv heads x page_size: a row coordinate from here on reads zeros
    float scale_log2;
    uint32_t v_lbo, v_sbo;      // descriptor strides of the MN-major value tile
    int* status;
};

template <int D> struct Cfg {
    static constexpr int HALVES = D / 64;
    static constexpr int Q_BYTES = BM * D * 2;
    static constexpr int KV_BYTES = BN * D * 2;       // one of K or V, one stage
    static constexpr int XCHG_BYTES = 2 * 2 * BM * 4;  // row maxima of the two halves, two parities
    static constexpr int TMEM_COLS = 256;                       // two score buffers (64 each) + O (D), power of two
    // 100,480 bytes at head_dim 128: two CTAs (plus the 1 KB the system keeps per CTA) fit in 227 KB
    static constexpr size_t SMEM = Q_BYTES + 4 * KV_BYTES + XCHG_BYTES + 144;   // 16 barriers, 2 words
};

template <int D>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __grid_constant__ CUtensorMap map_k4, const __grid_constant__ CUtensorMap map_v4,
                       const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_out,
                       const Params p) {
    using C = Cfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];     // swizzled tiles need 1024-byte alignment
    const uint32_t q_tile = smem_u32(smem);
    const uint32_t k_tiles = q_tile + C::Q_BYTES;                  // [2 stages]
    const uint32_t v_tiles = k_tiles + 2 * C::KV_BYTES;            // [2 stages]
    float* xchg = reinterpret_cast<float*>(smem + C::Q_BYTES + 4 * C::KV_BYTES);      // [parity][half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::Q_BYTES + 4 * C::KV_BYTES + C::XCHG_BYTES);
    uint64_t* q_full = bars;            // the query tile is in shared memory            (1 + bytes)
    uint64_t* k_full = bars + 1;        // [2] a key stage has landed                    (1 + bytes)
    uint64_t* k_empty = bars + 3;       // [2] its S product has read it                 (1, by commit)
    uint64_t* v_full = bars + 5;        // [2]
    uint64_t* v_empty = bars + 7;       // [2] its O product has read it
    uint64_t* s_full = bars + 9;        // [2] a score buffer holds S of a tile           (1, by commit)
    uint64_t* p_full = bars + 11;       // [2] a weight buffer holds a tile's weights, O is rescaled (8)
    uint64_t* p_empty = bars + 13;      // [2] O += P V has read it (and is complete)     (1, by commit)
    uint64_t* o_final = bars + 15;      // the last O += P V is complete                  (1, by commit)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    pdl_launch_dependents();
    // (What is read before the dependency wait below comes with the step's lists, which a
    // copy brought before any kernel of the step started: the loads, three in a row, run
    // while the barriers and the tensor memory are set up.)
    // Grid (heads, tiles), the last tile of the list first: within an entry the later
    // tiles see more keys, and the long ones should not be the last to start; the
    // heads of a tile, which share its keys and values, start together.
    const int item = gridDim.y - 1 - blockIdx.y;
    const int entry = p.work[2 * item], tile_tok = p.work[2 * item + 1];
    const int h = blockIdx.x, g = h / (p.n_q / p.n_kv);
    const int qs = p.q_start[entry], q_len = p.q_start[entry + 1] - qs;
    const int ctx = p.context_len[entry];
    // keys the tile may see: from the first token's window start to the last token
    const int tile_first = ctx + tile_tok, tile_last = ctx + min(tile_tok + BM - 1, q_len - 1);
    const int lo = p.window > 0 ? max(0, tile_first - p.window + 1) : 0, hi = tile_last;
    const int first_tile = lo / BN, last_tile = hi / BN;
    const int n_tiles = last_tile - first_tile + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&k_full[b], 1); mbar_init(&k_empty[b], 1);
            mbar_init(&v_full[b], 1); mbar_init(&v_empty[b], 1);
            mbar_init(&p_full[b], SOFTMAX_THREADS / 32); mbar_init(&p_empty[b], 1);
        }
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(o_final, 1);
        *abort_flag = (q_tile & 1023u) ? 1 : 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // columns: two score buffers [0, 64) and [64, 128); the weights of a tile (pairs of
    // bfloat16, 32 columns) overwrite the first half of the tile's own score buffer once
    // its scores are in registers; output [128, 128 + D)
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * BN;
    pdl_wait();


    if (warp == 8) {
        // ------------------------------------------------------------ TMA producer
        // Lane l fetches box l of a tile: rows [rb * box_rows, + box_rows) of the
        // 64-column half `half`; the rows of a box lie in one page.
        const int* table = p.block_table + (size_t)entry * p.table_width;
        const int rb = lane / C::HALVES, half = lane % C::HALVES;
        const bool has_box = rb * p.box_rows < BN;
        const uint32_t dst_off = (uint32_t)(half * (BN * 128) + rb * p.box_rows * 128);
        bool ok = true;
        // The query tile first: rows [qs + tile_tok, + 128) of head h, a box per 64-column half.
        // Rows past the entry's end are another entry's queries (or zeros past the step's last
        // token): their scores are masked and their output rows are never stored.
        if (lane == 0) mbar_expect_tx(q_full, C::Q_BYTES);
        __syncwarp();
        if (lane < C::HALVES) tma_load_2d(q_tile + lane * (BM * 128), &map_q, q_full, h * D + lane * 64, qs + tile_tok);
        // (This warp shares its scheduler with busy softmax warps and the stages come
        // back to it just in time: every instruction between a stage's release and
        // the issue of its load counts, so what can be is computed before the loop.)
        if (p.pages_per_box > 1) {
            // Pages of 8, 16 or 32 slots: a box is one page (box_rows = page_size), the
            // boxes of a tile are the table entries kt * pages_per_box + rb.  When those
            // pages follow one another in the pool (a request that grew without
            // interruption), the tile comes as one box per half from the 4-dimensional
            // map instead (a box costs the TMA unit about as much whatever its size).
            const int last_slot = min(hi / p.page_size, p.table_width - 1);
            const int page_rows = p.n_kv * p.page_size, head_row = g * p.page_size;
            const uint32_t whole_off = (uint32_t)(half * (BN * 128));
            for (int i = 0; i < n_tiles; ++i) {
                const int kt = first_tile + i, b = i & 1, use = i >> 1;
                const int slot = kt * p.pages_per_box + rb;
                const int page = (has_box && slot <= last_slot) ? __ldg(table + slot) : -1;
                const int first_page = __shfl_sync(0xffffffffu, page, 0);
                const bool whole = __all_sync(0xffffffffu, !has_box || page == first_page + rb) && first_page >= 0;
                const int row_coord = page >= 0 ? page * page_rows + head_row : p.rows_total;   // beyond the pool: zeros
                if (i >= 2 && ok && !mbar_wait(&k_empty[b], (use - 1) & 1, abort_flag)) ok = false;
                if (lane == 0) mbar_expect_tx(&k_full[b], C::KV_BYTES);
                __syncwarp();
                if (whole) {
                    if (rb == 0 && ok) tma_load_4d(k_tiles + b * C::KV_BYTES + whole_off, &map_k4, &k_full[b], half * 64, 0, g, first_page);
                } else if (has_box && ok) {
                    tma_load_2d(k_tiles + b * C::KV_BYTES + dst_off, &map_k, &k_full[b], half * 64, row_coord);
                }
                if (i >= 2 && ok && !mbar_wait(&v_empty[b], (use - 1) & 1, abort_flag)) ok = false;
                if (lane == 0) mbar_expect_tx(&v_full[b], C::KV_BYTES);
                __syncwarp();
                if (whole) {
                    if (rb == 0 && ok) tma_load_4d(v_tiles + b * C::KV_BYTES + whole_off, &map_v4, &v_full[b], half * 64, 0, g, first_page);
                } else if (has_box && ok) {
                    tma_load_2d(v_tiles + b * C::KV_BYTES + dst_off, &map_v, &v_full[b], half * 64, row_coord);
                }
            }
        } else {
            // Pages of 64 slots and multiples: a box is the 64-key half of a tile, inside one page.
            for (int i = 0; i < n_tiles; ++i) {
                const int kt = first_tile + i, b = i & 1, use = i >> 1;
                int row_coord = p.rows_total;                  // beyond the pool: zeros
                if (has_box) {
                    const int j = kt * BN;
                    const int slot = j / p.page_size;
                    const int page = (j <= hi && slot < p.table_width) ? __ldg(table + slot) : -1;
                    if (page >= 0) row_coord = (page * p.n_kv + g) * p.page_size + (j - slot * p.page_size);
                }
                if (i >= 2 && ok && !mbar_wait(&k_empty[b], (use - 1) & 1, abort_flag)) ok = false;
                if (lane == 0) mbar_expect_tx(&k_full[b], C::KV_BYTES);
                __syncwarp();
                if (has_box && ok) tma_load_2d(k_tiles + b * C::KV_BYTES + dst_off, &map_k, &k_full[b], half * 64, row_coord);
                if (i >= 2 && ok && !mbar_wait(&v_empty[b], (use - 1) & 1, abort_flag)) ok = false;
                if (lane == 0) mbar_expect_tx(&v_full[b], C::KV_BYTES);
                __syncwarp();
                if (has_box && ok) tma_load_2d(v_tiles + b * C::KV_BYTES + dst_off, &map_v, &v_full[b], half * 64, row_coord);
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------ MMA issuer: scores
        // The whole warp walks the loop and waits; one elected lane issues.  (With one lane
        // alone in a branch of its own the operands of every product came out of that
        // lane's registers, and a product took 60 to 80 cycles to issue.)
        constexpr uint32_t IDESC_S = idesc(BM, BN, 0);
        bool ok = mbar_wait(q_full, 0, abort_flag);
        // S(tile i) = Q K^T into score buffer i & 1 from key stage i & 1, as soon as the
        // output product of tile i - 2 has read the weights that lie in that buffer:
        // up to two tiles ahead of the softmax warps, never waiting for them
        for (int i = 0; i < n_tiles; ++i) {
            const int b = i & 1, use = i >> 1;
            // (the keys land long before the buffer is free: that wait first, so that nothing
            // stands between the buffer's release and the products)
            if (ok && !mbar_wait(&k_full[b], use & 1, abort_flag)) ok = false;
            if (i >= 2 && ok && !mbar_wait(&p_empty[b], (use - 1) & 1, abort_flag)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            const uint32_t acc = tmem_s + b * BN;
            const uint32_t k_stage = k_tiles + b * C::KV_BYTES;
            if (elect_one()) {
#pragma unroll
                for (int hh = 0; hh < C::HALVES; ++hh) {
                    const uint64_t qd = smem_desc(q_tile + hh * (BM * 128), 0, 1024);
                    const uint64_t kd = smem_desc(k_stage + hh * (BN * 128), 0, 1024);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(acc, qd + 2 * k, kd + 2 * k, IDESC_S, (hh | k) ? 1u : 0u);
                }
                umma_commit(&s_full[b]);
                umma_commit(&k_empty[b]);
            }
            __syncwarp();
        }
    } else if (warp == 10) {
        // ------------------------------------------------------------ MMA issuer: outputs
        constexpr uint32_t IDESC_O = idesc(BM, D, 1);
        bool ok = true;
        for (int i = 0; i < n_tiles; ++i) {
            const int b = i & 1, use = i >> 1;
            // the tile's weights are in its score buffer, O is rescaled, its values have landed
            if (ok && !mbar_wait(&v_full[b], use & 1, abort_flag)) ok = false;
            if (ok && !mbar_wait(&p_full[b], use & 1, abort_flag)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            const uint64_t vd = smem_desc(v_tiles + b * C::KV_BYTES, p.v_lbo, p.v_sbo);
            const uint32_t weights = tmem_s + b * BN;
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    // 16 keys further: 8 columns of P; 16 rows = 2048 bytes in the value tile
                    umma_bf16_a_tmem(tmem_o, weights + 8 * k, vd + 128 * k, IDESC_O, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&v_empty[b]);
                umma_commit(&p_empty[b]);
                if (i == n_tiles - 1) umma_commit(o_final);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ softmax warps 0-7
        // Threads r and r + 128 share query row r.  Warps w and w + 4 hold the same 32
        // rows (a warp reaches the tensor-memory lanes 32 (w % 4) .. + 31).
        const int row = threadIdx.x & (BM - 1), ch = threadIdx.x >> 7;
        const int tok = tile_tok + row;
        const bool live = tok < q_len;
        const int pos = ctx + tok;
        const int lo_row = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const uint32_t t_lane = (uint32_t)((warp & 3) * 32) << 16;   // this warp's tensor-memory lanes
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        // (A failed wait does not leave the loop: every thread must meet every barrier;
        // once the abort flag is up the remaining waits return at once.)
        for (int i = 0; i < n_tiles; ++i) {
            const int kt = first_tile + i, b = i & 1, use = i >> 1;
            if (!mbar_wait(&s_full[b], use & 1, abort_flag)) { if (ok) atomicMax(&p.status[2], 1); ok = false; }
            tc_fence_after();
            constexpr int HB = BN / 2;                     // keys per thread
            float s[HB];
            tmem_ld32(tmem_s + b * BN + t_lane + ch * HB, s);
            const int j0 = kt * BN + ch * HB;
            // Masking only where the tile crosses a row's limits (the diagonal, a
            // window's edge, rows beyond the entry): decided per warp.
            if (!__all_sync(0xffffffffu, live && j0 + HB - 1 <= pos && j0 >= lo_row)) {
#pragma unroll
                for (int j = 0; j < HB; ++j) {
                    const int key = j0 + j;
                    if (!(live && key >= lo_row && key <= pos)) s[j] = -INFINITY;
                }
            }
            float raw = -INFINITY;
#pragma unroll
            for (int j = 0; j < HB; j += 2) raw = max3(raw, s[j], s[j + 1]);
            // the row's maximum over both halves: through shared memory, between the two warps of the row
            {
                float* xb = xchg + b * (2 * BM);
                xb[ch * BM + row] = raw;
                named_barrier(1 + (warp & 3), 64);
                raw = fmaxf(raw, xb[(ch ^ 1) * BM + row]);
            }
            // The running maximum only has to bound the exponents: it moves when the
            // tile's maximum exceeds it by more than RESCALE_SLACK (weights up to
            // 2^RESCALE_SLACK, far inside bfloat16 and the fp32 sums); numerator and
            // denominator carry the same reference, so the quotient is unchanged.
            const float cand = raw * p.scale_log2;                  // scale > 0: the maximum commutes
            const float mx = (cand > m_run + RESCALE_SLACK || m_run == -INFINITY) ? fmaxf(m_run, cand) : m_run;
            const float corr = (m_run == -INFINITY) ? 0.f : (mx == m_run ? 1.f : fast_exp2(m_run - mx));
            const float neg_base = (mx == -INFINITY) ? 0.f : -mx;
            float2 sum2 = make_float2(0.f, 0.f);
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), base2 = make_float2(neg_base, neg_base);
            uint32_t packed[HB / 2];
#pragma unroll
            for (int j = 0; j < HB; j += 2) {
                const float2 x = fma2(make_float2(s[j], s[j + 1]), scale2, base2);
                const float2 pw = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                sum2 = add2(sum2, pw);
                __nv_bfloat162 pk = __floats2bfloat162_rn(pw.x, pw.y);
                packed[j / 2] = *reinterpret_cast<uint32_t*>(&pk);
            }
            l_run = l_run * corr + (sum2.x + sum2.y);      // this thread's half of the row's sum
            m_run = mx;
            // The weights of this thread's keys go over the first half of the tile's own
            // score buffer: both threads of the row hold their scores in registers since
            // they met at the exchange of the maxima above.
            tmem_st16_words(tmem_s + b * BN + t_lane + ch * (HB / 2), packed);
            // rescale the output accumulator when some row of the warp moved its maximum
            // (this thread: its half of the columns), once O += P V of the tile before
            // is complete: that is the latest product (the one before it was complete before
            // this tile's scores could be made).
            if (i > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                if (!mbar_wait(&p_empty[b ^ 1], ((i - 1) >> 1) & 1, abort_flag)) { if (ok) atomicMax(&p.status[2], 2); ok = false; }
                tc_fence_after();
#pragma unroll 1
                for (int c = ch * (D / 2); c < (ch + 1) * (D / 2); c += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + t_lane + c, o);
#pragma unroll
                    for (int k = 0; k < 32; ++k) o[k] *= corr;
                    tmem_st32(tmem_o + t_lane + c, o);
                }
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[b]);
        }
        if (!mbar_wait(o_final, 0, abort_flag)) { if (ok) atomicMax(&p.status[2], 2); ok = false; }
        tc_fence_after();

        // ---- result: o / l, this thread's half of its row's columns.  The tensor-memory
        // loads are warp-wide (.sync.aligned): every thread of the warp runs them, whether
        // its row exists or not.
        float* xl = xchg + (n_tiles & 1) * (2 * BM);       // not the buffer the last tile's maxima went through
        xl[ch * BM + row] = l_run;
        named_barrier(1 + (warp & 3), 64);
        const float l_row = l_run + xl[(ch ^ 1) * BM + row];
        const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
        bf16* dst = p.out + ((size_t)(qs + (live ? tok : 0)) * p.n_q + h) * D;
        // Where all 32 rows of the warp belong to the entry, its 32 x 64 block of the output goes
        // through shared memory (the query tile's, no product reads it any more; 128-byte rows,
        // swizzled as the unit expects) and leaves as ONE box: a thread's own stores would touch 16
        // bytes of 32 different lines each.  A warp at the entry's ragged end writes its rows itself.
        const int w4 = warp & 3;
        const bool as_box = (D == 128) && tile_tok + w4 * 32 + 31 < q_len;
        const uint32_t box = q_tile + ch * (BM * 128) + w4 * (32 * 128);     // 4 KB, 1,024-byte aligned
#pragma unroll 1
        for (int c = ch * (D / 2); c < (ch + 1) * (D / 2); c += 32) {
            float o[32];
            tmem_ld32(tmem_o + t_lane + c, o);
            if (ok && (live || as_box)) {
                uint4 pk[4];
                uint32_t* w = reinterpret_cast<uint32_t*>(pk);
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(o[2 * k] * inv, o[2 * k + 1] * inv);
                    w[k] = *reinterpret_cast<uint32_t*>(&h2);
                }
                if (as_box) {
                    const int chunk0 = (c - ch * (D / 2)) >> 3;               // 16-byte chunk of the 128-byte row
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        st_shared_v4(box + lane * 128 + (((chunk0 + k) ^ (lane & 7)) << 4), pk[k]);
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) reinterpret_cast<uint4*>(dst + c)[k] = pk[k];
                }
            }
        }
        if (as_box) {
            fence_async_proxy();                           // these stores before the unit's read
            __syncwarp();
            if (lane == 0 && ok) {
                tma_store_2d(&map_out, box, h * D + ch * 64, qs + tile_tok + w4 * 32);
                bulk_commit();
                bulk_wait_read();                          // the shared memory outlives the read
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(&p.status[1], 1);
    if (warp == 9) tmem_dealloc(tmem_base, C::TMEM_COLS);
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
    const void* ptr; long long rows; int cols, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
    }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.cols; h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// The pool of one layer as a matrix bf16 [rows, D] (a row = one key or value of
// one kv head); box = [box_rows, 64 columns], 128-byte swizzle, zeros outside.
int pool_map(CUtensorMap* out, const void* ptr, long long rows, int cols, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiled fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

// The same pool as [n_pages][n_kv][page_size][D]; box = [pages_per_box pages, one kv head,
// page_size slots, 64 columns] = 64 consecutive rows of a key tile when the pages
// follow one another.
int pool_map4(CUtensorMap* out, const void* ptr, int n_pages, int n_kv, int page_size, int cols, int pages_per_box) {
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    static std::mutex mu;
    MapKey key{ptr, (long long)n_pages * n_kv, cols, page_size * 1024 + pages_per_box};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiled fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)page_size, (cuuint64_t)n_kv, (cuuint64_t)n_pages};
    cuuint64_t strides[3] = {(cuuint64_t)cols * 2, (cuuint64_t)page_size * cols * 2,
                             (cuuint64_t)n_kv * page_size * cols * 2};
    cuuint32_t box[4] = {64u, (cuuint32_t)page_size, 1u, (cuuint32_t)pages_per_box};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

template <int D> int launch(const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mk4, const CUtensorMap& mv4,
                            const CUtensorMap& mq, const CUtensorMap& mo, const Params& p, int items, cudaStream_t s) {
    using C = Cfg<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return kipp_launch(attn_prefill_tc_kernel<D>, dim3(p.n_q, items), dim3(THREADS), C::SMEM, s, 1, mk, mv, mk4, mv4, mq, mo, p);
}
}  // namespace

extern "C" int kipp_attn_prefill_tc_supported(int head_dim, int n_q, int n_kv) {
    return (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0;
}

// Page sizes the kernel takes: a TMA box holds min(page_size, 64) rows of one page,
// in whole 8-row swizzle groups.
extern "C" int kipp_attn_prefill_tc_page_ok(int page_size) {
    return page_size == 8 || page_size == 16 || page_size == 32 || (page_size > 0 && page_size % 64 == 0);
}

// Prompt portions: `work` lists (entry, first token) of every 128-token tile.
// q: bf16 [tokens][n_q][head_dim], all of the step's tokens (the query tiles come by TMA, which
// fills what lies past the last token with zeros).
// k_pages and v_pages: one layer's pool, bf16 [n_pages][n_kv][page_size][head_dim].
extern "C" int kipp_attn_prefill_tc(void* out, const void* q, int tokens, const void* k_pages, const void* v_pages,
                                    int n_pages, const int* q_start, const int* context_len,
                                    const int* block_table, int table_width, int page_size, const int* work,
                                    int items, int n_q, int n_kv, int head_dim, float scale, int window,
                                    int* status, void* stream) {
    if (items <= 0) return 0;
    if (items > 65535) return KIPP_ERR_ARG;
    if (!kipp_attn_prefill_tc_supported(head_dim, n_q, n_kv) || !kipp_attn_prefill_tc_page_ok(page_size) ||
        n_pages <= 0 || window < 0 || status == nullptr || tokens <= 0)
        return KIPP_ERR_ARG;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 15))
        return -3;
    const long long rows = (long long)n_pages * n_kv * page_size;
    if (rows + BN > 0x7fffffffLL) return KIPP_ERR_ARG;
    Params p;
    p.out = (bf16*)out; p.q = (const bf16*)q;
    p.q_start = q_start; p.context_len = context_len; p.block_table = block_table; p.work = work;
    p.table_width = table_width; p.page_size = page_size; p.n_q = n_q; p.n_kv = n_kv; p.window = window;
    p.box_rows = page_size < BN ? page_size : BN;
    p.rows_total = (int)rows;
    p.scale_log2 = scale * 1.4426950408889634f;
    // The value tile is the MN-major operand of O += P V: leading offset = the next
    // 64-column half of the tile, stride offset = the next 8 keys (checked against
    // the other assignment on the device: that one gives wrong sums).
    p.v_lbo = (uint32_t)(BN * 128);
    p.v_sbo = 1024u;
    p.status = status;
    CUtensorMap mk, mv;
    int rc = pool_map(&mk, k_pages, rows, head_dim, p.box_rows);
    if (rc) return rc;
    rc = pool_map(&mv, v_pages, rows, head_dim, p.box_rows);
    if (rc) return rc;
    // pages of fewer than 64 slots: maps whose box is the whole 64-key half of a tile
    CUtensorMap mk4 = mk, mv4 = mv;
    p.pages_per_box = page_size < BN ? BN / page_size : 1;
    if (p.pages_per_box > 1) {
        rc = pool_map4(&mk4, k_pages, n_pages, n_kv, page_size, head_dim, p.pages_per_box);
        if (rc) return rc;
        rc = pool_map4(&mv4, v_pages, n_pages, n_kv, page_size, head_dim, p.pages_per_box);
        if (rc) return rc;
    }
    CUtensorMap mq;
    rc = pool_map(&mq, q, tokens, n_q * head_dim, BM);
    if (rc) return rc;
    CUtensorMap mo;                                  // the output as [tokens, n_q x head_dim]: boxes of 32 rows
    rc = pool_map(&mo, out, tokens, n_q * head_dim, 32);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    return head_dim == 64 ? launch<64>(mk, mv, mk4, mv4, mq, mo, p, items, s)
                          : launch<128>(mk, mv, mk4, mv4, mq, mo, p, items, s);
}
