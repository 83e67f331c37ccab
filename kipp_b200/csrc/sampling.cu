// Greedy and temperature sampling on the device.  A row of logits is worked on by a team:
// one thread block, or for long rows a thread-block cluster of eight whose blocks take an
// eighth of the row each and put their counts and sums together through distributed shared
// memory (every block reads all eight and decides alike, so nothing is broadcast; the
// cluster's hardware barrier stands between writing and reading).  One block alone scanned a
// 151,936-entry row some fifteen times at 40 to 70 us a scan.
//
// The token drawn is the one the reference's host sampler draws from the same
// logits and the same uniform number (kipp_sample_ex, src/kipp.c:3433-3559):
//   * greedy (temperature <= 0): first index of the maximum, strict '>';
//   * else scaled = logit * (1/T); candidates are scaled >= max - 20; they are
//     ordered by scaled value descending, ties by token id ascending; top-k
//     keeps the first k; weights w = expf(scaled - max) in float32, sums in
//     double; min-p keeps w >= min_p * w_top; the nucleus is the shortest
//     prefix whose sum reaches top_p * total; draw = u * kept picks the first
//     candidate whose inclusive prefix sum exceeds it.
// The reference sorts the candidates.  Here nothing is sorted: a position in
// that order is found by radix selection over the (value, token) keys, with
// per-bucket counts and weight sums, four 8-bit passes over the value and,
// only among equal values, four over the token id.  Bucket sums add the same
// float32 weights as integers in units of 2^-40 (see weight_units) where the
// reference keeps a running double sum, so a draw that lies within 2^-23 of a
// boundary may pick the neighbour.
//
// Also here: the penalties and logit bias the reference applies before
// sampling (apply_bias_and_penalties, src/kipp.c:3386-3431).
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned desc_key(float x) {
    // Ascending unsigned order of the result == descending float order of x.
    unsigned k = __float_as_uint(x);
    k = (k & 0x80000000u) ? ~k : (k | 0x80000000u);
    return ~k;
}

// ---- the team of blocks that shares a row (a cluster along x; one block when launched without)
__device__ __forceinline__ int team_size() { unsigned n; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n)); return (int)n; }
__device__ __forceinline__ int team_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return (int)r; }
// all threads of all blocks of the team: what was written to shared memory before is visible after
__device__ __forceinline__ void team_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t team_addr(const void* p, int rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
    return a;
}
__device__ __forceinline__ unsigned team_ld_u32(const void* p, int rank) {
    unsigned v; asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(team_addr(p, rank)) : "memory"); return v;
}
__device__ __forceinline__ float team_ld_f32(const void* p, int rank) {
    float v; asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(team_addr(p, rank)) : "memory"); return v;
}
__device__ __forceinline__ unsigned long long team_ld_u64(const void* p, int rank) {
    unsigned long long v; asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(team_addr(p, rank)) : "memory"); return v;
}
__device__ __forceinline__ double team_ld_f64(const void* p, int rank) {
    double v; asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(team_addr(p, rank)) : "memory"); return v;
}

struct RowCtx {
    const float* v;
    int n;
    int lo, hi;                 // this block's part of the row
    float inv_t, smax, cutoff;
    // filters
    bool has_topk;   unsigned topk_key, topk_tok;
    bool has_minp;   double minp_threshold;
    bool has_nucleus; unsigned nuc_key, nuc_tok;
};

__device__ __forceinline__ bool before_or_at(unsigned key, unsigned tok, unsigned bkey, unsigned btok) {
    return key < bkey || (key == bkey && tok <= btok);
}

// Whether element i is in the current candidate set; gives its key and weight.
__device__ __forceinline__ bool member(const RowCtx& c, int i, unsigned& key, float& w) {
    const float scaled = c.v[i] * c.inv_t;
    if (!(scaled >= c.cutoff)) return false;
    key = desc_key(scaled);
    if (c.has_topk && !before_or_at(key, (unsigned)i, c.topk_key, c.topk_tok)) return false;
    w = expf(scaled - c.smax);
    if (c.has_minp && (double)w < c.minp_threshold) return false;
    if (c.has_nucleus && !before_or_at(key, (unsigned)i, c.nuc_key, c.nuc_tok)) return false;
    return true;
}

struct Shared {
    unsigned cnt[256];          // this block's part of the row
    unsigned long long wfix[256];   // weight sums in units of 2^-40 (see weight_units)
    unsigned cnt_all[256];      // the team's: the blocks' parts added in block order
    double wsum_all[256];
    float red_val[32];
    int red_idx[32];
    double red_d[32];
    unsigned long long red_u[32];
    // results broadcast
    unsigned sel_digit; unsigned long long sel_cnt_before; double sel_w_before;
    unsigned sel_bucket_cnt; int found;
    int i_val; float f_val; double d_val; unsigned long long u_val;
};

enum { MODE_COUNT = 0, MODE_W_GE = 1, MODE_W_GT = 2 };

// Weights are summed as integers, in units of 2^-40 of the top weight (1): integer sums do not
// depend on their order, so a row's draw is the same whichever block or lane adds first, and
// the lanes of a warp that hit the same bucket add their weights with the warp's integer
// reduction and ONE atomic instead of 32 that the hardware runs one after the other (with
// float64 atomics the passes were bound by exactly that).  A weight is at least e^-20 = 2^-29,
// so it keeps eleven bits and more; a row's sums stay below 2^58.  Against the reference's
// running float64 sum a draw within 2^-23 of a boundary may pick the neighbour.
constexpr double WEIGHT_UNIT = 1.0 / 1099511627776.0;      // 2^-40
__device__ __forceinline__ unsigned long long weight_units(float w) {
    return (unsigned long long)((double)w * 1099511627776.0);
}
// Sum of `v` over the lanes of `peers` (all of them call this with the same mask; v < 2^41).
__device__ __forceinline__ unsigned long long peers_sum(unsigned peers, unsigned long long v) {
    const unsigned lo = __reduce_add_sync(peers, (unsigned)(v & 0xfffffu));          // 32 x 2^20 < 2^32
    const unsigned hi = __reduce_add_sync(peers, (unsigned)(v >> 20));               // 32 x 2^21 < 2^32
    return ((unsigned long long)hi << 20) + lo;
}

// One histogram pass.  level 0..3: value key digits (high to low); level 4..7:
// token digits among elements whose key == prefix_key.
__device__ void histogram_pass(const RowCtx& c, Shared& sh, int level, unsigned prefix_key,
                               unsigned prefix_tok) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) { sh.cnt[b] = 0; sh.wfix[b] = 0ull; }
    __syncthreads();
    // whole warps walk the part (every lane makes every round): the lanes of a round that fall
    // into one bucket are found with match.any and add as one
    const int lane = threadIdx.x & 31;
    for (int base = c.lo + (int)(threadIdx.x - lane); base < c.hi; base += blockDim.x) {
        const int i = base + lane;
        unsigned key = 0; float w = 0.f;
        unsigned digit = 256u;                                  // no bucket: not in the set at this level
        if (i < c.hi && member(c, i, key, w)) {
            if (level < 4) {
                const int shift = 24 - 8 * level;
                if (level == 0 || (key >> (shift + 8)) == (prefix_key >> (shift + 8))) digit = (key >> shift) & 0xffu;
            } else if (key == prefix_key) {
                const int shift = 24 - 8 * (level - 4);
                const unsigned tok = (unsigned)i;
                if (level == 4 || (tok >> (shift + 8)) == (prefix_tok >> (shift + 8))) digit = (tok >> shift) & 0xffu;
            }
        }
        const unsigned peers = __match_any_sync(0xffffffffu, digit);
        const unsigned long long units = peers_sum(peers, digit < 256u ? weight_units(w) : 0ull);
        if (digit < 256u && lane == __ffs(peers) - 1) {
            atomicAdd(&sh.cnt[digit], (unsigned)__popc(peers));
            atomicAdd(&sh.wfix[digit], units);
        }
    }
    __syncthreads();
    // the team's histogram: every block adds the blocks' parts in block order
    team_sync();
    const int blocks = team_size();
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {
        unsigned n8[8]; unsigned long long w8[8];    // all loads first: they travel together
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            n8[r] = r < blocks ? team_ld_u32(&sh.cnt[b], r) : 0u;
            w8[r] = r < blocks ? team_ld_u64(&sh.wfix[b], r) : 0ull;
        }
        unsigned n = 0; unsigned long long w = 0ull;
#pragma unroll
        for (int r = 0; r < 8; ++r) { n += n8[r]; w += w8[r]; }
        sh.cnt_all[b] = n; sh.wsum_all[b] = (double)w * WEIGHT_UNIT;
    }
    team_sync();                                   // nobody clears its part while another still reads it
}

// Position selection in the (value desc, token asc) order of the current set.
//   MODE_COUNT: the element with 1-based rank `target_count`;
//   MODE_W_GE : the first element whose inclusive weight sum >= target_w;
//   MODE_W_GT : the first element whose inclusive weight sum >  target_w.
// If no element qualifies, the last element of the set is returned.
// Outputs (uniform over the block): key, token, inclusive weight sum at it.
__device__ void select(const RowCtx& c, Shared& sh, int mode, unsigned long long target_count,
                       double target_w, unsigned& out_key, unsigned& out_tok, double& out_cum) {
    unsigned prefix_key = 0, prefix_tok = 0;
    unsigned long long cnt_before = 0;
    double w_before = 0.0;
    for (int level = 0; level < 8; ++level) {
        histogram_pass(c, sh, level, prefix_key, prefix_tok);
        if (threadIdx.x < 32) {
            // The first bucket (in order) at which the running count or weight reaches the target,
            // else the last bucket that is not empty.  One warp: a lane walks over its eight
            // buckets from the sums of the lanes before it (one thread alone took 256 dependent
            // steps, some 5 us a level).
            const int lane = threadIdx.x;
            unsigned n8[8]; double w8[8];
            unsigned long long ln = 0; double lw = 0.0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                n8[j] = sh.cnt_all[8 * lane + j]; w8[j] = sh.wsum_all[8 * lane + j];
                ln += n8[j]; lw += w8[j];
            }
            unsigned long long pn = ln; double pw = lw;             // inclusive over the lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long tn = __shfl_up_sync(0xffffffffu, pn, o);
                const double tw = __shfl_up_sync(0xffffffffu, pw, o);
                if (lane >= o) { pn += tn; pw += tw; }
            }
            unsigned long long cb = __shfl_up_sync(0xffffffffu, pn, 1);
            double wb = __shfl_up_sync(0xffffffffu, pw, 1);
            if (lane == 0) { cb = 0; wb = 0.0; }
            cb += cnt_before; wb += w_before;
            int chosen = -1, last_nonempty = -1;
            unsigned long long cb_hit = 0, cb_last = 0; double wb_hit = 0.0, wb_last = 0.0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (n8[j] == 0 || chosen >= 0) continue;
                last_nonempty = 8 * lane + j; cb_last = cb; wb_last = wb;
                bool hit;
                if (mode == MODE_COUNT) hit = cb + n8[j] >= target_count;
                else if (mode == MODE_W_GE) hit = wb + w8[j] >= target_w;
                else hit = wb + w8[j] > target_w;
                if (hit) { chosen = 8 * lane + j; cb_hit = cb; wb_hit = wb; }
                else { cb += n8[j]; wb += w8[j]; }
            }
            const unsigned hits = __ballot_sync(0xffffffffu, chosen >= 0);
            const unsigned some = __ballot_sync(0xffffffffu, last_nonempty >= 0);
            int src = -1;                                            // the lane whose answer counts
            if (hits) src = __ffs(hits) - 1;
            else if (some) { src = 31 - __clz(some); chosen = last_nonempty; cb_hit = cb_last; wb_hit = wb_last; }
            if (lane == src) {
                sh.found = chosen;
                sh.sel_cnt_before = cb_hit; sh.sel_w_before = wb_hit;
                sh.sel_bucket_cnt = sh.cnt_all[chosen];
                sh.d_val = wb_hit + sh.wsum_all[chosen];
            } else if (src < 0 && lane == 0) {
                sh.found = -1;
                sh.sel_cnt_before = cnt_before; sh.sel_w_before = w_before;
                sh.sel_bucket_cnt = 0;
                sh.d_val = w_before;
            }
        }
        __syncthreads();
        const int chosen = sh.found;
        cnt_before = sh.sel_cnt_before; w_before = sh.sel_w_before;
        const double cum_incl = sh.d_val;
        const unsigned bucket_cnt = sh.sel_bucket_cnt;
        __syncthreads();
        if (chosen < 0) { out_key = 0xffffffffu; out_tok = 0; out_cum = w_before; return; }  // empty set
        const int shift = 24 - 8 * (level & 3);
        if (level < 4) prefix_key |= (unsigned)chosen << shift;
        else prefix_tok |= (unsigned)chosen << shift;
        if (level == 7) { out_key = prefix_key; out_tok = prefix_tok; out_cum = cum_incl; return; }
        if (level == 3 && bucket_cnt == 1) {
            // One element has this value: find its token in one pass.
            if (threadIdx.x == 0) sh.i_val = 0x7fffffff;
            __syncthreads();
            for (int i = c.lo + threadIdx.x; i < c.hi; i += blockDim.x) {
                unsigned key; float w;
                if (member(c, i, key, w) && key == prefix_key) atomicMin(&sh.i_val, i);
            }
            __syncthreads();
            team_sync();
            int first = 0x7fffffff;
            for (int r = 0; r < team_size(); ++r) first = min(first, (int)team_ld_u32(&sh.i_val, r));
            team_sync();
            out_key = prefix_key; out_tok = (unsigned)first; out_cum = cum_incl;
            return;
        }
    }
}

// best_i = 0x7fffffff when the row holds no number (NaN only)
__device__ void block_argmax_raw(const float* v, int n, Shared& sh, float& best_v, int& best_i) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float x = v[i];
        if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
    }
    // A row of NaNs or -inf leaves bi unset in some threads; index 0 then wins
    // as in the reference (argmax starts at 0 and only '>' replaces it).
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sh.red_val[warp] = bv; sh.red_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? sh.red_val[lane] : -INFINITY;
        bi = lane < nw ? sh.red_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { sh.f_val = bv; sh.i_val = bi; }
    }
    __syncthreads();
    best_v = sh.f_val; best_i = sh.i_val;
    __syncthreads();
}

__device__ void block_argmax(const float* v, int n, Shared& sh, float& best_v, int& best_i) {
    block_argmax_raw(v, n, sh, best_v, best_i);
    if (best_i == 0x7fffffff) best_i = 0;
}

__global__ void __launch_bounds__(THREADS)
argmax_rows_kernel(const float* __restrict__ logits, long long ld, int n, int* __restrict__ out) {
    __shared__ Shared sh;
    pdl_launch_dependents();
    pdl_wait();
    float bv; int bi;
    block_argmax(logits + (size_t)blockIdx.x * ld, n, sh, bv, bi);
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
}

// A long row by many blocks: block (c, r) leaves the first maximum of its share of row r, the
// second kernel takes the first maximum of the shares (in share order, so the lowest index wins
// a tie as in the one-block kernel).  One block per row would scan a 150,000-entry row alone
// for 70 us; the shares take a few.
struct ArgmaxPart { float v; int i; };

__global__ void __launch_bounds__(THREADS)
argmax_parts_kernel(const float* __restrict__ logits, long long ld, int n, int per, ArgmaxPart* __restrict__ parts) {
    __shared__ Shared sh;
    pdl_launch_dependents();
    pdl_wait();
    const int first = blockIdx.x * per;
    const int count = min(per, n - first);
    float bv = -INFINITY; int bi = 0x7fffffff;
    if (count > 0) block_argmax_raw(logits + (size_t)blockIdx.y * ld + first, count, sh, bv, bi);
    if (threadIdx.x == 0)
        parts[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = ArgmaxPart{bv, bi == 0x7fffffff ? bi : first + bi};
}

__global__ void argmax_merge_kernel(const ArgmaxPart* __restrict__ parts, int n_parts, int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    // one warp per row; lane l takes shares l, l + 32, ... in order, then the lanes in order
    const ArgmaxPart* row = parts + (size_t)blockIdx.x * n_parts;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < n_parts; c += 32) {
        const ArgmaxPart p = row[c];
        if (p.v > bv || (p.v == bv && p.i < bi)) { bv = p.v; bi = p.i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    // a row without any number (NaN only) leaves every share without an index: index 0 then
    if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// The sum of the weights of the current set: the blocks' sums added in block order.
__device__ double team_weight_sum(const RowCtx& c, Shared& sh) {
    unsigned long long local = 0ull;
    for (int i = c.lo + threadIdx.x; i < c.hi; i += blockDim.x) {
        unsigned kk; float w;
        if (member(c, i, kk, w)) local += weight_units(w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0) sh.red_u[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0ull;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sh.red_u[w];
        sh.u_val = t;
    }
    __syncthreads();
    team_sync();
    unsigned long long total = 0ull;
    for (int b = 0; b < team_size(); ++b) total += team_ld_u64(&sh.u_val, b);
    team_sync();
    return (double)total * WEIGHT_UNIT;
}

__global__ void __launch_bounds__(THREADS)
sample_rows_kernel(const float* __restrict__ logits, long long ld, int n,
                   const float* __restrict__ temperature, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, const float* __restrict__ min_p,
                   const double* __restrict__ uniform, int* __restrict__ out) {
    __shared__ Shared sh;
    pdl_launch_dependents();
    pdl_wait();
    const int blocks = team_size(), rank = team_rank();
    const int r = blockIdx.x / blocks;
    const float* v = logits + (size_t)r * ld;
    const int part = ((n + blocks - 1) / blocks + 3) & ~3;
    const int lo = min(n, rank * part), hi = min(n, lo + part);
    // the row's first maximum: each block's over its part, then the first of those
    float best_v; int best_i;
    block_argmax_raw(v + lo, hi - lo, sh, best_v, best_i);
    if (threadIdx.x == 0) { sh.f_val = best_v; sh.i_val = best_i == 0x7fffffff ? best_i : lo + best_i; }
    __syncthreads();
    team_sync();
    best_v = -INFINITY; best_i = 0x7fffffff;
    for (int b = 0; b < blocks; ++b) {
        const float ov = team_ld_f32(&sh.f_val, b);
        const int oi = (int)team_ld_u32(&sh.i_val, b);
        if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
    }
    if (best_i == 0x7fffffff) best_i = 0;
    team_sync();
    const float T = temperature[r];
    if (!(T > 0.0f)) {
        if (threadIdx.x == 0 && rank == 0) out[r] = best_i;
        return;
    }
    RowCtx c;
    c.v = v; c.n = n; c.lo = lo; c.hi = hi;
    c.inv_t = 1.0f / T;
    c.smax = v[best_i] * c.inv_t;
    c.cutoff = c.smax - 20.0f;
    c.has_topk = c.has_minp = c.has_nucleus = false;
    c.topk_key = c.topk_tok = c.nuc_key = c.nuc_tok = 0;
    c.minp_threshold = 0.0;

    unsigned key, tok; double cum;
    const int k = top_k[r];
    if (k > 0) {
        // rank k in the order, or the last candidate when there are fewer
        select(c, sh, MODE_COUNT, (unsigned long long)k, 0.0, key, tok, cum);
        c.has_topk = true; c.topk_key = key; c.topk_tok = tok;
    }
    const float mp = min_p[r];
    if (mp > 0.0f) {
        // The top weight is expf(smax - smax) = 1.
        c.has_minp = true;
        c.minp_threshold = (double)mp * (double)expf(0.0f);
    }
    // total weight of the set (and, with a nucleus, the prefix that is kept)
    const float tp = top_p[r];
    double kept;
    if (tp < 1.0f) {
        const double total = team_weight_sum(c, sh);
        select(c, sh, MODE_W_GE, 0, (double)tp * total, key, tok, cum);
        c.has_nucleus = true; c.nuc_key = key; c.nuc_tok = tok;
        kept = cum;
    } else {
        kept = team_weight_sum(c, sh);
    }
    const double draw = uniform[r] * kept;
    select(c, sh, MODE_W_GT, 0, draw, key, tok, cum);
    if (threadIdx.x == 0 && rank == 0) out[r] = (key == 0xffffffffu && tok == 0 && kept == 0.0) ? best_i : (int)tok;
}

// Logit bias, then repetition / presence / frequency penalties over each row's
// window of recent tokens; each distinct token is adjusted once
// (src/kipp.c:3386-3431).  One block per row; the window is short.
__global__ void apply_penalties_kernel(float* __restrict__ logits, long long ld, int n,
                                       const int* __restrict__ recent, int recent_width,
                                       const int* __restrict__ recent_count,
                                       const float* __restrict__ repetition,
                                       const float* __restrict__ presence,
                                       const float* __restrict__ frequency,
                                       const int* __restrict__ bias_tokens,
                                       const float* __restrict__ bias_values, int bias_width,
                                       const int* __restrict__ bias_count) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    float* v = logits + (size_t)r * ld;
    if (bias_tokens != nullptr && threadIdx.x == 0) {
        // sequential: the same token may be listed twice and both add up
        const int nb = bias_count[r];
        for (int i = 0; i < nb; ++i) {
            const int tok = bias_tokens[(size_t)r * bias_width + i];
            if (tok >= 0 && tok < n) v[tok] += bias_values[(size_t)r * bias_width + i];
        }
    }
    __syncthreads();
    if (recent == nullptr) return;
    const float rep = repetition[r], pres = presence[r], freq = frequency[r];
    const bool has = freq != 0.0f || pres != 0.0f || (rep != 0.0f && rep != 1.0f);
    const int nr = recent_count[r];
    if (!has || nr == 0) return;
    const int* win = recent + (size_t)r * recent_width;
    for (int p = threadIdx.x; p < nr; p += blockDim.x) {
        const int tok = win[p];
        if (tok < 0 || tok >= n) continue;
        bool seen = false;
        for (int e = 0; e < p; ++e) if (win[e] == tok) { seen = true; break; }
        if (seen) continue;
        int count = 0;
        for (int o = 0; o < nr; ++o) count += win[o] == tok;
        float x = v[tok];
        if (rep != 0.0f && rep != 1.0f) x = x > 0.0f ? x / rep : x * rep;
        x -= pres;
        x -= freq * (float)count;
        v[tok] = x;
    }
}
}  // namespace

// Between two greedy decode steps that run without the host (captured in one CUDA
// graph with the step itself): the tokens just chosen become the next step's
// tokens and go into row `*counter` of the ring; every request moves on by one
// position.  What a mixer's kernels derive from the lengths (the keys per split of
// the decode attention) is made anew by that mixer's own kernel after this one.
// One block.
namespace {
__global__ void burst_advance_kernel(int* tokens, int* positions, int* context_len, const int* next, int* ring,
                                     int* counter, int n, int ring_rows) {
    pdl_launch_dependents();
    pdl_wait();                                      // the tokens are chosen, every kernel of the step is through
    const int c = *counter;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int t = next[i];
        tokens[i] = t;
        if (c < ring_rows) ring[(size_t)c * n + i] = t;
        positions[i] += 1;
        context_len[i] += 1;                         // cached tokens before the next step's token
    }
    __syncthreads();
    if (threadIdx.x == 0) *counter = c + 1;
}
}  // namespace

extern "C" int kipp_argmax_rows(const float* logits, long long ld, int rows, int n, int* out,
                                void* stream) {
    if (rows <= 0) return 0;
    if (n <= 0) return KIPP_ERR_ARG;
    return kipp_launch(argmax_rows_kernel, dim3(rows), dim3(THREADS), 0, (cudaStream_t)stream, 1, logits, ld, n, out);
}

// How a row of n entries is shared among blocks: shares of at least ARGMAX_SHARE entries, at most 64.
namespace {
constexpr int ARGMAX_SHARE = 4096;
inline int argmax_shares(int n) { return n >= 2 * ARGMAX_SHARE ? (n / ARGMAX_SHARE > 64 ? 64 : n / ARGMAX_SHARE) : 1; }
}  // namespace

// Bytes of scratch kipp_argmax_rows_split wants for rows of n entries (0: the one-block kernel does it).
extern "C" long long kipp_argmax_scratch_bytes(int rows, int n) {
    const int shares = argmax_shares(n);
    return shares > 1 ? (long long)rows * shares * (long long)sizeof(ArgmaxPart) : 0;
}

// kipp_argmax_rows with long rows shared among blocks; `scratch` of kipp_argmax_scratch_bytes,
// 8-byte aligned, is the caller's and holds nothing between calls.
extern "C" int kipp_argmax_rows_split(const float* logits, long long ld, int rows, int n, int* out, void* scratch,
                                      long long scratch_bytes, void* stream) {
    if (rows <= 0) return 0;
    if (n <= 0) return KIPP_ERR_ARG;
    const int shares = argmax_shares(n);
    if (shares <= 1) return kipp_argmax_rows(logits, ld, rows, n, out, stream);
    if (scratch == nullptr || ((uintptr_t)scratch & 7) || scratch_bytes < kipp_argmax_scratch_bytes(rows, n) || rows > 65535)
        return KIPP_ERR_ARG;
    const int per = (n + shares - 1) / shares;
    int rc = kipp_launch(argmax_parts_kernel, dim3(shares, rows), dim3(THREADS), 0, (cudaStream_t)stream, 1, logits, ld,
                         n, per, (ArgmaxPart*)scratch);
    if (rc) return rc;
    return kipp_launch(argmax_merge_kernel, dim3(rows), dim3(32), 0, (cudaStream_t)stream, 1,
                       (const ArgmaxPart*)scratch, shares, out);
}

extern "C" int kipp_sample_rows(const float* logits, long long ld, int rows, int n,
                                const float* temperature, const int* top_k, const float* top_p,
                                const float* min_p, const double* uniform, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (n <= 0) return KIPP_ERR_ARG;
    // long rows: a cluster of up to eight blocks a row (at most eight: the kernel's loops over the
    // team are unrolled to that), as many as keep all rows' blocks within one wave of the GPU
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    int blocks = 1;
    while (blocks < 8 && n >= 16384 * blocks && (long long)rows * blocks * 2 <= sms) blocks *= 2;
    if ((long long)rows * blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    return kipp_launch_cluster(sample_rows_kernel, dim3((unsigned)(rows * blocks)), dim3(THREADS), 0, (cudaStream_t)stream,
                               dim3(blocks, 1, 1), logits, ld, n, temperature, top_k, top_p, min_p, uniform, out);
}

extern "C" int kipp_apply_penalties(float* logits, long long ld, int rows, int n, const int* recent,
                                    int recent_width, const int* recent_count,
                                    const float* repetition, const float* presence,
                                    const float* frequency, const int* bias_tokens,
                                    const float* bias_values, int bias_width, const int* bias_count,
                                    void* stream) {
    if (rows <= 0) return 0;
    if (n <= 0) return KIPP_ERR_ARG;
    return kipp_launch(apply_penalties_kernel, dim3(rows), dim3(64), 0, (cudaStream_t)stream, 1, logits, ld, n,
                       recent, recent_width, recent_count, repetition, presence, frequency, bias_tokens,
                       bias_values, bias_width, bias_count);
}

// See burst_advance_kernel.  `next` holds the n tokens just chosen.
extern "C" int kipp_burst_advance(int* tokens, int* positions, int* context_len, const int* next, int* ring,
                                  int* counter, int n, int ring_rows, void* stream) {
    if (n <= 0) return 0;
    if (ring_rows <= 0) return KIPP_ERR_ARG;
    return kipp_launch(burst_advance_kernel, dim3(1), dim3(128), 0, (cudaStream_t)stream, 1, tokens, positions,
                       context_len, next, ring, counter, n, ring_rows);
}
