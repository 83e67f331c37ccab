// Causal grouped-query attention over the paged cache on the CUDA cores, for
// any mix of prompt portions and single decoded tokens.
//
// This is the attention of the true 32-bit path and the fallback of the
// bfloat16 path for head sizes the tensor-core kernels refuse.  Reference
// counterpart: cached_gqa_kernel (cuda/kipp_kernels.cu:160), formula
// src/kipp.c:2882-2922: s_j = (q . k_j) / sqrt(head_dim) for the keys j the
// query may see, softmax with the maximum subtracted, o = sum_j p_j v_j, the
// kv head of query head h being h / (n_q / n_kv).
//
// One warp handles one (token, query head).  Keys are walked in tiles of 32
// aligned to absolute positions, one key per lane, with a running maximum and
// sum (all float32).  The order of every sum depends only on the token's own
// position and window, never on the batch it is in.
//
// A window of w (0 = none) lets position p see keys j with p - w < j <= p.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int MAX_ACC = 8;         // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(T* __restrict__ out, const T* __restrict__ q,
                            const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                            const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                            const int* __restrict__ block_table, int table_width, int page_size,
                            int tokens, int n_q, int n_kv, int head_dim, float scale, int window,
                            int* __restrict__ status) {
    extern __shared__ float q_smem[];                 // [warps][head_dim]
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long wg = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (wg >= (long long)tokens * n_q) return;
    const int t = (int)(wg / n_q), h = (int)(wg % n_q);
    const int g = h / (n_q / n_kv);
    const int pos = positions[t];
    const int e = entry_of_token[t];
    const int* table = block_table + (size_t)e * table_width;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;

    float* qs = q_smem + warp * head_dim;
    const T* qrow = q + ((size_t)t * n_q + h) * head_dim;
    for (int i = lane; i < head_dim; i += 32) qs[i] = to_f32(qrow[i]);
    __syncwarp();

    float acc[MAX_ACC];
#pragma unroll
    for (int i = 0; i < MAX_ACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int j0 = (first / 32) * 32; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j >= first && j <= pos;
        float s = -INFINITY;
        const T* vrow = nullptr;
        if (valid) {
            const int page = j / page_size < table_width ? table[j / page_size] : -1;
            if (page < 0) {
                atomicExch(status, 3);        // a needed key is not mapped
            } else {
                const size_t row = (((size_t)page * n_kv + g) * page_size + (j % page_size)) * head_dim;
                const T* krow = k_pages + row;
                vrow = v_pages + row;
                float dot = 0.f;
                for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
                s = dot * scale;
            }
        }
        const float tile_max = warp_max(s);
        const float m_new = fmaxf(m, tile_max);
        if (m_new == -INFINITY) continue;              // nothing visible yet
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_ACC; ++i) acc[i] *= corr;
        m = m_new;
        const int count = min(32, pos - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
            if (vp == 0ull) continue;
            const T* vr = (const T*)vp;
#pragma unroll
            for (int i = 0; i < MAX_ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
    T* orow = out + ((size_t)t * n_q + h) * head_dim;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) orow[d] = from_f32<T>(acc[i] * inv);
    }
}
}  // namespace

extern "C" int kipp_paged_attention_simt(
    void* out, const void* q, const void* k_pages, const void* v_pages, int dtype,
    const int* positions, const int* entry_of_token, const int* block_table, int table_width,
    int page_size, int tokens, int n_q, int n_kv, int head_dim, float scale, int window,
    int* status, void* stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > 32 * MAX_ACC || n_q <= 0 || n_kv <= 0 || n_q % n_kv ||
        page_size <= 0 || window < 0)
        return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    const long long blocks = ((long long)tokens * n_q + warps - 1) / warps;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    if (dtype == KIPP_DT_F32)
        return kipp_launch(paged_attention_simt_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), smem, s, 1,
            (float*)out, (const float*)q, (const float*)k_pages, (const float*)v_pages, positions,
            entry_of_token, block_table, table_width, page_size, tokens, n_q, n_kv, head_dim, scale,
            window, status);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(paged_attention_simt_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), smem, s, 1,
            (bf16*)out, (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, positions,
            entry_of_token, block_table, table_width, page_size, tokens, n_q, n_kv, head_dim, scale,
            window, status);
    return KIPP_ERR_DTYPE;
}
