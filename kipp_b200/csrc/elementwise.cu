// Embedding gather and RMSNorm.
//
// Reference counterparts: embed_kernel (cuda/kipp_kernels.cu:35) handles one
// token per launch, rms_norm_kernel (cuda/kipp_kernels.cu:44) one row in one
// block.  These take any number of tokens / rows per launch.
#include "common.cuh"

// out[t, :] = float(table[ids[t], :]).  The residual stream is float32.
template <typename TW>
__global__ void embed_gather_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                    const int* __restrict__ ids, int hidden, int vocab,
                                    int* __restrict__ status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    if (id < 0 || id >= vocab) {           // never read outside the table
        if (threadIdx.x == 0) atomicExch(status, 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = 0.f;
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]);
}

extern "C" int kipp_embed_gather(float* out, const void* table, int table_dtype, const int* ids,
                                 int tokens, int hidden, int vocab, int* status, void* stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == KIPP_DT_F32)
        embed_gather_kernel<float><<<tokens, threads, 0, s>>>(out, (const float*)table, ids, hidden, vocab, status);
    else if (table_dtype == KIPP_DT_BF16)
        embed_gather_kernel<bf16><<<tokens, threads, 0, s>>>(out, (const bf16*)table, ids, hidden, vocab, status);
    else
        return KIPP_ERR_DTYPE;
    return kipp_launch_status();
}

// y[r, i] = x[src(r), i] * rsqrt(mean(x[src(r), :]^2) + eps) * w[i]
// (src/kipp.c:2221-2231).  Sum of squares and scale in float32.  `rows`, when
// not null, gathers the input rows (used for the rows whose logits are wanted).
template <typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x,
                               const void* __restrict__ w, int w_dtype, const int* __restrict__ rows,
                               int size, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = src[i];
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)size + eps);
    TO* dst = out + (size_t)r * size;
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        dst[i] = from_f32<TO>(src[i] * scale * load_w(w, w_dtype, i));
}

extern "C" int kipp_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype,
                            const int* rows, int n_rows, int size, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if (size <= 0) return KIPP_ERR_ARG;
    if (w_dtype != KIPP_DT_F32 && w_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = size >= 2048 ? 512 : (size >= 512 ? 256 : 64);
    if (out_dtype == KIPP_DT_F32)
        rmsnorm_kernel<float><<<n_rows, threads, 0, s>>>((float*)out, x, w, w_dtype, rows, size, eps);
    else if (out_dtype == KIPP_DT_BF16)
        rmsnorm_kernel<bf16><<<n_rows, threads, 0, s>>>((bf16*)out, x, w, w_dtype, rows, size, eps);
    else
        return KIPP_ERR_DTYPE;
    return kipp_launch_status();
}
