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
    pdl_launch_dependents();
    pdl_wait();
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
        return kipp_launch(embed_gather_kernel<float>, dim3(tokens), dim3(threads), 0, s, 1, out,
                           (const float*)table, ids, hidden, vocab, status);
    if (table_dtype == KIPP_DT_BF16)
        return kipp_launch(embed_gather_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, 1, out,
                           (const bf16*)table, ids, hidden, vocab, status);
    return KIPP_ERR_DTYPE;
}

// y[r, i] = x[src(r), i] * rsqrt(mean(x[src(r), :]^2) + eps) * w[i]
// (src/kipp.c:2221-2231).  Sum of squares and scale in float32.  `rows`, when
// not null, gathers the input rows (used for the rows whose logits are wanted).
template <typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x,
                               const void* __restrict__ w, int w_dtype, const int* __restrict__ rows,
                               int size, float eps, float* __restrict__ ssq_out) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = src[i];
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    // deferred form: x * w alone goes out, the sum of squares beside it (see kipp_rmsnorm_deferred)
    const float scale = ssq_out ? 1.0f : 1.0f / sqrtf(ss / (float)size + eps);
    if (ssq_out && threadIdx.x == 0) ssq_out[r] = ss;
    TO* dst = out + (size_t)r * size;
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        dst[i] = from_f32<TO>(src[i] * scale * load_w(w, w_dtype, i));
}

// Vector path: size a multiple of 4 and at most 4096; each of 256 threads keeps
// its float4 pieces of the row in registers, so the row is read once.
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(TO* __restrict__ out, const float* __restrict__ x, const void* __restrict__ w, int w_dtype,
                   const int* __restrict__ rows, int size, float eps, float* __restrict__ ssq_out) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * size);
    const int n4 = size >> 2;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < n4) {
            v[j] = src[i];
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = ssq_out ? 1.0f : 1.0f / sqrtf(ss / (float)size + eps);
    if (ssq_out && threadIdx.x == 0) ssq_out[r] = ss;
    TO* dst = out + (size_t)r * size;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i < n4) {
            const size_t e = (size_t)i * 4;
            const float a = v[j].x * scale * load_w(w, w_dtype, e), b = v[j].y * scale * load_w(w, w_dtype, e + 1);
            const float c = v[j].z * scale * load_w(w, w_dtype, e + 2), d = v[j].w * scale * load_w(w, w_dtype, e + 3);
            if (sizeof(TO) == 4) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + e) = make_float4(a, b, c, d);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(dst) + e) = packed;
            }
        }
    }
}

static int rmsnorm_launch(void* out, int out_dtype, const float* x, const void* w, int w_dtype, const int* rows,
                          int n_rows, int size, float eps, float* ssq_out, void* stream) {
    if (n_rows <= 0) return 0;
    if (size <= 0) return KIPP_ERR_ARG;
    if (w_dtype != KIPP_DT_F32 && w_dtype != KIPP_DT_BF16) return KIPP_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    if (size % 4 == 0 && size <= 4096 && size >= 256 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        if (out_dtype == KIPP_DT_F32)
            return kipp_launch(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(256), 0, s, 1, (float*)out, x, w,
                               w_dtype, rows, size, eps, ssq_out);
        if (out_dtype == KIPP_DT_BF16)
            return kipp_launch(rmsnorm_vec_kernel<bf16>, dim3(n_rows), dim3(256), 0, s, 1, (bf16*)out, x, w,
                               w_dtype, rows, size, eps, ssq_out);
        return KIPP_ERR_DTYPE;
    }
    int threads = size >= 2048 ? 512 : (size >= 512 ? 256 : 64);
    if (out_dtype == KIPP_DT_F32)
        return kipp_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, 1, (float*)out, x, w, w_dtype,
                           rows, size, eps, ssq_out);
    if (out_dtype == KIPP_DT_BF16)
        return kipp_launch(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, 1, (bf16*)out, x, w, w_dtype,
                           rows, size, eps, ssq_out);
    return KIPP_ERR_DTYPE;
}

extern "C" int kipp_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype,
                            const int* rows, int n_rows, int size, float eps, void* stream) {
    return rmsnorm_launch(out, out_dtype, x, w, w_dtype, rows, n_rows, size, eps, nullptr, stream);
}

// The norm with its per-row factor left to whoever reads the result: out[r, i] = x[row r, i] * w[i]
// (rounded to out's type) and ssq_out[r] = sum of x[row r, :]^2, so that
// rmsnorm(x)[r] = out[r] / sqrt(ssq_out[r] / size + eps).  A matrix product that follows applies
// the factor to its own result rows in float32 (kipp_gemm_tc_fold); a residual add that leaves
// x * w itself (the same kernel library) rounds the same values the same way, so both routes to
// the product's input agree to the bit.
extern "C" int kipp_rmsnorm_deferred(void* out, int out_dtype, float* ssq_out, const float* x, const void* w,
                                     int w_dtype, const int* rows, int n_rows, int size, void* stream) {
    if (ssq_out == nullptr) return KIPP_ERR_ARG;
    return rmsnorm_launch(out, out_dtype, x, w, w_dtype, rows, n_rows, size, 0.f, ssq_out, stream);
}
