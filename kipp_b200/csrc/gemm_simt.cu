// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores with float32 accumulation.
//
// This is the matrix product of the true 32-bit path (float32 operands, plain
// FMA, no tensor-core mode) and the fallback of the bfloat16 path for shapes
// the tensor-core kernels refuse.  The reference computes the same product
// one output row per block and one token per launch (matvec_kernel,
// cuda/kipp_kernels.cu:93; src/kipp.c:2233-2243).
//
// The sum over k runs in the same order for every output element whatever M
// is, so a token's result does not depend on what else is in the batch.
//
// Epilogues:
//   STORE   C[m,n]    = acc                 (C in float32 or bfloat16)
//   ADD     C[m,n]   += acc                 (C float32: the residual stream)
//   SWIGLU  C[m,n/2]  = silu(acc[n]) * acc[n+1] for even n, W holding gate and
//           up rows interleaved (src/kipp.c:2402-2404, 3002-3005)
#include "common.cuh"

#define EPI_STORE 0
#define EPI_ADD 1
#define EPI_SWIGLU 2

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W,
                 int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // 64x16 tile = 1024 elements, 256 threads -> 4 each; thread loads row
    // (tid / 4), k columns (tid % 4) * 4 .. + 3.
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + i][lrow] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
            Ws[lk + i][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)wn * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
        if (EPI == EPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < TN; j += 2) {
                const int n = n0 + tx * TN + j;
                if (n + 1 < N) {
                    const float g = acc[i][j], u = acc[i][j + 1];
                    C[(size_t)m * ldc + (n >> 1)] = from_f32<TC>(g / (1.0f + expf(-g)) * u);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int n = n0 + tx * TN + j;
                if (n >= N) continue;
                const size_t idx = (size_t)m * ldc + n;
                if (EPI == EPI_ADD) C[idx] = from_f32<TC>(to_f32(C[idx]) + acc[i][j]);
                else C[idx] = from_f32<TC>(acc[i][j]);
            }
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
           int epi, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return KIPP_ERR_ARG;
    switch (epi) {
    case EPI_STORE:
        return kipp_launch(gemm_simt_kernel<TA, TW, TC, EPI_STORE>, grid, dim3(256), 0, s, 1, (TC*)C, (const TA*)A,
                           (const TW*)W, M, N, K, lda, ldw, ldc);
    case EPI_ADD:
        return kipp_launch(gemm_simt_kernel<TA, TW, TC, EPI_ADD>, grid, dim3(256), 0, s, 1, (TC*)C, (const TA*)A,
                           (const TW*)W, M, N, K, lda, ldw, ldc);
    case EPI_SWIGLU:
        if (N & 1) return KIPP_ERR_ARG;
        return kipp_launch(gemm_simt_kernel<TA, TW, TC, EPI_SWIGLU>, grid, dim3(256), 0, s, 1, (TC*)C, (const TA*)A,
                           (const TW*)W, M, N, K, lda, ldw, ldc);
    default:
        return KIPP_ERR_ARG;
    }
}
}  // namespace

// in_dtype: dtype of A and W (both float32 or both bfloat16); out_dtype: dtype of C.
extern "C" int kipp_gemm_simt(void* C, int out_dtype, const void* A, const void* W, int in_dtype,
                              int M, int N, int K, int lda, int ldw, int ldc, int epilogue,
                              void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == EPI_ADD && out_dtype != KIPP_DT_F32) return KIPP_ERR_DTYPE;
    if (in_dtype == KIPP_DT_F32 && out_dtype == KIPP_DT_F32)
        return launch<float, float, float>(C, A, W, M, N, K, lda, ldw, ldc, epilogue, s);
    if (in_dtype == KIPP_DT_BF16 && out_dtype == KIPP_DT_F32)
        return launch<bf16, bf16, float>(C, A, W, M, N, K, lda, ldw, ldc, epilogue, s);
    if (in_dtype == KIPP_DT_BF16 && out_dtype == KIPP_DT_BF16)
        return launch<bf16, bf16, bf16>(C, A, W, M, N, K, lda, ldw, ldc, epilogue, s);
    return KIPP_ERR_DTYPE;
}
