// Shared helpers of the sm_100a kernels: element types, conversions, warp and
// block reductions with a fixed order, and the launch-status convention.
//
// Every exported launcher is `extern "C" int kipp_<name>(..., void* stream)`
// and returns 0 or a negative argument-error code / a positive cudaError_t.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KIPP_ERR_ARG (-1)        // a size the kernel refuses
#define KIPP_ERR_DTYPE (-2)      // unknown dtype code
#define KIPP_DT_F32 0
#define KIPP_DT_BF16 1

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
// Round to nearest even, as the reference narrows (src/kipp.c:2181-2186).
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Loads an element of a weight vector stored either as float32 or bfloat16.
__device__ __forceinline__ float load_w(const void* p, int dtype, size_t i) {
    return dtype == KIPP_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                                : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 32 floats.  Order is fixed by thread index.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float t = lane < nwarps ? scratch[lane] : 0.f;
    return warp_sum(t);
}

static inline int kipp_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
