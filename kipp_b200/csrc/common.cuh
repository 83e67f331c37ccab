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

// What goes into the cache must be a finite number in the cache's type: kernels that read whole
// tiles multiply masked keys and values by zero, and a page is handed from one request to the
// next as it is, so one request's overflow must not leave an infinity or a NaN behind for the
// next one.  A value that is not finite (or would round to an infinity in bfloat16) is stored as 0.
__device__ __forceinline__ float cache_value(float v) { return fabsf(v) < 3.38e38f ? v : 0.f; }
// the same for eight bfloat16 values in a 16-byte vector: lanes with all exponent bits set become 0
__device__ __forceinline__ uint4 cache_values_bf16x8(uint4 v) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if ((w[i] & 0x7f800000u) == 0x7f800000u) w[i] &= 0x0000ffffu;
        if ((w[i] & 0x00007f80u) == 0x00007f80u) w[i] &= 0xffff0000u;
    }
    return v;
}

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

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of this package is launched with
// the programmatic-stream-serialization attribute (unless KIPP_B200_PDL=0): its
// blocks may be scheduled while the kernel before it in the stream drains, so
// launch latency and each kernel's set-up hide behind the previous kernel's
// tail.  The rule every kernel keeps: call pdl_wait() before the first access
// to global memory that an earlier kernel may have written or may still read;
// only set-up that touches nothing of the sort (barrier init, tensor-memory
// allocation, loads of weights) may come before it.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#include <stdlib.h>
static inline bool kipp_pdl_enabled() {
    static int cached = -1;
    if (cached < 0) {
        const char* e = getenv("KIPP_B200_PDL");
        cached = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return cached == 1;
}

// Launches `kernel` with the package's attributes; a cluster of more than one
// CTA makes thread-block clusters of that shape.
template <typename... KArgs, typename... Args>
static inline int kipp_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, dim3 cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (kipp_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return 0;
}

// cluster_z > 1 makes the grid's z dimension one thread-block cluster.
template <typename... KArgs, typename... Args>
static inline int kipp_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_z, Args&&... args) {
    return kipp_launch_cluster(kernel, grid, block, smem, stream, dim3(1, 1, cluster_z > 1 ? cluster_z : 1),
                               static_cast<Args&&>(args)...);
}

static inline int kipp_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
