// Row-wise copy with a change of element type: how checkpoint tensors reach the
// form the kernels want when a model is bound.  One launch moves `rows` rows of
// `cols` elements from a source with its own pitch into a destination with its
// own pitch, so the same kernel concatenates matrices (q, k and v projections
// into one), interleaves them row by row (gate and up) and widens or narrows
// the elements on the way.  The reference uploads its tensors as stored and
// converts in every kernel (src/cuda/kipp_cuda.cu:563-577); here the conversion
// happens once.
//
// Source types: float32, bfloat16, float16 and the integer types a checkpoint
// may hold; destinations: float32, bfloat16 (round to nearest even, the
// reference's narrowing, src/kipp.c:2181-2186) or int32 for integer tables.
#include <cuda_fp16.h>

#include "common.cuh"

#define KIPP_DT_F16 2
#define KIPP_DT_I32 3
#define KIPP_DT_I64 4
#define KIPP_DT_I16 5
#define KIPP_DT_I8 6
#define KIPP_DT_U8 7

namespace {
__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
    switch (dtype) {
        case KIPP_DT_F32: return reinterpret_cast<const float*>(p)[i];
        case KIPP_DT_BF16: return __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
        case KIPP_DT_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
        default: return 0.f;
    }
}
__device__ __forceinline__ int load_as_int(const void* p, int dtype, size_t i) {
    switch (dtype) {
        case KIPP_DT_I32: return reinterpret_cast<const int*>(p)[i];
        case KIPP_DT_I64: return (int)reinterpret_cast<const long long*>(p)[i];
        case KIPP_DT_I16: return reinterpret_cast<const short*>(p)[i];
        case KIPP_DT_I8: return reinterpret_cast<const signed char*>(p)[i];
        case KIPP_DT_U8: return reinterpret_cast<const unsigned char*>(p)[i];
        default: return 0;
    }
}

__global__ void convert_rows_kernel(void* __restrict__ dst, int dst_dtype, long long dst_pitch,
                                    const void* __restrict__ src, int src_dtype, long long src_pitch,
                                    long long rows, long long cols) {
    const long long n = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i - r * cols;
        const size_t s = (size_t)(r * src_pitch + c), d = (size_t)(r * dst_pitch + c);
        if (dst_dtype == KIPP_DT_I32) {
            reinterpret_cast<int*>(dst)[d] = load_as_int(src, src_dtype, s);
        } else {
            const float v = load_as_float(src, src_dtype, s);
            if (dst_dtype == KIPP_DT_F32) reinterpret_cast<float*>(dst)[d] = v;
            else reinterpret_cast<bf16*>(dst)[d] = __float2bfloat16_rn(v);
        }
    }
}
}  // namespace

// dst[r * dst_pitch + c] = convert(src[r * src_pitch + c]); pitches in elements.
extern "C" int kipp_convert_rows(void* dst, int dst_dtype, long long dst_pitch, const void* src, int src_dtype,
                                 long long src_pitch, long long rows, long long cols, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const bool float_dst = dst_dtype == KIPP_DT_F32 || dst_dtype == KIPP_DT_BF16;
    const bool float_src = src_dtype == KIPP_DT_F32 || src_dtype == KIPP_DT_BF16 || src_dtype == KIPP_DT_F16;
    const bool int_src = src_dtype >= KIPP_DT_I32 && src_dtype <= KIPP_DT_U8;
    if (!(float_dst && float_src) && !(dst_dtype == KIPP_DT_I32 && int_src)) return KIPP_ERR_DTYPE;
    const long long n = rows * cols;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    // a plain launch (no dependent-launch attribute): binding is not on the step path
    convert_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(dst, dst_dtype, dst_pitch, src, src_dtype,
                                                                            src_pitch, rows, cols);
    return kipp_launch_status();
}
