// Per-head q/k RMSNorm and rotation of bfloat16 heads, with every rounding spelled out
// (explicit fused multiply-adds instead of what the compiler would contract), so that the
// kernels that include this file give the same bits for the same head: the kernel that
// reads the stored projection and the projection's own epilogue.
//
// A head of D values is handled in blocks of 16: 8 values a[i] = x[8 s + i] of the first half
// and their rotation partners b[i] = x[D / 2 + 8 s + i], s = 0 .. D / 16 - 1.  The sum of squares
// is formed per block in the order of `head_ssq8` and the D / 16 block sums are added as a
// butterfly over s (distance D / 32 first), `head_ssq_tree` being the same sum in one thread.
// Formulas: src/kipp.c:2316-2330 (norm over the head), 2352-2382 (half-split rotation).
#pragma once
#include "common.cuh"

__device__ __forceinline__ float head_ssq8(const float (&a)[8], const float (&b)[8]) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = __fmaf_rn(b[i], b[i], __fmaf_rn(a[i], a[i], ss));
    return ss;
}

// The butterfly sum over the block sums part[0 .. N), N a power of two: what every lane holds
// after `ss += shfl_xor(ss, o)` for o = N / 2, N / 4, .. 1.
template <int N> __device__ __forceinline__ float head_ssq_tree(float (&part)[N]) {
#pragma unroll
    for (int o = N / 2; o > 0; o >>= 1) {
#pragma unroll
        for (int s = 0; s < o; ++s) part[s] = __fadd_rn(part[s], part[s + o]);
    }
    return part[0];
}

__device__ __forceinline__ float head_rstd(float ss, int head_dim, float eps) {
    return __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)head_dim), eps)));
}

// x * rstd * w, in this order
__device__ __forceinline__ void head_scale8(float (&x)[8], float rstd, const float (&w)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(__fmul_rn(x[i], rstd), w[i]);
}

// Rotates the pair (a, b) by the angle whose (cos, sin) is cs.
__device__ __forceinline__ void head_rotate(float& a, float& b, float2 cs) {
    const float a0 = a, b0 = b;
    a = __fmaf_rn(a0, cs.x, -__fmul_rn(b0, cs.y));
    b = __fmaf_rn(b0, cs.x, __fmul_rn(a0, cs.y));
}
// The pairs (a[i], b[i]) by the angles whose (cos, sin) lie at cs[i] (16-byte aligned).
__device__ __forceinline__ void head_rotate8(float (&a)[8], float (&b)[8], const float2* cs) {
    const float4* cs4 = reinterpret_cast<const float4*>(cs);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 c = cs4[i];                  // (cos, sin) of pairs 2 i and 2 i + 1
        head_rotate(a[2 * i], b[2 * i], make_float2(c.x, c.y));
        head_rotate(a[2 * i + 1], b[2 * i + 1], make_float2(c.z, c.w));
    }
}

__device__ __forceinline__ void unpack8(float (&x)[8], const uint4& raw) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { x[2 * i] = __low2float(h2[i]); x[2 * i + 1] = __high2float(h2[i]); }
}
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
    uint4 out;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    return out;
}
// elements first .. first + 7 of a norm weight (16-byte aligned)
__device__ __forceinline__ void load_w8(float (&w)[8], const void* nw, int norm_dtype, int first) {
    if (norm_dtype == KIPP_DT_F32) {
        const float4 a = reinterpret_cast<const float4*>(nw)[first / 4], b = reinterpret_cast<const float4*>(nw)[first / 4 + 1];
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else {
        unpack8(w, reinterpret_cast<const uint4*>(nw)[first / 8]);
    }
}
