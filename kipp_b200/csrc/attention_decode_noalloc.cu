// Split-K decode attention with its scratch memory built into the library, for
// callers that cannot allocate on the device.  See attention_decode_noalloc.h
// for who needs this, what it costs and the rules; no counterpart in the
// reference.
//
// The kernels are those of attention_mma.cu, compiled into this library too;
// only where the scratch comes from differs.
#include "attention_mma.cu"
#include "attention_decode_noalloc.h"

namespace {
// The scratch itself: device memory that every GPU loading this library holds
// until the process ends.
static __device__ __align__(256) unsigned char g_noalloc_scratch[KIPP_NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
float* g_scratch_ptr[MAX_DEVICES];      // device address of the array, per device, once looked up

// In host code `g_noalloc_scratch` names a host-side stand-in, not device
// memory: the kernels must be given the address cudaGetSymbolAddress returns
// for the CURRENT device.  Done once per device, on the first call there.
int scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return KIPP_ERR_ARG;
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return (int)cudaErrorInvalidSymbol;
        g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_ptr[dev];
    return 0;
}
}  // namespace

// partial outputs and (max, sum) pairs of every split (this entry point cuts every token into
// splits of the given length, which needs nothing more)
extern "C" long long kipp_attn_decode_noalloc_scratch_bytes(int n, int n_q, int head_dim, int max_splits) {
    return (long long)n * n_q * max_splits * (head_dim + 2) * 4;
}

extern "C" int kipp_attn_decode_mma_noalloc(void* out, const void* q, const void* k_pages, const void* v_pages,
                                            const int* q_start, const int* context_len,
                                            const int* block_table, int table_width, int page_size,
                                            const int* rows, int n, int n_q, int n_kv, int head_dim,
                                            float scale, int window, int max_splits, const int* split_keys,
                                            void* stream) {
    if (n <= 0) return 0;
    if (n_q <= 0 || head_dim <= 0 || max_splits <= 0) return KIPP_ERR_ARG;
    // refuse before anything is launched: the built-in scratch has one size
    if (kipp_attn_decode_noalloc_scratch_bytes(n, n_q, head_dim, max_splits) > KIPP_NOALLOC_SCRATCH_BYTES)
        return KIPP_ERR_SCRATCH;
    float* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    return kipp_attn_decode_mma(out, q, k_pages, v_pages, q_start, context_len, block_table, table_width,
                                page_size, rows, n, n_q, n_kv, head_dim, scale, window, max_splits, split_keys, 0,
                                0, scratch, stream);
}
