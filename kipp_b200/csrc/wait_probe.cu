// A probe of the bounded mbarrier wait (mbarrier.cuh), for the test that makes a wait run out
// without making any kernel of the engine fail: one CTA initialises a barrier that nothing
// ever arrives at, waits on it with a limit of `limit_cycles` SM clocks through the helper the
// tensor-core kernels use, and writes what the helper returned and how long it waited.  It
// allocates no tensor memory and starts no copy, so there is nothing to drain; it returns by
// itself when the limit has passed.
#include "common.cuh"
#include "mbarrier.cuh"

namespace {
__global__ void wait_probe_kernel(int* status, long long* waited, long long limit_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(kipp_smem_u32(&bar)), "r"(1));
    }
    __syncthreads();
    const long long t0 = clock64();
    const bool ok = kipp_mbar_wait_limited(&bar, 0, &abort_flag, limit_cycles);
    const long long dt = clock64() - t0;
    if (!ok) atomicMax(&status[1], 1);            // the word the tensor-core kernels set when a wait ran out
    if (threadIdx.x == 0) *waited = dt;
}
}  // namespace

// limit_cycles is clamped to [1 thousand, 100 million] SM clocks (at most some 50 ms).
extern "C" int kipp_wait_probe(int* status, long long* waited_cycles, long long limit_cycles, void* stream) {
    if (status == nullptr || waited_cycles == nullptr) return KIPP_ERR_ARG;
    if (limit_cycles < 1000) limit_cycles = 1000;
    if (limit_cycles > 100000000ll) limit_cycles = 100000000ll;
    wait_probe_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, waited_cycles, limit_cycles);
    return kipp_launch_status();
}
