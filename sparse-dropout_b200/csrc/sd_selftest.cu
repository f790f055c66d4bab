// Self-test of the bounded device-side waits: a one-warp kernel waits on an mbarrier nobody arrives on and on a
// counter nobody increments, with a caller-chosen (short) limit.  Both waits must give up, record their code in the
// status word and let the kernel return normally, leaving the context usable.  This is how the time-out path of the
// GEMM kernel is exercised without ever hanging or faulting a GPU.
#include "sd_common.h"
#include "sd_ptx.cuh"

namespace sd {

__global__ void bounded_wait_selftest_kernel(int* words, unsigned long long limit_ns) {
    __shared__ unsigned long long bar;
    __shared__ int abort_a, abort_b;
    if (threadIdx.x == 0) {
        abort_a = abort_b = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
        const unsigned long long t0 = global_timer_ns();
        const bool ok_bar = mbar_wait(smem_u32(&bar), 0, &abort_a, words + 0, 101, limit_ns);       // never completes
        const bool ok_cnt = counter_wait(words + 1, 1, &abort_b, words + 0, 102, limit_ns);        // words[1] stays 0
        words[2] = (ok_bar ? 1 : 0) | (ok_cnt ? 2 : 0) | (abort_a ? 4 : 0) | (abort_b ? 8 : 0);
        words[3] = int((global_timer_ns() - t0) / 1000);                                            // microseconds
    }
}

}  // namespace sd

extern "C" int sd_selftest_bounded_wait(int* words, uint64_t limit_ns, void* stream) {
    if (!words) return sd::fail(SD_ERR_INVALID_ARG, "words is null");
    if (limit_ns == 0 || limit_ns > 1000000000ull)
        return sd::fail(SD_ERR_INVALID_ARG, "limit_ns must be in (0, 1e9]: the self-test is meant to give up quickly");
    SD_CUDA_TRY(cudaMemsetAsync(words, 0, 4 * sizeof(int), static_cast<cudaStream_t>(stream)));
    sd::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(words, limit_ns);
    SD_CUDA_TRY(cudaGetLastError());
    return SD_OK;
}
