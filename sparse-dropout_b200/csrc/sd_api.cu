// Library-level pieces of the C ABI: version, thread-local error text, cached device facts.
#include <string.h>

#include <atomic>

#include "sd_common.h"

namespace sd {

char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

int sm_count_current_device(int* out) {
    static std::atomic<int> cached[64] = {};   // read from several host threads at once
    int dev = 0;
    SD_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64) {
        const int have = cached[dev].load(std::memory_order_relaxed);
        if (have > 0) {
            *out = have;
            return SD_OK;
        }
    }
    int n = 0;
    SD_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    if (dev < 64) cached[dev].store(n, std::memory_order_relaxed);
    *out = n;
    return SD_OK;
}

}  // namespace sd

extern "C" {

int sd_version(void) { return 100; }

const char* sd_last_error(void) { return sd::error_buffer(); }

}  // extern "C"
