// Host-side helpers shared by the C-ABI translation units: thread-local error text,
// CUDA error mapping and a per-device cache of immutable device properties.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include "../../include/sparsedrop.h"

namespace sd {

char* error_buffer();                       // thread-local, 512 bytes
int fail(int code, const char* fmt, ...);   // formats into error_buffer() and returns code
int sm_count_current_device(int* out);      // cached cudaDevAttrMultiProcessorCount

#define SD_CUDA_TRY(expr)                                                                     \
    do {                                                                                      \
        cudaError_t err__ = (expr);                                                           \
        if (err__ != cudaSuccess)                                                             \
            return ::sd::fail(SD_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

}  // namespace sd
