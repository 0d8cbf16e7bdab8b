// Shared host-side helpers of libchxq: status codes, thread-local error text, dtype helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "../../include/chxq.h"
#include "../../include/chxq_testing.h"

namespace chxq {

// Records the message returned by chxq_last_error() for this thread and returns `code`.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

inline bool is_q8(int dtype) {
    return dtype == CHXQ_UINT8 || dtype == CHXQ_INT8;
}

inline cudaStream_t as_stream(void* s) {
    return reinterpret_cast<cudaStream_t>(s);
}

// Device status word (one per device; set by kernels whose bounded waits expire).
int* device_status_ptr();

// Process-wide count of kernels this library has launched (chxq_launch_count()).
void count_launch(int n = 1);

#define CHXQ_CHECK_ARG(cond, ...)                                         \
    do {                                                                  \
        if (!(cond)) return ::chxq::set_error(CHXQ_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define CHXQ_CUDA(expr)                                                                                           \
    do {                                                                                                          \
        cudaError_t e_ = (expr);                                                                                  \
        if (e_ != cudaSuccess)                                                                                    \
            return ::chxq::set_error(CHXQ_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

#define CHXQ_LAUNCH_CHECK()            \
    do {                               \
        ::chxq::count_launch(1);       \
        CHXQ_CUDA(cudaGetLastError()); \
    } while (0)

}  // namespace chxq
