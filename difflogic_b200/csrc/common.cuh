// Shared host/device helpers of the difflogic_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "difflogic_b200.h"

namespace dl {

constexpr int kThreads = 256;  // CTA size of the row kernels: 8 warps

// Records a message for dl_last_error_string() on this thread and returns `code`.
int fail(int code, const char *fmt, ...);
// Status of the launch just issued (no synchronisation).
int launch_status(const char *what);

static inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }
static inline int pow2_at_least(int64_t v, int cap) {
    int g = 1;
    while (g < cap && g < v) g <<= 1;
    return g;
}

}  // namespace dl

#define DL_REQUIRE(cond, code, ...)                       \
    do {                                                  \
        if (!(cond)) return dl::fail((code), __VA_ARGS__); \
    } while (0)
