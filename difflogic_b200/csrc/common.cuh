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

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  With DL_LAUNCH_OVERLAP_SETUP the small training kernels are
// launched so that a kernel's set-up (reading the connection indices / the gather plan) may run
// while the previous kernel in the stream is still draining; everything else is touched only
// after grid_dependency_wait().  Without the launch attribute the two device calls are no-ops,
// so the same kernels are correct under an ordinary launch.  dl_set_tuning(DL_TUNE_NO_PDL, 1) (or DL_PDL=0 in the
// environment when the library is loaded) turns the attribute off everywhere.
// ---------------------------------------------------------------------------------------------
namespace dl {

bool pdl_enabled();
int tuning(int key);  // current value of a DL_TUNE_* switch (dl_set_tuning); 0 = automatic choice

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Asks for a line to be brought into L2 without reading its value: safe before grid_dependency_wait() even
// when the previous kernel may still be writing the line (L2 is where its writes land anyway).
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_dependent(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                           Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = (overlap && pdl_enabled()) ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

}  // namespace dl
