// Gradient exchange and optimizer step of batch-sharded training in ONE kernel, over peer memory.
//
// Every rank (one process per GPU) keeps the flat gradient buffer and the flat parameter buffer of the network in
// memory that its peers have mapped (CUDA IPC over NVLink).  After the backward pass each rank owns one slice of
// the parameters:
//   1. barrier A: every rank tells every peer that its gradients are complete (a flag store into the peer's
//      memory) and waits until all peers have said so;
//   2. for its slice it reads that slice of ALL ranks' gradients straight from their memory (16-byte loads over
//      NVLink), averages, applies Adam with its slice of the moments, and stores the new parameters into its own
//      parameter buffer and into every peer's;
//   3. barrier B: when all its stores are out (system-wide fence) it tells the peers, and waits for theirs; the
//      kernel ends with every rank holding the complete updated parameters.
// This replaces an NCCL all-reduce of the gradients followed by a full Adam step on every rank: the bytes that
// cross NVLink are the same as a reduce-scatter plus all-gather, there is no extra launch, and each rank touches
// only 1/N of the optimizer state.
//
// The peers are other GPUs of this machine mapped by plain peer-to-peer access; the loads and stores are ordinary
// ld/st instructions.  Every wait is bounded (kExchangeSpinLimit polls); when one runs out the kernel records it
// in the state words and carries on, so a missing rank cannot hang the others.
#include <string.h>

#include "common.cuh"

namespace dl {

constexpr int kMaxRanks = 16;
constexpr unsigned kExchangeSpinLimit = 1u << 22;

struct ExchangePeers {
    float *param[kMaxRanks];      // flat parameter buffer of each rank (index = rank; own entry is local memory)
    const float *grad[kMaxRanks]; // flat gradient buffer of each rank
    int *flags[kMaxRanks];        // flag words of each rank: flags[r][2*p + b] is written by rank p for barrier b
};

__device__ __forceinline__ int ld_acquire_sys(const int *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int *p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer(const float4 *p) {
    // peers rewrite this memory every step: read it past the L1 cache
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// Waits until every peer's flag for barrier `b` has reached `epoch`; false when the poll limit ran out.
__device__ __forceinline__ bool wait_peers(const int *my_flags, int world, int b, int epoch) {
    for (int p = 0; p < world; ++p) {
        unsigned spin = 0;
        while (ld_acquire_sys(my_flags + 2 * p + b) < epoch) {
            if (++spin > kExchangeSpinLimit) return false;
        }
    }
    return true;
}

// state: [0] steps done, [1] ticket of finished blocks, [2] error (a wait ran out)
__global__ void __launch_bounds__(kThreads)
adam_exchange_kernel(ExchangePeers peers, int rank, int world, float *__restrict__ m, float *__restrict__ v, int64_t n4_total,
                     float lr, float beta1, float beta2, float eps, int *__restrict__ state) {
    __shared__ float s_step_size, s_bc2_sqrt;
    __shared__ int s_ok;
    grid_dependency_wait();  // this rank's gradients come from the kernels just before
    const int epoch = state[0] + 1;
    // barrier A: announce (once per rank), then everybody waits on the local flag words
    if (blockIdx.x == 0 && threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + 2 * rank + 0, epoch);
    if (threadIdx.x == 0) {
        s_ok = wait_peers(peers.flags[rank], world, 0, epoch) ? 1 : 0;
        const float t = (float)epoch;
        s_step_size = lr / (1.f - powf(beta1, t));
        s_bc2_sqrt = sqrtf(1.f - powf(beta2, t));
    }
    __syncthreads();
    if (!s_ok && threadIdx.x == 0) state[2] = 1;
    const float step_size = s_step_size, bc2_sqrt = s_bc2_sqrt;
    const float omb1 = 1.f - beta1, omb2 = 1.f - beta2, inv_world = 1.f / (float)world;

    // this rank's slice, in float4 units
    const int64_t per = (n4_total + world - 1) / world;
    const int64_t lo = min((int64_t)rank * per, n4_total), hi = min(lo + per, n4_total);
    float4 *m4 = reinterpret_cast<float4 *>(m), *v4 = reinterpret_cast<float4 *>(v);  // moments of the slice only
    for (int64_t i = lo + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < hi; i += (int64_t)gridDim.x * kThreads) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < world; ++p) {
            const float4 gp = ld_peer(reinterpret_cast<const float4 *>(peers.grad[p]) + i);
            g.x += gp.x; g.y += gp.y; g.z += gp.z; g.w += gp.w;
        }
        float4 pp = reinterpret_cast<float4 *>(peers.param[rank])[i];
        float4 mm = m4[i - lo], vv = v4[i - lo];
#define DL_ADAM1(c)                                          \
    {                                                        \
        const float gr = g.c * inv_world;                    \
        mm.c = mm.c + (gr - mm.c) * omb1;                    \
        vv.c = vv.c * beta2 + gr * gr * omb2;                \
        const float denom = sqrtf(vv.c) / bc2_sqrt + eps;    \
        pp.c = pp.c - step_size * (mm.c / denom);            \
    }
        DL_ADAM1(x) DL_ADAM1(y) DL_ADAM1(z) DL_ADAM1(w)
#undef DL_ADAM1
        m4[i - lo] = mm;
        v4[i - lo] = vv;
        for (int p = 0; p < world; ++p) reinterpret_cast<float4 *>(peers.param[p])[i] = pp;
    }

    // barrier B: every thread pushes its stores out to system scope; the last block to finish announces, waits
    // for the peers, and advances the step counter
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const int done = atomicAdd(state + 1, 1);
        if (done == (int)gridDim.x - 1) {
            for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 2 * rank + 1, epoch);
            if (!wait_peers(peers.flags[rank], world, 1, epoch)) state[2] = 1;
            state[1] = 0;
            state[0] = epoch;
        }
    }
}

}  // namespace dl

using namespace dl;

// ---- set-up helpers: memory that peers can map.  These allocate; they are not part of the per-step path. ----

extern "C" DL_API int dl_comm_alloc(size_t bytes, void **ptr) {
    DL_REQUIRE(ptr != nullptr && bytes > 0, DL_ERR_INVALID_ARG, "dl_comm_alloc: bad argument");
    const cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(DL_ERR_CUDA, "dl_comm_alloc: %s", cudaGetErrorString(e));
    }
    if (cudaMemset(*ptr, 0, bytes) != cudaSuccess) return launch_status("dl_comm_alloc (clearing)");
    return DL_OK;
}

extern "C" DL_API int dl_comm_free(void *ptr) {
    if (ptr != nullptr && cudaFree(ptr) != cudaSuccess) return launch_status("dl_comm_free");
    return DL_OK;
}

// handle: 64 bytes that another process on the same machine turns into a pointer with dl_comm_import
extern "C" DL_API int dl_comm_export(void *ptr, unsigned char *handle) {
    DL_REQUIRE(ptr && handle, DL_ERR_INVALID_ARG, "dl_comm_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(DL_ERR_CUDA, "dl_comm_export: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, 64);
    return DL_OK;
}

extern "C" DL_API int dl_comm_import(const unsigned char *handle, void **ptr) {
    DL_REQUIRE(ptr && handle, DL_ERR_INVALID_ARG, "dl_comm_import: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(DL_ERR_CUDA, "dl_comm_import: %s", cudaGetErrorString(e));
    }
    return DL_OK;
}

extern "C" DL_API int dl_comm_close(void *ptr) {
    if (ptr != nullptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) return launch_status("dl_comm_close");
    return DL_OK;
}

// param_ptrs / grad_ptrs / flag_ptrs: HOST arrays of `world` device pointers, index = rank (own entry: own buffers).
extern "C" DL_API int dl_adam_exchange_step_f32(void *const *param_ptrs, void *const *grad_ptrs, void *const *flag_ptrs, int rank,
                                                int world, float *exp_avg, float *exp_avg_sq, int64_t n, float lr, float beta1,
                                                float beta2, float eps, int32_t *state, void *stream) {
    DL_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, DL_ERR_INVALID_ARG,
               "dl_adam_exchange_step_f32: rank %d of %d (at most %d ranks)", rank, world, kMaxRanks);
    DL_REQUIRE(n >= 0 && n % 4 == 0, DL_ERR_INVALID_ARG, "dl_adam_exchange_step_f32: n must be a multiple of 4");
    DL_REQUIRE(param_ptrs && grad_ptrs && flag_ptrs && state && exp_avg && exp_avg_sq, DL_ERR_INVALID_ARG,
               "dl_adam_exchange_step_f32: null pointer");
    ExchangePeers peers;
    for (int p = 0; p < world; ++p) {
        DL_REQUIRE(param_ptrs[p] && grad_ptrs[p] && flag_ptrs[p], DL_ERR_INVALID_ARG, "dl_adam_exchange_step_f32: null peer pointer");
        DL_REQUIRE(aligned_to(param_ptrs[p], 16) && aligned_to(grad_ptrs[p], 16), DL_ERR_INVALID_ARG,
                   "dl_adam_exchange_step_f32: buffers must be 16-byte aligned");
        peers.param[p] = reinterpret_cast<float *>(param_ptrs[p]);
        peers.grad[p] = reinterpret_cast<const float *>(grad_ptrs[p]);
        peers.flags[p] = reinterpret_cast<int *>(flag_ptrs[p]);
    }
    const int64_t n4 = n / 4;
    const int64_t per = ceil_div(n4, world);
    int64_t blocks = ceil_div(per > 0 ? per : 1, kThreads);
    if (blocks > 148 * 4) blocks = 148 * 4;  // all blocks resident: none of them waits for another one of this grid
    launch_dependent(true, adam_exchange_kernel, dim3((unsigned)blocks), dim3(kThreads), 0, as_stream(stream), peers, rank, world,
                     exp_avg, exp_avg_sq, n4, lr, beta1, beta2, eps, reinterpret_cast<int *>(state));
    return launch_status("dl_adam_exchange_step_f32");
}
