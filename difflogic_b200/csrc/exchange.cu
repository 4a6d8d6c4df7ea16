// Gradient exchange and optimizer step of batch-sharded training in ONE kernel, over peer memory.
//
// Every rank (one process per GPU) keeps the flat gradient buffer and the flat parameter buffer of the network in
// memory that its peers have mapped (CUDA IPC over NVLink).  After the backward pass each rank owns one slice of
// the parameters:
//   1. barrier A: every rank tells every peer that its gradients are complete (a flag store into the peer's
//      memory) and waits until all peers have said so;
//   2. for its slice it reads that slice of ALL ranks' gradients straight from their memory (16-byte loads over
//      NVLink), averages, applies Adam with its slice of the moments, and stores the new parameters into its OWN
//      parameter buffer;
//   3. barrier B: when a rank's slice is complete (a fence over local stores: cheap) it tells the peers; every block
//      waits until all ranks have said so;
//   4. it pulls the other ranks' slices of the new parameters from their memory into its own parameter buffer
//      (peer loads again).  The kernel ends with every rank holding the complete updated parameters.
// Pulling instead of pushing the new parameters matters: after stores INTO peer memory a rank has to wait for
// their system-wide visibility before it may raise its flag, and that fence measured 8 us of a 27 us kernel.
// This replaces an NCCL all-reduce of the gradients followed by a full Adam step on every rank: the bytes that
// cross NVLink are the same as a reduce-scatter plus all-gather, there is no extra launch, and each rank touches
// only 1/N of the optimizer state.
//
// The peers are other GPUs of this machine mapped by plain peer-to-peer access; the loads and stores are ordinary
// ld/st instructions.  Every wait is bounded (kExchangeSpinLimit polls); when one runs out the kernel records it
// in the state words and carries on, so a missing rank cannot hang the others.
#include <string.h>

#include "adam_math.cuh"
#include "common.cuh"
#include "tma.cuh"

namespace dl {

constexpr int kMaxRanks = 16;
constexpr unsigned kExchangeSpinLimit = 1u << 22;
constexpr int kGatherVecs = 512;  // float4 per piece of the gather phase: 8 KB

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

__device__ __forceinline__ int ld_relaxed_sys(const int *p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by ALL threads of a block: waits until every peer's flag for barrier `b` has reached `epoch`; false when a
// poll limit ran out.  Thread p polls peer p's flag with relaxed loads and reads it once more with acquire when it has seen it: a chain of
// `world` acquire loads per block, from hundreds of blocks on the same few words, cost tens of microseconds at
// eight ranks.  The block barrier passes the ordering on to the other threads.
__device__ __forceinline__ bool wait_peers(const int *my_flags, int world, int b, int epoch) {
    bool ok = true;
    if ((int)threadIdx.x < world) {
        unsigned spin = 0;
        while (ld_relaxed_sys(my_flags + 2 * threadIdx.x + b) < epoch) {
            if (++spin > kExchangeSpinLimit) {
                ok = false;
                break;
            }
        }
        (void)ld_acquire_sys(my_flags + 2 * threadIdx.x + b);  // one acquire once the flag is there (a system-scope
                                                               // fence here cost 10 us per barrier)
    }
    return __syncthreads_and(ok ? 1 : 0) != 0;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// state: [0] steps done, [1] ticket of blocks that finished their part of the slice, [2] error (a wait ran out),
// [3] ticket of blocks that finished pulling, [4..15] six 64-bit time stamps of the latest step in nanoseconds:
// entry, after barrier A (block 0), slice done (last block), after barrier B (block 0), block 0's elements stored, end
// WORLD = number of ranks when it is 2, 4 or 8 (all loads of an iteration are then issued before the first one is
// used: 8 peer loads of 16 bytes in flight per thread, i.e. 8 / WORLD elements per iteration), 0 = any number of ranks
// (one element per iteration, peers read one after the other).
template <int WORLD>
__global__ void __launch_bounds__(kThreads, 2)
adam_exchange_kernel(ExchangePeers peers, int rank, int world, float *__restrict__ m, float *__restrict__ v, int64_t n4_total,
                     float lr, float beta1, float beta2, float eps, int *__restrict__ state) {
    __shared__ float s_step_size, s_bc2_sqrt;
    __shared__ __align__(128) float4 s_gather[2][kGatherVecs];
    __shared__ __align__(8) uint64_t s_gather_bar[2];
    if (threadIdx.x == 0) {
        mbar_init(&s_gather_bar[0], 1);
        mbar_init(&s_gather_bar[1], 1);
        mbar_fence_init();
    }
    grid_dependency_wait();  // this rank's gradients come from the kernels just before
    unsigned long long *stamps = reinterpret_cast<unsigned long long *>(state + 4);
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[0] = global_timer_ns();
    const int epoch = state[0] + 1;
    // barrier A: announce (once per rank), then everybody waits on the local flag words
    if (blockIdx.x == 0 && threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + 2 * rank + 0, epoch);
    if (threadIdx.x == kThreads - 1) {  // a thread that polls no flag
        const float t = (float)epoch;
        s_step_size = lr / (1.f - powf(beta1, t));
        s_bc2_sqrt = sqrtf(1.f - powf(beta2, t));
    }
    const bool ok_a = wait_peers(peers.flags[rank], world, 0, epoch);  // ends with a block barrier
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[1] = global_timer_ns();
    if (!ok_a && threadIdx.x == 0) state[2] = 1;
    const float step_size = s_step_size, bc2_sqrt = s_bc2_sqrt;
    const float omb1 = 1.f - beta1, omb2 = 1.f - beta2, inv_world = 1.f / (float)world;

    // this rank's slice, in float4 units
    const int64_t per = (n4_total + world - 1) / world;
    const int64_t lo = min((int64_t)rank * per, n4_total), hi = min(lo + per, n4_total);
    float4 *m4 = reinterpret_cast<float4 *>(m), *v4 = reinterpret_cast<float4 *>(v);  // moments of the slice only
    float4 *own_param = reinterpret_cast<float4 *>(peers.param[rank]);

    const AdamConsts consts = {omb1, beta2, omb2, step_size, bc2_sqrt, eps};
    if (WORLD > 0) {
        constexpr int W = WORLD > 0 ? WORLD : 1;
        constexpr int U = 8 / W;  // elements per thread and iteration
        const int64_t stride = (int64_t)gridDim.x * kThreads;
        for (int64_t base = lo + (int64_t)blockIdx.x * kThreads + threadIdx.x; base < hi; base += stride * U) {
            float4 gp[U][W], pp_[U], mm_[U], vv_[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = base + u * stride;
                if (i < hi) {
#pragma unroll
                    for (int p = 0; p < W; ++p) gp[u][p] = ld_peer(reinterpret_cast<const float4 *>(peers.grad[p]) + i);
                    pp_[u] = own_param[i];
                    mm_[u] = m4[i - lo];
                    vv_[u] = v4[i - lo];
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = base + u * stride;
                if (i < hi) {
                    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int p = 0; p < W; ++p) {  // same order of additions as the generic loop
                        g.x += gp[u][p].x; g.y += gp[u][p].y; g.z += gp[u][p].z; g.w += gp[u][p].w;
                    }
                    float4 pp = pp_[u], mm = mm_[u], vv = vv_[u];
                    g.x = __fmul_rn(g.x, inv_world); g.y = __fmul_rn(g.y, inv_world);
                    g.z = __fmul_rn(g.z, inv_world); g.w = __fmul_rn(g.w, inv_world);
                    adam_update4(pp, g, mm, vv, consts);
                    m4[i - lo] = mm;
                    v4[i - lo] = vv;
                    own_param[i] = pp;
                }
            }
        }
    } else {
        for (int64_t i = lo + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < hi; i += (int64_t)gridDim.x * kThreads) {
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = 0; p < world; ++p) {
                const float4 gp = ld_peer(reinterpret_cast<const float4 *>(peers.grad[p]) + i);
                g.x += gp.x; g.y += gp.y; g.z += gp.z; g.w += gp.w;
            }
            float4 pp = own_param[i];
            float4 mm = m4[i - lo], vv = v4[i - lo];
            g.x = __fmul_rn(g.x, inv_world); g.y = __fmul_rn(g.y, inv_world);
            g.z = __fmul_rn(g.z, inv_world); g.w = __fmul_rn(g.w, inv_world);
            adam_update4(pp, g, mm, vv, consts);
            m4[i - lo] = mm;
            v4[i - lo] = vv;
            own_param[i] = pp;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[4] = global_timer_ns();  // first block: its elements are stored

    // barrier B: the last block of this rank to finish its part of the slice tells the peers; every block then waits
    // until all ranks' slices are complete.  (All blocks of the grid are resident together -- the host sizes the
    // grid for that -- so waiting for this grid's own last block cannot starve it.)
    // Every thread orders its stores at GPU scope (they are stores to this GPU's own memory: once they are visible
    // on this GPU, a peer's load over NVLink sees them too); only the one thread that raises the flag pays for a
    // system-scope fence.  A system-scope fence in every thread measured 8 us.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(state + 1, 1);
        if (done == (int)gridDim.x - 1) {
            __threadfence_system();
            stamps[2] = global_timer_ns();
            for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 2 * rank + 1, epoch);
        }
    }
    const bool ok_b = wait_peers(peers.flags[rank], world, 1, epoch);
    if (!ok_b && threadIdx.x == 0) state[2] = 1;
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[3] = global_timer_ns();

    // Pull the other ranks' slices: 8 KB pieces, each fetched by ONE bulk asynchronous copy (the 1-D TMA form, peer
    // memory -> this CTA's shared memory, no multicast) and written to this rank's parameter buffer with 16-byte stores.
    // Two pieces per block are in flight at a time; the copy engine needs no registers for its requests.  (With eight
    // ranks this phase measured the same 22 us for 4.5 MB as plain 16-byte peer loads, eight in flight per thread.)
    {
        const int64_t per_pieces = (per + kGatherVecs - 1) / kGatherVecs;  // pieces per source slice
        const int64_t npieces = (int64_t)(world - 1) * per_pieces;
        uint32_t fills[2] = {0u, 0u};  // how often each buffer has been filled: the parity of its barrier's phase
        bool ok = true;
        // the peers' slices were written with ordinary stores; order the asynchronous copies below behind the flags
        // that announced them
        if (threadIdx.x == 0) asm volatile("fence.proxy.async;" ::: "memory");
        for (int64_t c0 = blockIdx.x; c0 < npieces; c0 += 2 * (int64_t)gridDim.x) {
            int64_t start[2];
            int count[2], src_of[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int64_t c = c0 + (int64_t)i * gridDim.x;
                count[i] = 0;
                start[i] = 0;
                src_of[i] = 0;
                if (c < npieces) {
                    int src = (int)(c / per_pieces);
                    if (src >= rank) ++src;  // skip this rank's own slice
                    const int64_t first = (int64_t)src * per + (c % per_pieces) * kGatherVecs;
                    const int64_t end = min((int64_t)(src + 1) * per, n4_total);
                    if (first < end) {
                        start[i] = first;
                        count[i] = (int)min((int64_t)kGatherVecs, end - first);
                        src_of[i] = src;
                    }
                }
            }
            if (threadIdx.x == 0) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (count[i] > 0) {
                        mbar_arrive_expect_tx(&s_gather_bar[i], (uint32_t)count[i] * 16u);
                        bulk_load(s_gather[i], reinterpret_cast<const float4 *>(peers.param[src_of[i]]) + start[i],
                                  (uint32_t)count[i] * 16u, &s_gather_bar[i]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (count[i] > 0) {
                    if (ok && !mbar_wait(&s_gather_bar[i], fills[i] & 1u)) ok = false;  // bounded
                    ++fills[i];
                    if (ok)
                        for (int v = threadIdx.x; v < count[i]; v += kThreads) own_param[start[i] + v] = s_gather[i][v];
                }
            }
            __syncthreads();  // the pieces are consumed before their buffers are refilled
        }
        if (!ok && threadIdx.x == 0) state[2] = 1;
    }

    // the last block to finish everything resets the tickets and advances the step counter
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const int done = atomicAdd(state + 3, 1);
        if (done == (int)gridDim.x - 1) {
            stamps[5] = global_timer_ns();
            state[1] = 0;
            state[3] = 0;
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
    // One wave of blocks that are all resident together: every block waits at barrier B for this grid's own last
    // block, so a block that could not be scheduled would stall the others until their wait limit.  The limit is
    // what the occupancy calculator gives for the kernel that is launched, not a constant.
    const int per_thread = (world == 2 || world == 4 || world == 8) ? 8 / world : 1;
    int *st = reinterpret_cast<int *>(state);
    cudaStream_t cs = as_stream(stream);
    auto launch = [&](auto kernel) -> int {
        int dev = 0, sms = 0, per_sm = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || sms <= 0 || per_sm <= 0)
            return launch_status("dl_adam_exchange_step_f32 (occupancy query)");
        // enough blocks for one pass over the slice, and for the gather of the other ranks' slices (world - 1 times as
        // many elements, 8 per thread and pass: loads over NVLink need many requests in flight), never more than fit
        int64_t blocks = ceil_div(per > 0 ? per : 1, (int64_t)kThreads * per_thread);
        const int64_t for_gather = ceil_div((int64_t)(world - 1) * ceil_div(per, (int64_t)kGatherVecs), (int64_t)2);  // two pieces per block
        if (blocks < for_gather) blocks = for_gather;
        const int64_t resident = (int64_t)sms * per_sm;
        if (blocks > resident) blocks = resident;
        launch_dependent(true, kernel, dim3((unsigned)blocks), dim3(kThreads), 0, cs, peers, rank, world, exp_avg, exp_avg_sq, n4, lr,
                         beta1, beta2, eps, st);
        return DL_OK;
    };
    int rc;
    switch (world) {
        case 2: rc = launch(adam_exchange_kernel<2>); break;
        case 4: rc = launch(adam_exchange_kernel<4>); break;
        case 8: rc = launch(adam_exchange_kernel<8>); break;
        default: rc = launch(adam_exchange_kernel<0>); break;
    }
    if (rc != DL_OK) return rc;
    return launch_status("dl_adam_exchange_step_f32");
}
