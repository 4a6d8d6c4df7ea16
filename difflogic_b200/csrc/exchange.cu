// Gradient exchange and optimizer step of batch-sharded training over peer memory, one bucket at a time.
//
// Every rank (one process per GPU) keeps the flat gradient buffer and the flat parameter buffer of the network in
// memory that its peers have mapped (CUDA IPC over NVLink).  The buffers are cut into buckets (one per layer, say);
// the last block of the backward_w kernel that completes a bucket's gradients tells every peer so (a flag store into
// the peer's memory), and the rank launches ONE small kernel for the bucket, beside the backward pass of the layers
// below:
//   1. wait until all ranks have announced their gradients of the bucket;
//   2. read ITS slice of the bucket from all ranks' gradient buffers (16-byte loads over NVLink), average, apply
//      Adam with its slice of the moments and store the new parameters into its OWN parameter buffer; the last block
//      to finish tells the peers "my slice of this bucket is complete";
//   3. wait until all ranks have said that, and pull the other ranks' slices of the new parameters from their memory
//      into its own parameter buffer.
// The kernel waits only for OTHER GPUs (and, between its two phases, for the last block of its own small grid), never
// for a kernel launched later on its own GPU.  What crosses NVLink is what a reduce-scatter plus an all-gather moves.
// Only the bucket of the layer whose gradients come last is not hidden behind the backward pass.
// Pulling instead of pushing the new parameters matters: after stores INTO peer memory a rank has to wait for their
// system-wide visibility before it may raise its flag, and that fence measured 8 us.
// Small buckets go another way (exchange_packets_kernel, further down): everything is pushed, as 8-byte packets that
// carry their own flag, so that there is neither a fence nor a flag round trip; it moves twice the bytes.
//
// The peers are other GPUs of this machine mapped by plain peer-to-peer access; every access to their memory is an
// ordinary ld/st instruction (no bulk copy, no TMA, no multicast).  Every wait is bounded (wait_limit_us microseconds); a kernel
// whose wait runs out sets the error word of the bucket's state, changes NOTHING else (parameters, moments and step
// count stay as they were) and returns, so a missing rank cannot hang the others and cannot corrupt the weights.
#include <string.h>

#include "adam_math.cuh"
#include "common.cuh"

namespace dl {

constexpr int kMaxRanks = 16;
constexpr int kMaxBuckets = 32;
constexpr unsigned kExchangeWaitUs = 20u * 1000u * 1000u;  // default limit of a wait for the peers: 20 seconds
constexpr int kFlagBytes = kMaxBuckets * kMaxRanks * 2 * 4;

struct ExchangePeers {
    float *param[kMaxRanks];      // flat parameter buffer of each rank (index = rank; own entry is local memory)
    const float *grad[kMaxRanks]; // flat gradient buffer of each rank
    int *flags[kMaxRanks];        // flag words of each rank: word (bucket, p, which) is written by rank p
};

__device__ __forceinline__ int flag_index(int bucket, int peer, int which) { return (bucket * kMaxRanks + peer) * 2 + which; }

__device__ __forceinline__ int ld_acquire_sys(const int *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int *p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
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

// Called by ALL threads of a block: waits until every rank's flag (bucket, rank, which) in this rank's flag words has
// reached `epoch`; false when the wait took longer than `limit_us` microseconds (read off %globaltimer every 32
// polls).  Thread p polls rank p's flag with relaxed loads and reads it once more with acquire when it has seen it;
// the block barrier passes the ordering on to the other threads.
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool wait_peers(const int *my_flags, int world, int bucket, int which, int epoch, unsigned limit_us) {
    bool ok = true;
    if ((int)threadIdx.x < world) {
        const int *f = my_flags + flag_index(bucket, threadIdx.x, which);
        unsigned spin = 0;
        unsigned long long t0 = 0;
        while (ld_relaxed_sys(f) < epoch) {
            if ((++spin & 31u) == 0u) {
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > (unsigned long long)limit_us * 1000ull) {
                    ok = false;
                    break;
                }
            }
        }
        (void)ld_acquire_sys(f);
    }
    return __syncthreads_and(ok ? 1 : 0) != 0;
}

// state of a bucket, 16 ints: [0] steps done, [1] ticket of the slice phase, [2] error (a wait ran out), [3] ticket
// of the gather phase, [4..15] six 64-bit time stamps of the latest step in nanoseconds: kernel entered (after the
// grid dependency), all ranks' gradients seen (block 0), slice complete (last block), [unused], all ranks' slices
// seen (block 0), done (last block).
//
// One kernel per bucket and step, in one of two forms.
//   Two passes (whole_bucket == 0): wait for all ranks' gradients -> reduce + Adam on this rank's slice -> tell the
//   peers -> wait for all ranks' slices -> pull them.  Blocks wait for the LAST block of their own grid between the two
//   phases; the grid is small (at most 64 blocks), and the only kernels that can hold it up are backward kernels,
//   which wait for nothing.  NVLink carries 2 (N-1)/N of the bucket per rank.
//   One pass (whole_bucket == 1): wait for all ranks' gradients -> every rank reduces the WHOLE bucket and applies Adam
//   to all of it (the same additions in the same order on every rank: bit-identical replicas) -> the last block waits
//   until every rank has finished reading.  NVLink carries (N-1) times the bucket per rank, but there is one flag
//   round trip less and no second pass: the form for a small bucket that nothing else can hide (the one whose
//   gradients come last in the backward pass).  A bucket must keep its form from step to step (one-pass buckets keep
//   full moments on every rank, two-pass buckets only their slices).
//
// WORLD = number of ranks when it is 2, 4 or 8 (all loads of an iteration are then issued before the first one is
// used: 8 peer loads of 16 bytes in flight per thread, i.e. 8 / WORLD elements per iteration), 0 = any number of ranks
// (one element per iteration, peers read one after the other).  The sum over the ranks is formed in rank order in
// every variant, so all of them give the same bits.
template <int WORLD>
__global__ void __launch_bounds__(kThreads)
exchange_bucket_kernel(ExchangePeers peers, int rank, int world, float *__restrict__ m, float *__restrict__ v, int64_t off4,
                       int64_t n4, int bucket, float lr, float beta1, float beta2, float eps, int *__restrict__ state,
                       int announce_here, int whole_bucket, unsigned wait_us) {
    __shared__ float s_step_size, s_bc2_sqrt;
    unsigned long long *stamps = reinterpret_cast<unsigned long long *>(state + 4);
    // the step count of this bucket was last written by this kernel one step ago: safe before the dependency wait
    const int epoch = state[0] + 1;
    if (threadIdx.x == kThreads - 1) {  // a thread that polls no flag
        const float t = (float)epoch;
        s_step_size = lr / (1.f - powf(beta1, t));
        s_bc2_sqrt = sqrtf(1.f - powf(beta2, t));
    }
    grid_dependency_wait();  // this rank's gradients come from the kernel just before (when launched right behind it)
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[0] = global_timer_ns();
    // announce, unless the kernel that wrote the gradients has done it (dl_backward_w_announce_f32): this rank's
    // gradients of the bucket were written by kernels that completed before this point; the release store (system scope)
    // orders them before the flag for observers on other GPUs.  (A separate system-scope fence in front of it was
    // redundant and cost microseconds on the only path nothing hides.)
    if (announce_here && blockIdx.x == 0 && (int)threadIdx.x < world)
        st_release_sys(peers.flags[threadIdx.x] + flag_index(bucket, rank, 0), epoch);
    const bool ok_a = wait_peers(peers.flags[rank], world, bucket, 0, epoch, wait_us);  // ends with a block barrier
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[1] = global_timer_ns();

    const int64_t per = (n4 + world - 1) / world;  // float4 per slice
    float4 *own_param = reinterpret_cast<float4 *>(peers.param[rank]);
    if (ok_a) {
        const AdamConsts consts = {1.f - beta1, beta2, 1.f - beta2, s_step_size, s_bc2_sqrt, eps};
        const float inv_world = 1.f / (float)world;
        // this rank's slice of the bucket (the whole bucket in the one-pass form), in float4 units of the flat buffers
        const int64_t lo = whole_bucket ? off4 : off4 + min((int64_t)rank * per, n4);
        const int64_t hi = whole_bucket ? off4 + n4 : min(lo + per, off4 + n4);
        float4 *m4 = reinterpret_cast<float4 *>(m), *v4 = reinterpret_cast<float4 *>(v);
        constexpr int W = WORLD > 0 ? WORLD : 1;
        constexpr int U = WORLD > 0 ? 8 / W : 1;  // elements per thread and iteration
        const int64_t stride = (int64_t)gridDim.x * kThreads;
        for (int64_t base = lo + (int64_t)blockIdx.x * kThreads + threadIdx.x; base < hi; base += stride * U) {
            float4 gp[U][W], g[U], pp[U], mm[U], vv[U];
            // every load of the iteration is issued before the first one is used
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = base + u * stride;
                g[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < hi) {
                    if (WORLD > 0) {
#pragma unroll
                        for (int p = 0; p < W; ++p) gp[u][p] = ld_peer(reinterpret_cast<const float4 *>(peers.grad[p]) + i);
                    } else {
                        for (int p = 0; p < world; ++p) {
                            const float4 one = ld_peer(reinterpret_cast<const float4 *>(peers.grad[p]) + i);
                            g[u].x += one.x; g[u].y += one.y; g[u].z += one.z; g[u].w += one.w;
                        }
                    }
                    pp[u] = own_param[i];
                    mm[u] = m4[i];
                    vv[u] = v4[i];
                }
            }
            if (WORLD > 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (base + u * stride < hi) {
#pragma unroll
                        for (int p = 0; p < W; ++p) {  // rank order, as in the generic loop
                            g[u].x += gp[u][p].x; g[u].y += gp[u][p].y; g[u].z += gp[u][p].z; g[u].w += gp[u][p].w;
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = base + u * stride;
                if (i < hi) {
                    g[u].x = __fmul_rn(g[u].x, inv_world); g[u].y = __fmul_rn(g[u].y, inv_world);
                    g[u].z = __fmul_rn(g[u].z, inv_world); g[u].w = __fmul_rn(g[u].w, inv_world);
                    adam_update4(pp[u], g[u], mm[u], vv[u], consts);
                    m4[i] = mm[u];
                    v4[i] = vv[u];
                    own_param[i] = pp[u];
                }
            }
        }
    }

    // The last block of this rank to finish its part of the slice tells the peers -- unless a wait ran out in any block
    // of this launch: then the flag stays down and the gather phase runs out everywhere, instead of fetching a slice
    // that is only partly updated.  The block barrier orders every thread's stores before thread 0's fence (they are
    // stores to this GPU's own memory: once they are visible on this GPU, a peer's load over NVLink sees them too);
    // only the one thread that raises the flags pays for a system-scope fence.
    __shared__ int s_last_and_sound;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!ok_a) atomicExch(state + 2, 1);
        __threadfence();
        const int add = ok_a ? 1 : 0x10001;  // low half: blocks that are through; high half: those whose wait ran out
        const int all = atomicAdd(state + 1, add) + add;
        s_last_and_sound = 0;
        if ((all & 0xffff) == (int)gridDim.x) {
            state[1] = 0;
            if ((all >> 16) == 0) {
                // the ticket (atomic + GPU-scope fences) has ordered every block's stores before this thread; its release
                // stores at system scope pass that on to the peers
                stamps[2] = global_timer_ns();
                for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + flag_index(bucket, rank, 1), epoch);
                s_last_and_sound = 1;
            }
        }
    }

    if (whole_bucket) {
        // One-pass form: every rank has averaged and updated the WHOLE bucket, so there is nothing to fetch.  The flag
        // just raised says "this rank has finished reading the others' gradients"; the kernel must not end before all
        // ranks have said so, because the next step's backward_w overwrites the gradients.  Only the block that
        // finished last waits (the ranks work in lockstep after the first wait, so this is one flag latency).
        __syncthreads();
        if (!s_last_and_sound) return;
        const bool ok_d = wait_peers(peers.flags[rank], world, bucket, 1, epoch, wait_us);
        if (threadIdx.x == 0) {
            const unsigned long long now = global_timer_ns();
            stamps[4] = now;
            stamps[5] = now;
            if (ok_d)
                state[0] = epoch;
            else
                atomicExch(state + 2, 1);
        }
        return;
    }

    // gather: wait until every rank's slice is complete (this rank's own flag included: it comes from this grid's last
    // block), then pull the other ranks' slices, 8 peer loads of 16 bytes in flight per thread.  After a wait that
    // ran out in the first phase there is nothing to wait for (this rank will never raise its flag).
    const bool ok_b = ok_a && wait_peers(peers.flags[rank], world, bucket, 1, epoch, wait_us);
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[4] = global_timer_ns();
    if (ok_b && world > 1) {
        constexpr int UG = 8;
        const int64_t total = (int64_t)(world - 1) * per;  // positions in the other ranks' slices (the tail may be short)
        const int64_t end4 = off4 + n4;
        const int64_t stride = (int64_t)gridDim.x * kThreads;
        for (int64_t base = (int64_t)blockIdx.x * kThreads + threadIdx.x; base < total; base += stride * UG) {
            float4 val[UG];
            int64_t at[UG];
#pragma unroll
            for (int u = 0; u < UG; ++u) {
                const int64_t idx = base + u * stride;
                at[u] = -1;
                if (idx < total) {
                    int src = (int)(idx / per);
                    const int64_t within = idx - (int64_t)src * per;
                    if (src >= rank) ++src;  // skip this rank's own slice
                    const int64_t i = off4 + (int64_t)src * per + within;
                    if (i < end4) {
                        at[u] = i;
                        val[u] = ld_peer(reinterpret_cast<const float4 *>(peers.param[src]) + i);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UG; ++u)
                if (at[u] >= 0) own_param[at[u]] = val[u];
        }
    }
    // the last block to finish advances the bucket's step count -- only when no block's wait ran out
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!ok_b) atomicExch(state + 2, 1);
        __threadfence();
        const int add = ok_b ? 1 : 0x10001;
        const int all = atomicAdd(state + 3, add) + add;
        if ((all & 0xffff) == (int)gridDim.x) {
            state[3] = 0;
            if ((all >> 16) == 0) {
                stamps[5] = global_timer_ns();
                state[0] = epoch;
            }
        }
    }
}

// Announces this rank's gradients of a bucket when no backward_w kernel did it (dl_backward_w_announce_f32 does it from
// its last block): one thread per rank stores the bucket's next epoch into that rank's flag words.
__global__ void exchange_announce_kernel(ExchangePeers peers, int rank, int world, int bucket, const int *__restrict__ state) {
    if ((int)threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + flag_index(bucket, rank, 0), state[0] + 1);
}

// ---- the exchange with the flags inside the data ("packets") ------------------------------------------------------------
// For small buckets the flag round trips of the kernel above cost more than the data: a flag store, the peer loads it
// allows (a round trip over NVLink), another flag, more peer loads.  Here nothing is pulled and no flag is raised.  Every
// float travels as an 8-byte packet {value, epoch} written with ONE store into the receiver's memory; 8-byte stores
// arrive whole, so a receiver that reads a packet with this step's epoch has its value, and every packet announces
// itself.  No fences, no tickets between the phases, no block waits for another block of its grid:
//   1. push: each float4 of this rank's gradients outside its own slice goes, as 4 packets, into the OWNER's inbox;
//   2. reduce: for its own slice the rank adds up -- in rank order, as the kernels above do -- its own gradients and the
//      packets of the other ranks as they arrive, applies Adam, stores the new parameters and pushes them, as packets,
//      into every peer's parameter inbox;
//   3. collect: the other slices' new parameters are taken out of the inbox as they arrive.
// One-way latencies only: push -> reduce -> push -> collect.  NVLink carries 4 (N-1)/N times the bucket per rank (the
// packets double the bytes), which is why this is the form for SMALL buckets.  An inbox holds, per bucket, one region
// per sending rank of `per` = ceil(n4 / world) float4 slots (32 bytes each, in two planes of 16).  It may be overwritten by the sender's next
// step because the sender gets there only after it has collected this step's parameters from this rank, which this
// rank sends after it has read the sender's gradient packets; and the parameter packets of the next step are sent only
// after the receiver's gradient packets of the next step have arrived, which it sends after it has collected this
// step's.  A packet that does not arrive within the limit sets the bucket's error word; unlike the kernels above this
// form may then have updated part of the bucket.  The grid is small enough to be resident as a whole (blocks in phase 2
// wait for OTHER ranks' phase 1, which waits for nothing).
struct PacketPeers {
    unsigned long long *grad_inbox[kMaxRanks];   // of each rank (index = rank); own entry: this rank's inbox
    unsigned long long *param_inbox[kMaxRanks];
};

// A float4 slot is two 16-byte halves, {x, y} and {z, w} as two packets each, in two PLANES of the inbox `half` u64
// apart, so that the 32 lanes of a warp write (and read) 512 contiguous bytes per instruction.
__device__ __forceinline__ void st_packets(unsigned long long *dst, int64_t half, const float4 &v, unsigned epoch) {
    const unsigned long long e = (unsigned long long)epoch << 32;
    const unsigned long long p0 = e | __float_as_uint(v.x), p1 = e | __float_as_uint(v.y);
    const unsigned long long p2 = e | __float_as_uint(v.z), p3 = e | __float_as_uint(v.w);
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(p0), "l"(p1) : "memory");
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst + half), "l"(p2), "l"(p3) : "memory");
}

struct Packets4 {
    unsigned long long p[4];
    __device__ __forceinline__ void load(const unsigned long long *src, int64_t half) {
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(p[0]), "=l"(p[1]) : "l"(src) : "memory");
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(p[2]), "=l"(p[3]) : "l"(src + half) : "memory");
    }
    __device__ __forceinline__ bool complete(unsigned epoch) const {
        return (unsigned)(p[0] >> 32) == epoch && (unsigned)(p[1] >> 32) == epoch && (unsigned)(p[2] >> 32) == epoch &&
               (unsigned)(p[3] >> 32) == epoch;
    }
    __device__ __forceinline__ float4 value() const {
        return make_float4(__uint_as_float((unsigned)p[0]), __uint_as_float((unsigned)p[1]), __uint_as_float((unsigned)p[2]),
                           __uint_as_float((unsigned)p[3]));
    }
};

// polls one slot until its four packets carry `epoch`; false when that took longer than limit_us (t0: the thread's first
// look at the clock, shared by its waits of this launch)
__device__ __forceinline__ bool wait_packets(Packets4 &pk, const unsigned long long *src, int64_t half, unsigned epoch,
                                             unsigned limit_us, unsigned long long &t0) {
    unsigned spin = 0;
    for (;;) {
        pk.load(src, half);
        if (pk.complete(epoch)) return true;
        if ((++spin & 63u) == 0u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > (unsigned long long)limit_us * 1000ull) return false;
        }
    }
}

// inbox_off: first float4 slot of this bucket inside a sender's region; inbox_stride: float4 slots per sender's region
// (the sum of `per` over all buckets).  WORLD as in exchange_bucket_kernel.
template <int WORLD>
__global__ void __launch_bounds__(kThreads)
exchange_packets_kernel(PacketPeers peers, int rank, int world, float *__restrict__ param, const float *__restrict__ grad,
                        float *__restrict__ m, float *__restrict__ v, int64_t off4, int64_t n4, int64_t inbox_off,
                        int64_t inbox_stride, float lr, float beta1, float beta2, float eps, int *__restrict__ state,
                        int pushed, unsigned wait_us) {
    __shared__ float s_step_size, s_bc2_sqrt;
    unsigned long long *stamps = reinterpret_cast<unsigned long long *>(state + 4);
    const int epoch_i = state[0] + 1;  // last written by this kernel one step ago: safe before the dependency wait
    const unsigned epoch = (unsigned)epoch_i;
    if (threadIdx.x == 0) {
        const float t = (float)epoch_i;
        s_step_size = lr / (1.f - powf(beta1, t));
        s_bc2_sqrt = sqrtf(1.f - powf(beta2, t));
    }
    grid_dependency_wait();  // this rank's gradients come from the kernel just before (when launched right behind it)
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[0] = global_timer_ns();

    const int64_t per = (n4 + world - 1) / world;  // float4 per slice
    const int64_t my_lo = min((int64_t)rank * per, n4), my_hi = min(my_lo + per, n4);  // this rank's slice within the bucket
    const int64_t stride = (int64_t)gridDim.x * kThreads, first = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const float4 *g4 = reinterpret_cast<const float4 *>(grad) + off4;
    float4 *p4 = reinterpret_cast<float4 *>(param) + off4;
    float4 *m4 = reinterpret_cast<float4 *>(m) + off4, *v4 = reinterpret_cast<float4 *>(v) + off4;
    unsigned long long t0 = 0;
    bool ok = true;
    const int64_t half = (int64_t)world * inbox_stride * 2;  // u64 between the two planes of an inbox
    // first u64 of float4 slot k of this bucket in the region of rank `from`
#define DL_SLOT(from, k) (((int64_t)(from) * inbox_stride + inbox_off + (k)) * 2)

    // 1. push the gradients of the other ranks' slices into their owners' inboxes (this rank's region there) -- unless
    // the backward_w kernels that wrote them have done so (dl_backward_w_push_f32)
    const int64_t others = n4 - (my_hi - my_lo);
    for (int64_t idx = first; idx < (pushed ? 0 : others); idx += stride) {
        const int64_t i = idx < my_lo ? idx : idx + (my_hi - my_lo);  // position within the bucket, own slice skipped
        const int owner = (int)(i / per);
        const int64_t k = i - (int64_t)owner * per;
        st_packets(peers.grad_inbox[owner] + DL_SLOT(rank, k), half, g4[i], epoch);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[1] = global_timer_ns();

    // 2. own slice: sum in rank order, Adam, new parameters to every peer
    const AdamConsts consts = {1.f - beta1, beta2, 1.f - beta2, s_step_size, s_bc2_sqrt, eps};
    const float inv_world = 1.f / (float)world;
    const unsigned long long *my_gin = peers.grad_inbox[rank];
    for (int64_t k = first; k < my_hi - my_lo; k += stride) {
        const int64_t i = my_lo + k;
        const float4 own = g4[i];
        float4 pp = p4[i], mm = m4[i], vv = v4[i];
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        if (WORLD > 0) {
            // all peers' slots are read at once, then those that have not arrived yet are polled
            Packets4 pk[WORLD > 0 ? WORLD : 1];
#pragma unroll
            for (int p = 0; p < WORLD; ++p)
                if (p != rank) pk[p].load(my_gin + DL_SLOT(p, k), half);
#pragma unroll
            for (int p = 0; p < WORLD; ++p) {
                float4 one = own;
                if (p != rank) {
                    if (!pk[p].complete(epoch)) ok = wait_packets(pk[p], my_gin + DL_SLOT(p, k), half, epoch, wait_us, t0) && ok;
                    one = pk[p].value();
                }
                g.x += one.x; g.y += one.y; g.z += one.z; g.w += one.w;
            }
        } else {
            for (int p = 0; p < world; ++p) {
                float4 one = own;
                if (p != rank) {
                    Packets4 pk;
                    ok = wait_packets(pk, my_gin + DL_SLOT(p, k), half, epoch, wait_us, t0) && ok;
                    one = pk.value();
                }
                g.x += one.x; g.y += one.y; g.z += one.z; g.w += one.w;
            }
        }
        if (!ok) break;  // a packet is missing: this element and the thread's later ones stay as they are
        g.x = __fmul_rn(g.x, inv_world); g.y = __fmul_rn(g.y, inv_world);
        g.z = __fmul_rn(g.z, inv_world); g.w = __fmul_rn(g.w, inv_world);
        adam_update4(pp, g, mm, vv, consts);
        m4[i] = mm;
        v4[i] = vv;
        p4[i] = pp;
        for (int p = 0; p < world; ++p)
            if (p != rank) st_packets(peers.param_inbox[p] + DL_SLOT(rank, k), half, pp, epoch);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[2] = global_timer_ns();

    // 3. the other slices' new parameters, as they arrive
    const unsigned long long *my_pin = peers.param_inbox[rank];
    if (ok) {
        for (int64_t idx = first; idx < others; idx += stride) {
            const int64_t i = idx < my_lo ? idx : idx + (my_hi - my_lo);
            const int owner = (int)(i / per);
            const int64_t k = i - (int64_t)owner * per;
            Packets4 pk;
            if (!wait_packets(pk, my_pin + DL_SLOT(owner, k), half, epoch, wait_us, t0)) {
                ok = false;
                break;
            }
            p4[i] = pk.value();
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) stamps[4] = global_timer_ns();

    // the last block to finish advances the bucket's step count -- only when no packet was missed anywhere
    const bool block_ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (threadIdx.x == 0) {
        if (!block_ok) atomicExch(state + 2, 1);
        __threadfence();
        const int add = block_ok ? 1 : 0x10001;
        const int all = atomicAdd(state + 3, add) + add;
        if ((all & 0xffff) == (int)gridDim.x) {
            state[3] = 0;
            if ((all >> 16) == 0) {
                stamps[5] = global_timer_ns();
                state[0] = epoch_i;
            }
        }
    }
#undef DL_SLOT
}

// All ranks meet on the device: this rank stores the barrier's next epoch into its word (bucket, rank, 0) of every rank's
// flags and waits until all ranks' words in its own flags have reached it.  state: sixteen ints like a bucket's, of
// which [0] counts the barriers passed and [2] is set when the wait ran out (the count then stays).  Like the exchange
// kernels it waits only for OTHER GPUs.
__global__ void rank_barrier_kernel(ExchangePeers peers, int rank, int world, int bucket, int *__restrict__ state, unsigned wait_us) {
    const int epoch = state[0] + 1;
    if ((int)threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + flag_index(bucket, rank, 0), epoch);
    const bool ok = wait_peers(peers.flags[rank], world, bucket, 0, epoch, wait_us);
    if (threadIdx.x == 0) {
        if (ok)
            state[0] = epoch;
        else
            atomicExch(state + 2, 1);
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

extern "C" DL_API size_t dl_exchange_flag_bytes(void) { return (size_t)kFlagBytes; }

static int exchange_peers(const char *who, ExchangePeers &peers, void *const *param_ptrs, void *const *grad_ptrs, void *const *flag_ptrs,
                          int rank, int world, int64_t offset, int64_t count, int bucket, const int32_t *state) {
    DL_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, DL_ERR_INVALID_ARG, "%s: rank %d of %d (at most %d ranks)",
               who, rank, world, kMaxRanks);
    DL_REQUIRE(bucket >= 0 && bucket < kMaxBuckets, DL_ERR_INVALID_ARG, "%s: bucket %d outside 0 .. %d", who, bucket, kMaxBuckets - 1);
    DL_REQUIRE(offset >= 0 && count >= 0 && offset % 4 == 0 && count % 4 == 0, DL_ERR_INVALID_ARG,
               "%s: offset and count must be non-negative multiples of 4", who);
    DL_REQUIRE(param_ptrs && flag_ptrs && state, DL_ERR_INVALID_ARG, "%s: null pointer", who);
    for (int p = 0; p < world; ++p) {
        DL_REQUIRE(param_ptrs[p] && flag_ptrs[p] && (grad_ptrs == nullptr || grad_ptrs[p]), DL_ERR_INVALID_ARG, "%s: null peer pointer", who);
        DL_REQUIRE(aligned_to(param_ptrs[p], 16) && (grad_ptrs == nullptr || aligned_to(grad_ptrs[p], 16)), DL_ERR_INVALID_ARG,
                   "%s: buffers must be 16-byte aligned", who);
        peers.param[p] = reinterpret_cast<float *>(param_ptrs[p]);
        peers.grad[p] = grad_ptrs ? reinterpret_cast<const float *>(grad_ptrs[p]) : nullptr;
        peers.flags[p] = reinterpret_cast<int *>(flag_ptrs[p]);
    }
    return DL_OK;
}

// param_ptrs / grad_ptrs / flag_ptrs: HOST arrays of `world` device pointers, index = rank (own entry: own buffers).
extern "C" DL_API int dl_exchange_bucket_f32(void *const *param_ptrs, void *const *grad_ptrs, void *const *flag_ptrs, int rank, int world,
                                             float *exp_avg, float *exp_avg_sq, int64_t offset, int64_t count, int bucket, float lr,
                                             float beta1, float beta2, float eps, int32_t *state, int announce_here,
                                             int whole_bucket, uint32_t wait_limit_us, int flags, void *stream) {
    ExchangePeers peers;
    DL_REQUIRE(grad_ptrs != nullptr, DL_ERR_INVALID_ARG, "dl_exchange_bucket_f32: null pointer");
    if (int s = exchange_peers("dl_exchange_bucket_f32", peers, param_ptrs, grad_ptrs, flag_ptrs, rank, world, offset, count, bucket, state))
        return s;
    DL_REQUIRE(exp_avg && exp_avg_sq && aligned_to(exp_avg, 16) && aligned_to(exp_avg_sq, 16), DL_ERR_INVALID_ARG,
               "dl_exchange_bucket_f32: moments must be non-null and 16-byte aligned");
    const int64_t n4 = count / 4, per = whole_bucket ? n4 : ceil_div(n4, world);
    const int per_thread = (world == 2 || world == 4 || world == 8) ? 8 / world : 1;
    // enough blocks for one pass over the slice and for one pass of the gather (8 elements per thread; grids of 2 and 4 times
    // as many blocks with fewer elements per thread made the step of 2 ranks 10 and 30 us slower: the blocks compete with
    // the backward kernels); two passes: never
    // more than 64, the blocks wait for their grid's last block between the phases and a small grid is resident as a
    // whole; one pass: no block waits for another, up to two blocks per SM
    int64_t blocks = ceil_div(per > 0 ? per : 1, (int64_t)kThreads * per_thread);
    const int64_t for_gather = whole_bucket ? 0 : ceil_div((int64_t)(world - 1) * per, (int64_t)kThreads * 8);
    if (blocks < for_gather) blocks = for_gather;
    const int64_t most = whole_bucket ? 2 * 148 : 64;
    if (blocks > most) blocks = most;
    const unsigned limit = wait_limit_us ? wait_limit_us : kExchangeWaitUs;
    int *st = reinterpret_cast<int *>(state);
    cudaStream_t cs = as_stream(stream);
    const bool overlap = (flags & DL_LAUNCH_OVERLAP_SETUP) != 0;
#define DL_EXCHANGE_BUCKET(WW)                                                                                                          \
    launch_dependent(overlap, exchange_bucket_kernel<WW>, dim3((unsigned)blocks), dim3(kThreads), 0, cs, peers, rank, world, exp_avg,   \
                     exp_avg_sq, offset / 4, n4, bucket, lr, beta1, beta2, eps, st, announce_here, whole_bucket ? 1 : 0, limit)
    switch (world) {
        case 2: DL_EXCHANGE_BUCKET(2); break;
        case 4: DL_EXCHANGE_BUCKET(4); break;
        case 8: DL_EXCHANGE_BUCKET(8); break;
        default: DL_EXCHANGE_BUCKET(0); break;
    }
#undef DL_EXCHANGE_BUCKET
    return launch_status("dl_exchange_bucket_f32");
}

// The exchange of one bucket with the flags inside the data (exchange_packets_kernel).  param, grad, exp_avg, exp_avg_sq:
// THIS rank's flat buffers (ordinary device memory will do); grad_inbox_ptrs / param_inbox_ptrs: host arrays of `world`
// device pointers, index = rank, to every rank's two inboxes (each 32 * world * inbox_stride bytes, zero at first).
// offset, count: the bucket in floats; inbox_offset: its first float4 slot inside a sender's region of inbox_stride slots.
// pushed: the gradients of the other ranks' slices have been pushed already, by dl_backward_w_push_f32.
extern "C" DL_API int dl_exchange_packets_f32(float *param, const float *grad, void *const *grad_inbox_ptrs,
                                              void *const *param_inbox_ptrs, int rank, int world, float *exp_avg, float *exp_avg_sq,
                                              int64_t offset, int64_t count, int64_t inbox_offset, int64_t inbox_stride, float lr,
                                              float beta1, float beta2, float eps, int32_t *state, int pushed, uint32_t wait_limit_us,
                                              int flags, void *stream) {
    const char *who = "dl_exchange_packets_f32";
    DL_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, DL_ERR_INVALID_ARG, "%s: rank %d of %d (at most %d ranks)",
               who, rank, world, kMaxRanks);
    DL_REQUIRE(offset >= 0 && count >= 0 && offset % 4 == 0 && count % 4 == 0, DL_ERR_INVALID_ARG,
               "%s: offset and count must be non-negative multiples of 4", who);
    DL_REQUIRE(param && grad && exp_avg && exp_avg_sq && state && grad_inbox_ptrs && param_inbox_ptrs, DL_ERR_INVALID_ARG,
               "%s: null pointer", who);
    DL_REQUIRE(aligned_to(param, 16) && aligned_to(grad, 16) && aligned_to(exp_avg, 16) && aligned_to(exp_avg_sq, 16), DL_ERR_INVALID_ARG,
               "%s: buffers must be 16-byte aligned", who);
    const int64_t n4 = count / 4, per = ceil_div(n4, (int64_t)world);
    DL_REQUIRE(inbox_offset >= 0 && inbox_stride > 0 && inbox_offset + per <= inbox_stride, DL_ERR_INVALID_ARG,
               "%s: slots %lld + %lld outside a region of %lld", who, (long long)inbox_offset, (long long)per, (long long)inbox_stride);
    PacketPeers peers;
    for (int p = 0; p < world; ++p) {
        DL_REQUIRE(grad_inbox_ptrs[p] && param_inbox_ptrs[p] && aligned_to(grad_inbox_ptrs[p], 16) && aligned_to(param_inbox_ptrs[p], 16),
                   DL_ERR_INVALID_ARG, "%s: null or misaligned inbox pointer", who);
        peers.grad_inbox[p] = reinterpret_cast<unsigned long long *>(grad_inbox_ptrs[p]);
        peers.param_inbox[p] = reinterpret_cast<unsigned long long *>(param_inbox_ptrs[p]);
    }
    // one float4 per thread and phase where that fits; never more than 64 blocks: blocks wait for other ranks' blocks, so
    // the grid must be resident as a whole (and 64 measured best for a 1 MB bucket with 2 ranks: 16, 32, 128 and 256 blocks
    // made the step 7, 4, 3 and 2 us longer)
    int64_t blocks = ceil_div(n4 > 0 ? n4 : 1, (int64_t)kThreads);
    if (blocks > 64) blocks = 64;
    const unsigned limit = wait_limit_us ? wait_limit_us : kExchangeWaitUs;
    int *st = reinterpret_cast<int *>(state);
    cudaStream_t cs = as_stream(stream);
    const bool overlap = (flags & DL_LAUNCH_OVERLAP_SETUP) != 0;
#define DL_EXCHANGE_PACKETS(WW)                                                                                                       \
    launch_dependent(overlap, exchange_packets_kernel<WW>, dim3((unsigned)blocks), dim3(kThreads), 0, cs, peers, rank, world, param,  \
                     grad, exp_avg, exp_avg_sq, offset / 4, n4, inbox_offset, inbox_stride, lr, beta1, beta2, eps, st, pushed ? 1 : 0,   \
                     limit)
    switch (world) {
        case 2: DL_EXCHANGE_PACKETS(2); break;
        case 4: DL_EXCHANGE_PACKETS(4); break;
        case 8: DL_EXCHANGE_PACKETS(8); break;
        default: DL_EXCHANGE_PACKETS(0); break;
    }
#undef DL_EXCHANGE_PACKETS
    return launch_status(who);
}

extern "C" DL_API int dl_exchange_announce(void *const *flag_ptrs, int rank, int world, int bucket, const int32_t *state, void *stream) {
    ExchangePeers peers;
    DL_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world && bucket >= 0 && bucket < kMaxBuckets && flag_ptrs && state,
               DL_ERR_INVALID_ARG, "dl_exchange_announce: bad argument");
    for (int p = 0; p < world; ++p) {
        DL_REQUIRE(flag_ptrs[p], DL_ERR_INVALID_ARG, "dl_exchange_announce: null peer pointer");
        peers.flags[p] = reinterpret_cast<int *>(flag_ptrs[p]);
    }
    exchange_announce_kernel<<<1, 32, 0, as_stream(stream)>>>(peers, rank, world, bucket, reinterpret_cast<const int *>(state));
    return launch_status("dl_exchange_announce");
}

// A barrier of the ranks on the device, on flag words of a bucket number that no exchange uses (see rank_barrier_kernel).
extern "C" DL_API int dl_rank_barrier(void *const *flag_ptrs, int rank, int world, int bucket, int32_t *state, uint32_t wait_limit_us,
                                      void *stream) {
    ExchangePeers peers;
    DL_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world && bucket >= 0 && bucket < kMaxBuckets && flag_ptrs && state,
               DL_ERR_INVALID_ARG, "dl_rank_barrier: bad argument");
    for (int p = 0; p < world; ++p) {
        DL_REQUIRE(flag_ptrs[p], DL_ERR_INVALID_ARG, "dl_rank_barrier: null peer pointer");
        peers.flags[p] = reinterpret_cast<int *>(flag_ptrs[p]);
    }
    rank_barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(peers, rank, world, bucket, reinterpret_cast<int *>(state),
                                                       wait_limit_us ? wait_limit_us : kExchangeWaitUs);
    return launch_status("dl_rank_barrier");
}

// Word of a rank's flag array that rank `rank` raises for (bucket, which): for callers that announce from kernels of
// their own (dl_backward_w_announce_f32 computes it itself).
extern "C" DL_API int dl_exchange_flag_word(int bucket, int rank, int which) { return (bucket * kMaxRanks + rank) * 2 + which; }
