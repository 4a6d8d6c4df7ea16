// Last logic layer and group bit-sum in one kernel: the layer's output is counted as it is computed and is never
// written to memory.
//
// Unfused, the last layer writes n_out rows and the group bit-sum reads them back: two passes over the largest
// array of the network.  Here a thread-block CLUSTER of S CTAs owns one work unit = (column block of up to 2 KB, class):
// CTA q of the cluster takes the q-th share of the class's neurons.  A CTA has three kinds of warps:
//   * two PRODUCER warps stage the two gathered input rows of 8 neurons at a time in shared memory (one 2 KB bulk
//     copy per row, ring of 3 stages) together with the neurons' gate masks;
//   * 256 CONSUMER threads own one 64-bit word column each, apply the gate and feed the result to a bit-sliced
//     counter in registers; at the end of a unit they drop the counter's planes into shared memory and go straight
//     on to the next unit;
//   * two REDUCER warps add the planes of all S CTAs through distributed shared memory -- CTA q does it for the
//     q-th share of the word columns, as a bit-sliced ripple-carry addition -- turn the sum into integers and store
//     out[sample][class].  This runs beside the consumers' next unit, off their critical path (done by the
//     consumers themselves it cost 60-160 us of a 370-470 us kernel).
// No atomics, no scratch memory, no second kernel.
//
// The cluster is also what keeps the gathers in L2: all CTAs of a cluster read the same 2 KB column block of x, the
// clusters that are resident together cover classes first (unit = column block * k + class), so only a handful
// of column blocks (n_in * 2 KB each) are live at a time and the second reader of an input row hits L2.
//
// Synchronisation inside the cluster uses two mbarriers per CTA with remote arrivals (one per warp and peer):
// red_full -- every consumer warp of every CTA has published its planes of the unit; red_free -- every reducer warp
// of every CTA has loaded what it needs from this CTA's planes.  Every wait is bounded; a wait that runs out raises
// the error flag that dl_async_error() reads and the CTA carries on without waiting (its output is then wrong,
// which the flag says).  All threads meet at one hardware cluster barrier at the start (barriers initialised) and
// one at the end (no CTA leaves while a peer may still touch its shared memory).
#include <cooperative_groups.h>
#include <stdlib.h>

#include "bitcount.cuh"
#include "common.cuh"
#include "gates.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace dl {

constexpr int kFgRows = 8;            // neurons per stage
constexpr int kFgStages = 3;
constexpr int kFgChunk = 2048;        // bytes of a row per unit: 256 words of 64 bits
constexpr int kFgWords = kFgChunk / 8;
constexpr int kFgProducers = 2;       // producer warps; stage i of the CTA is issued by warp i % kFgProducers
constexpr int kFgConsumers = kFgWords;
constexpr int kFgReducers = 2;        // reducer warps
constexpr int kFgThreads = 32 * kFgProducers + kFgConsumers + 32 * kFgReducers;
constexpr int kFgRedPlanes = 8;       // planes a CTA publishes: its share of a class is at most 255 neurons
constexpr int kFgMaxShare = (1 << kFgRedPlanes) - 1;
constexpr int kFgSumPlanes = kFgRedPlanes + 3;  // the sum over at most 8 CTAs
constexpr size_t kFgStageBytes = (size_t)2 * kFgRows * kFgChunk;

__device__ int g_fg_async_error = 0;

// ---- cluster-scope mbarrier and shared-memory helpers ----
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ unsigned long long ld_remote_u64(uint32_t remote_addr) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote_addr) : "memory");
    return v;
}

// Bounded waits; both give up at once when this CTA has already recorded a failure.
__device__ __forceinline__ bool fg_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (*abort_flag) return false;
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ bool fg_wait_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (*abort_flag) return false;
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

struct FgUnit {
    int64_t col0;    // first byte of the column block within a row
    int64_t row0;    // first neuron of this CTA's share
    int rows;        // neurons in the share
    int cls;
    uint32_t bytes;  // bytes per row segment
};

__device__ __forceinline__ FgUnit fg_unit(int64_t u, int64_t row_bytes, int block_bytes, int k, int m, int q, int nq) {
    FgUnit g;
    g.cls = (int)(u % k);
    g.col0 = (u / k) * block_bytes;
    g.bytes = (uint32_t)min((int64_t)block_bytes, row_bytes - g.col0);
    const int64_t r0 = ((int64_t)m * q) / nq, r1 = ((int64_t)m * (q + 1)) / nq;
    g.row0 = (int64_t)g.cls * m + r0;
    g.rows = (int)(r1 - r0);
    return g;
}

// Walks the stages of a CTA in order: over the units of its cluster, 8 neurons of its share at a time.
struct FgCursor {
    int64_t u, it;  // unit, stage number since the start of the kernel
    int r;          // first row of the stage within the share
    FgUnit g;
    bool valid;
    __device__ __forceinline__ void seek(int64_t nclusters, int64_t nunits, int64_t row_bytes, int block_bytes, int k, int m, int q, int nq) {
        // first unit from u on whose share has rows
        for (valid = false; u < nunits; u += nclusters) {
            g = fg_unit(u, row_bytes, block_bytes, k, m, q, nq);
            if (g.rows > 0) { valid = true; break; }
        }
    }
    __device__ __forceinline__ void start(int64_t cluster_id, int64_t nclusters, int64_t nunits, int64_t row_bytes, int block_bytes, int k,
                                          int m, int q, int nq) {
        u = cluster_id;
        it = 0;
        r = 0;
        seek(nclusters, nunits, row_bytes, block_bytes, k, m, q, nq);
    }
    __device__ __forceinline__ void next(int64_t nclusters, int64_t nunits, int64_t row_bytes, int block_bytes, int k, int m, int q, int nq) {
        if (!valid) return;
        ++it;
        r += kFgRows;
        if (r >= g.rows) {
            u += nclusters;
            r = 0;
            seek(nclusters, nunits, row_bytes, block_bytes, k, m, q, nq);
        }
    }
};

// gate on 32 sample bits from the masks {x: m0, y: ma, z: mb, w: mab}: m0 ^ (ma & a) ^ (mb & b) ^ (mab & a & b),
// arranged as three 3-input operations
__device__ __forceinline__ uint32_t gate_from_masks(uint32_t a, uint32_t b, const uint4 &mk) {
    const uint32_t u = mk.y ^ (mk.w & b);
    const uint32_t w = (a & u) ^ mk.x;
    return w ^ (mk.z & b);
}

// 8 x 8 bit-matrix transpose: bit c of byte r  <->  bit r of byte c
__device__ __forceinline__ unsigned long long transpose8x8(unsigned long long v) {
    unsigned long long t;
    t = (v ^ (v >> 7)) & 0x00AA00AA00AA00AAull;
    v = v ^ t ^ (t << 7);
    t = (v ^ (v >> 14)) & 0x0000CCCC0000CCCCull;
    v = v ^ t ^ (t << 14);
    t = (v ^ (v >> 28)) & 0x00000000F0F0F0F0ull;
    v = v ^ t ^ (t << 28);
    return v;
}

// 4 x 4 byte transpose: c[j] = (r[0].byte j, r[1].byte j, r[2].byte j, r[3].byte j)
__device__ __forceinline__ void transpose4x4_bytes(const uint32_t (&r)[4], uint32_t (&c)[4]) {
    const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[0], r[1], 0x7362);
    const uint32_t t2 = __byte_perm(r[2], r[3], 0x5140), t3 = __byte_perm(r[2], r[3], 0x7362);
    c[0] = __byte_perm(t0, t2, 0x5410);
    c[1] = __byte_perm(t0, t2, 0x7632);
    c[2] = __byte_perm(t1, t3, 0x5410);
    c[3] = __byte_perm(t1, t3, 0x7632);
}

// Eight planes of a bit-sliced counter (bit s of P[pl] = bit pl of the count of sample s) -> one byte per sample:
// byte i of T[j] = count of sample 8 j + i.
__device__ __forceinline__ void planes_to_bytes(const unsigned long long (&P)[8], unsigned long long (&T)[8]) {
    uint32_t lo[2][4], hi[2][4], tl[2][4], th[2][4];
#pragma unroll
    for (int pl = 0; pl < 8; ++pl) {
        lo[pl / 4][pl % 4] = (uint32_t)P[pl];
        hi[pl / 4][pl % 4] = (uint32_t)(P[pl] >> 32);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        transpose4x4_bytes(lo[h], tl[h]);
        transpose4x4_bytes(hi[h], th[h]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        // byte pl of `rows` = byte j of plane pl
        const unsigned long long rows = j < 4 ? ((unsigned long long)tl[1][j & 3] << 32) | tl[0][j & 3]
                                              : ((unsigned long long)th[1][j & 3] << 32) | th[0][j & 3];
        T[j] = transpose8x8(rows);
    }
}

template <int S>
__global__ void __launch_bounds__(kFgThreads, 2)
eval_groupbitsum_kernel(const uint8_t *__restrict__ x, const int64_t *__restrict__ a, const int64_t *__restrict__ b,
                        const uint8_t *__restrict__ gate, int32_t *__restrict__ out, int64_t row_bytes, int block_bytes,
                        int64_t batch, int k, int m, int nplanes, int64_t nunits) {
    extern __shared__ __align__(128) uint8_t smem[];
    unsigned long long *red = reinterpret_cast<unsigned long long *>(smem + kFgStages * kFgStageBytes);  // [planes][words]
    uint4 *meta = reinterpret_cast<uint4 *>(red + kFgRedPlanes * kFgWords);                               // [stages][rows]
    uint64_t *full = reinterpret_cast<uint64_t *>(meta + kFgStages * kFgRows);
    uint64_t *empty = full + kFgStages;
    uint64_t *red_full = empty + kFgStages;  // every CTA of the cluster has published its planes of the current unit
    uint64_t *red_free = red_full + 1;       // every CTA of the cluster has read this CTA's planes of the current unit
    __shared__ int s_abort;

    cg::cluster_group cluster = cg::this_cluster();
    const int q = (int)cluster.block_rank();
    const int64_t cluster_id = blockIdx.x / S, nclusters = gridDim.x / S;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    if (tid == 0) {
        for (int s = 0; s < kFgStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kFgConsumers / 32);
        }
        mbar_init(red_full, S * (kFgConsumers / 32));  // one arrival per consumer warp of every CTA of the cluster
        mbar_init(red_free, S * kFgReducers);          // one arrival per reducer warp of every CTA of the cluster
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    cluster.sync();  // every CTA's barriers exist before anybody arrives on them remotely
    volatile int *abort_flag = &s_abort;

    if (warp < kFgProducers) {
        // ---------------- producers: lane l < 16 copies input (l / 8) of neuron (l % 8) of the stage ----------------
        const int r_in = lane % kFgRows, which = (lane / kFgRows) & 1;
        const bool copier = lane < 2 * kFgRows;
        // The connection indices and gate of this warp's NEXT stage are fetched before the current stage's slot is
        // waited for, so their latency never sits between a slot becoming free and its refill.
        int64_t last = -1;  // latest stage this warp filled
        bool ok = true;
        FgCursor cur;
        cur.start(cluster_id, nclusters, nunits, row_bytes, block_bytes, k, m, q, S);
        for (int i = 0; i < warp; ++i) cur.next(nclusters, nunits, row_bytes, block_bytes, k, m, q, S);
        int64_t idx = 0;
        uint32_t op = 0;
        if (cur.valid && copier && r_in < cur.g.rows - cur.r) {
            idx = __ldg((which ? b : a) + cur.g.row0 + cur.r + r_in);
            op = __ldg(gate + cur.g.row0 + cur.r + r_in);
        }
        while (cur.valid) {
            FgCursor nxt = cur;
            for (int i = 0; i < kFgProducers; ++i) nxt.next(nclusters, nunits, row_bytes, block_bytes, k, m, q, S);
            int64_t idx_next = 0;
            uint32_t op_next = 0;
            if (nxt.valid && copier && r_in < nxt.g.rows - nxt.r) {
                idx_next = __ldg((which ? b : a) + nxt.g.row0 + nxt.r + r_in);
                op_next = __ldg(gate + nxt.g.row0 + nxt.r + r_in);
            }
            const int nr = min(kFgRows, cur.g.rows - cur.r);
            const bool valid = copier && r_in < nr;
            const int s = (int)(cur.it % kFgStages);
            const uint32_t use = (uint32_t)(cur.it / kFgStages);
            if (!fg_wait(empty + s, (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
            if (valid && which == 0) {
                const GateMasks gm = gate_masks((int)op);
                meta[s * kFgRows + r_in] = make_uint4(gm.m0, gm.ma, gm.mb, gm.mab);
            }
            // an input that the neuron's gate ignores is not fetched: its mask is zero, whatever the stage holds there
            const bool needed = valid && gate_needs_input(op, which);
            const uint32_t copies = (uint32_t)__popc(__ballot_sync(0xffffffffu, needed));
            __syncwarp();  // the masks / gate ids written above are ordered before lane 0's arrival
            if (lane == 0) mbar_arrive_expect_tx(full + s, copies * cur.g.bytes);
            __syncwarp();
            if (needed)
                bulk_load(smem + s * kFgStageBytes + (size_t)(which * kFgRows + r_in) * kFgChunk, x + idx * row_bytes + cur.g.col0,
                          cur.g.bytes, full + s);
            last = cur.it;
            cur = nxt;
            idx = idx_next;
            op = op_next;
        }
        if (!ok || *abort_flag) {
            // flag it, stop the consumers' waiting, and give this warp's last copies time to land
            if (lane == 0) {
                g_fg_async_error = 1;
                s_abort = 1;
            }
            __syncwarp();
            if (last >= 0) mbar_wait(full + (last % kFgStages), (uint32_t)(last / kFgStages) & 1u);
        }
    } else if (warp < kFgProducers + kFgConsumers / 32) {
        // ---------------- consumers: one 64-bit word column per thread ----------------
        const int ct = tid - 32 * kFgProducers;
        uint32_t remote_full = 0;  // lane p < S: the red_full barrier of rank p
        if (lane < S) remote_full = map_to_rank(smem_addr(red_full), (uint32_t)lane);
        int64_t it = 0;
        uint32_t n = 0;  // units done
        for (int64_t u = cluster_id; u < nunits; u += nclusters, ++n) {
            const FgUnit g = fg_unit(u, row_bytes, block_bytes, k, m, q, S);
            const bool mine = (uint32_t)ct * 8u < g.bytes;
            BitCounterT<kFgRedPlanes - 3> cn;  // a share is at most 255 neurons
            cn.clear();
            for (int r = 0; r < g.rows; r += kFgRows, ++it) {
                const int s = (int)(it % kFgStages);
                const uint32_t use = (uint32_t)(it / kFgStages);
                if (!fg_wait(full + s, use & 1u, abort_flag)) {
                    g_fg_async_error = 1;
                    s_abort = 1;
                    continue;  // keep the iteration counts; nothing is waited for any more
                }
                const int nr = min(kFgRows, g.rows - r);
                // the gates' results first, then the slot goes back to the producers, then the counting: the slot is
                // not held while the adder tree runs
                unsigned long long v[kFgRows];
                if (mine) {
                    const uint2 *col_a = reinterpret_cast<const uint2 *>(smem + s * kFgStageBytes) + ct;
                    const uint2 *col_b = col_a + kFgRows * kFgWords;
                    const uint4 *mk = meta + s * kFgRows;
                    // rows past the end of the share count as zero words
#pragma unroll
                    for (int i = 0; i < kFgRows; ++i) {
                        v[i] = 0ull;
                        if (i < nr) {
                            const uint2 va = col_a[i * kFgWords], vb = col_b[i * kFgWords];
                            const uint4 mm = mk[i];
                            v[i] = ((unsigned long long)gate_from_masks(va.y, vb.y, mm) << 32) | gate_from_masks(va.x, vb.x, mm);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + s);
                if (mine) cn.add8(v);
            }

            // ---- publish this CTA's planes of unit n ----
            if (n > 0 && !fg_wait_cluster(red_free, (n - 1u) & 1u, abort_flag)) {  // every reducer has read the planes of unit n - 1
                g_fg_async_error = 1;
                s_abort = 1;
            }
#pragma unroll
            for (int pl = 0; pl < kFgRedPlanes; ++pl)
                if (pl < nplanes) red[pl * kFgWords + ct] = mine ? cn.plane(pl) : 0ull;
            // the warp converges (which orders every lane's stores before it), then lane p arrives, with release at
            // cluster scope, at rank p
            __syncwarp();
            if (lane < S) mbar_arrive_remote(remote_full);
        }
    } else {
        // ---------------- reducers: sum of the S CTAs' planes for this CTA's share of the word columns ----------------
        const int rt = tid - 32 * kFgProducers - kFgConsumers;  // 0 .. 32 * kFgReducers - 1
        constexpr int kWordsPerCta = kFgWords / S;
        uint32_t remote_free = 0;  // lane p < S: the red_free barrier of rank p
        if (lane < S) remote_free = map_to_rank(smem_addr(red_free), (uint32_t)lane);
        uint32_t remote_red[S];
#pragma unroll
        for (int p = 0; p < S; ++p) remote_red[p] = map_to_rank(smem_addr(red), (uint32_t)p);
        const int sum_planes = min(kFgSumPlanes, nplanes + (S == 8 ? 3 : S == 4 ? 2 : 1));
        uint32_t n = 0;
        for (int64_t u = cluster_id; u < nunits; u += nclusters, ++n) {
            const FgUnit g = fg_unit(u, row_bytes, block_bytes, k, m, q, S);
            if (!fg_wait_cluster(red_full, n & 1u, abort_flag)) {
                g_fg_async_error = 1;
                s_abort = 1;
            }
            for (int w0 = 0; w0 < kWordsPerCta; w0 += 32 * kFgReducers) {
                const int wl = w0 + rt;                  // word within this CTA's share
                const int w = q * kWordsPerCta + wl;     // word within the column block
                const bool active = wl < kWordsPerCta;
                // bit-sliced sum: sum[i] holds bit i of the count of each of the word's 64 samples
                unsigned long long sum[kFgSumPlanes];
#pragma unroll
                for (int i = 0; i < kFgSumPlanes; ++i) sum[i] = 0ull;
                if (active) {
#pragma unroll
                    for (int p = 0; p < S; ++p) {
                        unsigned long long pv[kFgRedPlanes];
#pragma unroll
                        for (int i = 0; i < kFgRedPlanes; ++i)
                            pv[i] = i < nplanes ? ld_remote_u64(remote_red[p] + 8u * (uint32_t)(i * kFgWords + w)) : 0ull;
                        unsigned long long carry = 0ull;
#pragma unroll
                        for (int i = 0; i < kFgSumPlanes; ++i) {
                            const unsigned long long add = i < kFgRedPlanes ? pv[i] : 0ull;
                            const unsigned long long t = sum[i] ^ add;
                            const unsigned long long c_out = (sum[i] & add) | (carry & t);
                            sum[i] = t ^ carry;
                            carry = c_out;
                        }
                    }
                }
                if (w0 + 32 * kFgReducers >= kWordsPerCta) {
                    // last pass: everything this warp needs from its peers is in registers
                    __syncwarp();
                    if (lane < S) mbar_arrive_remote(remote_free);
                }
                if (active && (uint32_t)w * 8u < g.bytes) {
                    unsigned long long lo_planes[8], hi_planes[8], lo_bytes[8], hi_bytes[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        lo_planes[i] = sum[i];
                        hi_planes[i] = 8 + i < kFgSumPlanes ? sum[8 + i] : 0ull;
                    }
                    planes_to_bytes(lo_planes, lo_bytes);
                    const bool wide = sum_planes > 8;  // counts above 255 are possible
                    if (wide) planes_to_bytes(hi_planes, hi_bytes);
                    const int64_t s0 = (g.col0 + (int64_t)w * 8) * 8;  // first sample of the word
                    int32_t *dst = out + s0 * k + g.cls;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            int32_t cnt = (int32_t)((lo_bytes[j] >> (8 * i)) & 0xFFull);
                            if (wide) cnt |= (int32_t)((hi_bytes[j] >> (8 * i)) & 0xFFull) << 8;
                            if (s0 + 8 * j + i < batch) dst[(int64_t)(8 * j + i) * k] = cnt;
                        }
                    }
                }
            }
        }
    }
    cluster.sync();  // nobody leaves while a peer may still read its planes or arrive on its barriers
}

int eval_groupbitsum_async_error() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, g_fg_async_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return flag;
}

static size_t fg_shared_bytes() {
    return kFgStages * kFgStageBytes + (size_t)kFgRedPlanes * kFgWords * 8 + (size_t)kFgStages * kFgRows * sizeof(uint4) +
           (2 * kFgStages + 2) * sizeof(uint64_t);
}

static int fg_cluster_size(int64_t m) {
    // The consumers are instruction bound, and every unit costs a fixed number of instructions for the reduction:
    // the fewer CTAs share a class the better, as long as a share stays within 255 neurons (and above 16).
    // DL_TUNE_FUSED_CLUSTER = 2 | 4 | 8 overrides (for A/B timing).
    const int force = tuning(DL_TUNE_FUSED_CLUSTER);
    if (force == 2 || force == 4 || force == 8) return force;
    if (m <= 2 * kFgMaxShare && m < 4 * 64) return 2;
    if (m <= 4 * kFgMaxShare) return 4;
    return 8;
}

template <int S>
static int launch_fg(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, int32_t *out, int64_t row_bytes,
                     int64_t batch, int64_t k, int64_t m, cudaStream_t st) {
    const size_t smem = fg_shared_bytes();
    if (cudaFuncSetAttribute(eval_groupbitsum_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return launch_status("dl_eval_groupbitsum (shared memory opt-in)");
    int nplanes = 1;
    while (nplanes < kFgRedPlanes && ((int64_t)1 << nplanes) <= ceil_div(m, S)) ++nplanes;

    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.blockDim = dim3(kFgThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    // persistent grid: as many clusters as can be resident together (clusters do not span GPCs, so this is a
    // little under 2 CTAs x SMs / S), never more than there are units
    cfg.gridDim = dim3((unsigned)(S * 64));
    int resident = 0;
    if (cudaOccupancyMaxActiveClusters(&resident, eval_groupbitsum_kernel<S>, &cfg) != cudaSuccess || resident <= 0) {
        cudaGetLastError();
        return fail(DL_ERR_CUDA, "dl_eval_groupbitsum: no cluster of %d CTAs can be resident", S);
    }
    // Column block: 2 KB.  Narrower blocks that would fill the last round of the static round-robin better were
    // measured slower throughout: the kernel's time goes with the number of stages, not with their width.  So was
    // sharing the last round's units among all clusters stage by stage, with the parts' counts added to a zeroed out
    // by atomics: 300 against 288 us for 8000 gates x 2^20 samples, 70 against 64 us for 2^17 samples.
    const int block_bytes = (int)(row_bytes < kFgChunk ? row_bytes : kFgChunk);
    const int64_t nunits = ceil_div(row_bytes, block_bytes) * k;
    const int64_t nclusters = nunits < resident ? nunits : resident;
    cfg.gridDim = dim3((unsigned)(nclusters * S));
    const uint8_t *xb = reinterpret_cast<const uint8_t *>(x);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, eval_groupbitsum_kernel<S>, xb, a, b, gate, out, row_bytes, block_bytes, batch, (int)k,
                                             (int)m, nplanes, nunits);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(DL_ERR_CUDA, "dl_eval_groupbitsum: %s", cudaGetErrorString(e));
    }
    return launch_status("dl_eval_groupbitsum");
}

}  // namespace dl

using namespace dl;

// 1 when dl_eval_groupbitsum accepts these sizes and pointers, else 0 (the caller then runs dl_eval_packed and
// dl_groupbitsum one after the other).
extern "C" DL_API int dl_eval_groupbitsum_applicable(const void *x, int64_t n_in, int64_t n_out, int64_t words, int bit_count,
                                                     int64_t k) {
    if (!(bit_count == 8 || bit_count == 16 || bit_count == 32 || bit_count == 64)) return 0;
    if (n_in <= 0 || n_out <= 0 || k <= 0 || words <= 0 || n_out % k != 0) return 0;
    const int64_t row_bytes = words * (bit_count / 8), m = n_out / k;
    if (row_bytes % 16 != 0 || row_bytes < 512 || !aligned_to(x, 16)) return 0;
    if (m < 32 || ceil_div(m, fg_cluster_size(m)) > kFgMaxShare || k > 65535) return 0;
    return 1;
}

extern "C" DL_API int dl_eval_groupbitsum(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, int32_t *out,
                                          int64_t n_in, int64_t n_out, int64_t words, int64_t pad_len, int64_t k, int bit_count,
                                          void *stream) {
    DL_REQUIRE(dl_eval_groupbitsum_applicable(x, n_in, n_out, words, bit_count, k) == 1, DL_ERR_INVALID_ARG,
               "dl_eval_groupbitsum: sizes outside the fused kernel's range (ask dl_eval_groupbitsum_applicable first)");
    DL_REQUIRE(pad_len >= 0 && pad_len < bit_count, DL_ERR_INVALID_ARG, "dl_eval_groupbitsum: pad_len %lld out of range",
               (long long)pad_len);
    DL_REQUIRE(x && a && b && gate && out, DL_ERR_INVALID_ARG, "dl_eval_groupbitsum: null pointer");
    const int64_t row_bytes = words * (bit_count / 8), m = n_out / k, batch = words * bit_count - pad_len;
    cudaStream_t st = as_stream(stream);
    switch (fg_cluster_size(m)) {
        case 8: return launch_fg<8>(x, a, b, gate, out, row_bytes, batch, k, m, st);
        case 4: return launch_fg<4>(x, a, b, gate, out, row_bytes, batch, k, m, st);
        default: return launch_fg<2>(x, a, b, gate, out, row_bytes, batch, k, m, st);
    }
}
