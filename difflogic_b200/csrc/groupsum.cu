// Float GroupSum on the feature-major activation of the last layer, forward and backward.
//
//   out[s][c]    = (sum_{r < m} x[c*m + r][s]) / tau          m = n / k
//   grad_x[i][s] = grad_out[s][i / m] / tau
//
// Forward.  The rows of a class are split into `chunks` pieces; a CTA sums one piece for a
// block of 128 batch columns (32 lanes x float4, 8 warps striding the rows, shared-memory
// merge) and stores the partial sum in the caller's workspace.  The CTA that finishes a
// (class, column block) last adds the pieces in a fixed order and writes the result, so the
// sum does not depend on scheduling and no float atomics are used.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "common.cuh"

namespace dl {

constexpr int kGsCols = 128;          // batch columns per CTA
constexpr int kGsCounterBytes = 4096;  // counters at the head of the workspace
constexpr int kGsMaxCounters = kGsCounterBytes / 4;

static int64_t groupsum_chunks(int64_t n, int64_t batch, int64_t k) {
    const int64_t m = n / k;
    const int64_t colblocks = ceil_div(batch, kGsCols);
    // aim at ~2 CTAs per SM over 148 SMs, at least 16 rows per piece
    int64_t chunks = ceil_div(296, k * colblocks);
    if (chunks > ceil_div(m, 16)) chunks = ceil_div(m, 16);
    if (chunks < 1) chunks = 1;
    return chunks;
}

// True when dl_groupsum_f32 runs the cluster kernel (no scratch) for this shape: several pieces per class and classes
// of 64 .. 4096 rows.  DL_TUNE_GROUPSUM_KERNEL = 1 forces the workspace kernel (for A/B measurements).
static bool groupsum_takes_cluster_kernel(int64_t n, int64_t batch, int64_t k) {
    const int64_t m_rows = n / k;
    return tuning(DL_TUNE_GROUPSUM_KERNEL) != 1 && groupsum_chunks(n, batch, k) > 1 && m_rows >= 64 && m_rows <= 4096 &&
           ceil_div(batch, kGsCols) <= 65535;
}

__global__ void __launch_bounds__(kThreads)
groupsum_kernel(const float *__restrict__ x, float *__restrict__ out, unsigned int *__restrict__ counters,
                float *__restrict__ partial, int64_t batch, int k, int m, int chunks, float tau) {
    __shared__ float s_part[8][kGsCols];
    __shared__ bool s_last;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int colblock = blockIdx.x, c = blockIdx.y, q = blockIdx.z;
    const int64_t col0 = (int64_t)colblock * kGsCols + lane * 4;
    const int64_t rbeg = (int64_t)c * m + ((int64_t)m * q) / chunks;
    const int64_t rend = (int64_t)c * m + ((int64_t)m * (q + 1)) / chunks;

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool vec = (batch % 4 == 0) && col0 + 3 < batch;
    if (vec) {
#pragma unroll 4
        for (int64_t r = rbeg + warp; r < rend; r += 8) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x + r * batch + col0));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    } else {
        for (int64_t r = rbeg + warp; r < rend; r += 8) {
            const float *p = x + r * batch + col0;
            if (col0 + 0 < batch) acc.x += __ldg(p + 0);
            if (col0 + 1 < batch) acc.y += __ldg(p + 1);
            if (col0 + 2 < batch) acc.z += __ldg(p + 2);
            if (col0 + 3 < batch) acc.w += __ldg(p + 3);
        }
    }
    s_part[warp][lane * 4 + 0] = acc.x;
    s_part[warp][lane * 4 + 1] = acc.y;
    s_part[warp][lane * 4 + 2] = acc.z;
    s_part[warp][lane * 4 + 3] = acc.w;
    __syncthreads();

    const int64_t gcol = (int64_t)colblock * kGsCols + tid;
    float sum = 0.f;
    if (tid < kGsCols) {
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) sum += s_part[wv][tid];
    }
    if (chunks == 1) {
        if (tid < kGsCols && gcol < batch) out[gcol * k + c] = sum / tau;
        return;
    }
    // partial[(c * chunks + q)][batch]
    if (tid < kGsCols && gcol < batch) partial[((int64_t)c * chunks + q) * batch + gcol] = sum;
    __threadfence();
    __syncthreads();
    unsigned int *counter = counters + ((int64_t)c * gridDim.x + colblock) % kGsMaxCounters;
    if (tid == 0) {
        const unsigned int done = atomicAdd(counter, 1u);
        s_last = (done == (unsigned)chunks - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid < kGsCols && gcol < batch) {
        float total = 0.f;
        for (int qq = 0; qq < chunks; ++qq) total += __ldcg(partial + ((int64_t)c * chunks + qq) * batch + gcol);
        out[gcol * k + c] = total / tau;
    }
    if (tid == 0) *counter = 0u;  // ready for the next call
}

// Forward for classes of moderate size: a thread-block cluster of kGcCluster CTAs shares one (class, column
// block); each CTA sums its piece of the rows, the pieces meet in the first CTA's view of the others' shared
// memory (distributed shared memory) and are added there in a fixed order.  No scratch in global memory,
// no fence, no atomics: one memory round trip plus a cluster barrier.
constexpr int kGcThreads = 512;
constexpr int kGcCluster = 8;

__global__ void __launch_bounds__(kGcThreads)
groupsum_cluster_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t batch, int k, int m, float tau) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float s_part[kGcThreads / 32][kGsCols];
    __shared__ float s_sum[kGsCols];
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int colblock = blockIdx.x, c = blockIdx.y;
    const int q = (int)cluster.block_rank(), nq = (int)cluster.num_blocks();
    const int64_t col0 = (int64_t)colblock * kGsCols + lane * 4;
    const int64_t rbeg = (int64_t)c * m + ((int64_t)m * q) / nq;
    const int64_t rend = (int64_t)c * m + ((int64_t)m * (q + 1)) / nq;

    grid_dependency_wait();  // x is the output of the kernel just before
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((batch % 4 == 0) && col0 + 3 < batch) {
#pragma unroll 8
        for (int64_t r = rbeg + warp; r < rend; r += kGcThreads / 32) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x + r * batch + col0));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    } else {
        for (int64_t r = rbeg + warp; r < rend; r += kGcThreads / 32) {
            const float *p = x + r * batch + col0;
            if (col0 + 0 < batch) acc.x += __ldg(p + 0);
            if (col0 + 1 < batch) acc.y += __ldg(p + 1);
            if (col0 + 2 < batch) acc.z += __ldg(p + 2);
            if (col0 + 3 < batch) acc.w += __ldg(p + 3);
        }
    }
    s_part[warp][lane * 4 + 0] = acc.x;
    s_part[warp][lane * 4 + 1] = acc.y;
    s_part[warp][lane * 4 + 2] = acc.z;
    s_part[warp][lane * 4 + 3] = acc.w;
    __syncthreads();
    if (tid < kGsCols) {
        float sum = 0.f;
#pragma unroll
        for (int wv = 0; wv < kGcThreads / 32; ++wv) sum += s_part[wv][tid];
        s_sum[tid] = sum;
    }
    cluster.sync();
    const int64_t gcol = (int64_t)colblock * kGsCols + tid;
    if (q == 0 && tid < kGsCols && gcol < batch) {
        float total = 0.f;
        for (int r = 0; r < nq; ++r) total += *cluster.map_shared_rank(&s_sum[tid], r);
        out[gcol * k + c] = total / tau;
    }
    cluster.sync();  // the other CTAs' shared memory must stay alive until the first one has read it
}

// Mean cross-entropy loss over ALL samples from the scores in global memory, and the gradient of the loss w.r.t. the
// scores laid out as one row per class; run by the one CTA that holds the ticket.  THREADS: its size.
template <int THREADS>
__device__ __forceinline__ void cross_entropy_of_scores(const float *__restrict__ scores, const int64_t *__restrict__ target,
                                                        float *__restrict__ loss, float *__restrict__ grad_classes,
                                                        unsigned int *__restrict__ counter, int64_t batch, int k, float tau,
                                                        float *s_red) {
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const float scale = 1.f / (float)batch;
    float local = 0.f;
    constexpr int kRowRegs = 16;  // classes held in registers (one read of the scores instead of three)
    for (int64_t s = tid; s < batch; s += THREADS) {
        const float *row = scores + s * k;
        const int64_t t = target[s];
        if (k <= kRowRegs) {
            float r[kRowRegs];
#pragma unroll
            for (int cc = 0; cc < kRowRegs; ++cc) r[cc] = cc < k ? __ldcg(row + cc) : -INFINITY;
            float mx = -INFINITY;
#pragma unroll
            for (int cc = 0; cc < kRowRegs; ++cc) mx = fmaxf(mx, r[cc]);  // the padding never wins: max is order-free
            float sum = 0.f;
#pragma unroll
            for (int cc = 0; cc < kRowRegs; ++cc)
                if (cc < k) sum += expf(r[cc] - mx);
            const float lse = mx + logf(sum);
#pragma unroll
            for (int cc = 0; cc < kRowRegs; ++cc) {
                if (cc < k) {
                    const float p = expf(r[cc] - lse);
                    const float g = (p - (t == cc ? 1.f : 0.f)) * scale;
                    grad_classes[(int64_t)cc * batch + s] = g / tau;
                    if (t == cc) local += lse - r[cc];
                }
            }
        } else {
            float mx = -INFINITY;
            for (int cc = 0; cc < k; ++cc) mx = fmaxf(mx, __ldcg(row + cc));
            float sum = 0.f;
            for (int cc = 0; cc < k; ++cc) sum += expf(__ldcg(row + cc) - mx);
            const float lse = mx + logf(sum);
            for (int cc = 0; cc < k; ++cc) {
                const float p = expf(__ldcg(row + cc) - lse);
                const float g = (p - (t == cc ? 1.f : 0.f)) * scale;
                grad_classes[(int64_t)cc * batch + s] = g / tau;
            }
            if (t >= 0 && t < k) local += lse - __ldcg(row + t);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    if (lane == 0) s_red[warp] = local;
    __syncthreads();
    if (warp == 0) {
        float v = lane < THREADS / 32 ? s_red[lane] : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) {
            loss[0] = v / (float)batch;
            *counter = 0u;  // ready for the next call
        }
    }
}

// GroupSum forward + cross-entropy loss (mean over the batch) + the gradient of the loss w.r.t. the class scores, in
// ONE launch: the head of a training step.  Same cluster scheme as above with one barrier less (every CTA pushes its
// piece into the first CTA's shared memory, then one cluster barrier), and the first CTA of the cluster that finishes
// LAST (a ticket in global memory) computes the loss over all samples:
//   scores[s][c] = class sums / tau;  p = softmax(scores[s]);  loss = -(1/B) sum_s log p[s][target[s]]
//   grad_classes[c][s] = ((p[s][c] - [c == target[s]]) * (1/B)) / tau      -- feature-major [k][batch]
// grad_classes is what the last layer's backward kernels read as "one grad_y row per class"
// (dl_backward_w_classes_f32 / dl_backward_x_classes_f32): the [n][batch] gradient of the layer's output, whose rows
// are equal within a class, is never formed.  The arithmetic per sample is that of cross_entropy_kernel followed by
// cross_entropy_backward_kernel (grad_loss = 1) and groupsum_backward_kernel, in the same order.
__global__ void __launch_bounds__(kGcThreads)
groupsum_ce_kernel(const float *__restrict__ x, const int64_t *__restrict__ target, float *__restrict__ scores,
                   float *__restrict__ loss, float *__restrict__ grad_classes, unsigned int *__restrict__ counter, int64_t batch,
                   int k, int m, float tau) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float s_part[kGcThreads / 32][kGsCols];
    __shared__ float s_all[kGcCluster][kGsCols];  // used in the first CTA of the cluster: the pieces of all CTAs
    __shared__ float s_red[kGcThreads / 32];
    __shared__ bool s_last;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int colblock = blockIdx.x, c = blockIdx.y;
    const int q = (int)cluster.block_rank(), nq = (int)cluster.num_blocks();
    const int64_t col0 = (int64_t)colblock * kGsCols + lane * 4;
    const int64_t rbeg = (int64_t)c * m + ((int64_t)m * q) / nq;
    const int64_t rend = (int64_t)c * m + ((int64_t)m * (q + 1)) / nq;

    grid_dependency_wait();  // x is the output of the kernel just before
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((batch % 4 == 0) && col0 + 3 < batch) {
#pragma unroll 16
        for (int64_t r = rbeg + warp; r < rend; r += kGcThreads / 32) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x + r * batch + col0));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    } else {
        for (int64_t r = rbeg + warp; r < rend; r += kGcThreads / 32) {
            const float *p = x + r * batch + col0;
            if (col0 + 0 < batch) acc.x += __ldg(p + 0);
            if (col0 + 1 < batch) acc.y += __ldg(p + 1);
            if (col0 + 2 < batch) acc.z += __ldg(p + 2);
            if (col0 + 3 < batch) acc.w += __ldg(p + 3);
        }
    }
    s_part[warp][lane * 4 + 0] = acc.x;
    s_part[warp][lane * 4 + 1] = acc.y;
    s_part[warp][lane * 4 + 2] = acc.z;
    s_part[warp][lane * 4 + 3] = acc.w;
    __syncthreads();
    if (tid < kGsCols) {
        float sum = 0.f;
#pragma unroll
        for (int wv = 0; wv < kGcThreads / 32; ++wv) sum += s_part[wv][tid];
        *cluster.map_shared_rank(&s_all[q][tid], 0) = sum;  // into the first CTA's shared memory
    }
    cluster.sync();
    if (q != 0) return;
    const int64_t gcol = (int64_t)colblock * kGsCols + tid;
    if (tid < kGsCols && gcol < batch) {
        float total = 0.f;
        for (int r = 0; r < nq; ++r) total += s_all[r][tid];  // same order as groupsum_cluster_kernel
        scores[gcol * k + c] = total / tau;
    }
    // ---- ticket: the first CTA of the last cluster to get here computes the loss
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int total_units = gridDim.x * gridDim.y;
        s_last = atomicAdd(counter, 1u) == total_units - 1u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    cross_entropy_of_scores<kGcThreads>(scores, target, loss, grad_classes, counter, batch, k, tau, s_red);
}

// Head of a training step when the last layer's forward kernel has already added up its rows per class and CTA
// (dl_forward_class_sums_f32): `sums` is [2 * runs][batch], rows 2*i and 2*i+1 holding the sums of the i-th run of `nb`
// rows for the class of its first row and for the next class.  A CTA takes (128 batch columns, class): its eight
// groups of 128 threads add the class's pieces in a fixed order (piece p goes to group p % 8, the groups are added in
// order) and write the scores; the CTA that holds the ticket computes the loss and the class-row gradients as in
// groupsum_ce_kernel.  Reads pieces * batch floats per class that the forward kernel has just written (L2).
constexpr int kCsThreads = 1024;
constexpr int kCsGroups = kCsThreads / kGsCols;  // 8

__global__ void __launch_bounds__(kCsThreads)
class_sums_ce_kernel(const float *__restrict__ sums, const int64_t *__restrict__ target, float *__restrict__ scores,
                     float *__restrict__ loss, float *__restrict__ grad_classes, unsigned int *__restrict__ counter, int64_t batch, int k,
                     int m, int nb, float tau) {
    __shared__ float s_part[kCsGroups][kGsCols];
    __shared__ float s_red[kCsThreads / 32];
    __shared__ bool s_last;
    const int tid = threadIdx.x, g = tid / kGsCols, col = tid % kGsCols;
    const int c = blockIdx.y;
    const int64_t gcol = (int64_t)blockIdx.x * kGsCols + col;
    const unsigned row0 = (unsigned)c * (unsigned)m;  // n < 2^31
    const unsigned first = row0 / (unsigned)nb, last = (row0 + (unsigned)m - 1u) / (unsigned)nb;  // runs that hold rows of class c
    grid_dependency_wait();  // sums is the output of the kernel just before
    float acc = 0.f;
    if (gcol < batch) {
#pragma unroll 8
        for (unsigned i = first + (unsigned)g; i <= last; i += kCsGroups) {
            const unsigned e = i * (unsigned)nb >= row0 ? 0u : 1u;  // the run's first row is of class c, or of the class before it
            acc += __ldcg(sums + (int64_t)(2u * i + e) * batch + gcol);
        }
    }
    s_part[g][col] = acc;
    __syncthreads();
    if (g == 0 && gcol < batch) {
        float total = 0.f;
#pragma unroll
        for (int gg = 0; gg < kCsGroups; ++gg) total += s_part[gg][col];
        scores[gcol * k + c] = total / tau;
    }
    // ---- ticket: the CTA that gets here last computes the loss over all samples
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(counter, 1u) == gridDim.x * gridDim.y - 1u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    cross_entropy_of_scores<kCsThreads>(scores, target, loss, grad_classes, counter, batch, k, tau, s_red);
}

// The same head for a batch of at most 128 samples in ONE thread-block cluster of eight CTAs, with nothing but the final
// results going through global memory (at most KC classes of at most IT * 64 pieces each).  Piece p of a class goes
// to CTA p % 8, thread group (p / 8) % 8: every thread has at most IT loads per class, all classes' loads in flight
// together.  The groups meet in shared memory, the CTAs in the first CTA's view of the others' shared memory
// (distributed shared memory), always added in a fixed order; the first CTA's first 128 threads go on to the softmax,
// the loss and the class-row gradients of their sample.  One round of loads, two barriers, no fence, no ticket.
constexpr int kCsCluster = 8;

template <int KC, int IT>
__global__ void __launch_bounds__(kCsThreads, 1)
class_sums_ce_cluster_kernel(const float *__restrict__ sums, const int64_t *__restrict__ target, float *__restrict__ scores,
                             float *__restrict__ loss, float *__restrict__ grad_classes, int64_t batch, int k, int m, int nb, float tau) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ float s_dyn[];  // [k][kCsGroups][kGsCols] partial sums of the groups
    __shared__ float s_cta[KC][kGsCols];  // this CTA's sum per class and column
    __shared__ unsigned s_first[KC], s_last[KC];
    __shared__ float s_red[kGsCols / 32];
    const int tid = threadIdx.x, g = tid / kGsCols, col = tid % kGsCols;
    const unsigned q = cluster.block_rank();
    if (tid < KC && tid < k) {  // runs that hold rows of class tid (32-bit arithmetic: n < 2^31)
        const unsigned row0 = (unsigned)tid * (unsigned)m;
        s_first[tid] = row0 / (unsigned)nb;
        s_last[tid] = (row0 + (unsigned)m - 1u) / (unsigned)nb;
    }
    __syncthreads();
    grid_dependency_wait();  // sums is the output of the kernel just before
    float acc[KC];
#pragma unroll
    for (int c = 0; c < KC; ++c) {
        acc[c] = 0.f;
        if (c < k) {  // uniform: no divergence, the loads of all classes are issued back to back
            const unsigned first = s_first[c], last = s_last[c], row0 = (unsigned)c * (unsigned)m;
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                // a piece beyond the class's last run, or a column beyond the batch, reads a valid address and adds zero
                const unsigned want = first + q + (unsigned)(kCsCluster * g) + (unsigned)(it * kCsCluster * kCsGroups);
                const bool live = want <= last && col < batch;
                const unsigned i = live ? want : first;
                // a run whose first row lies before the class's first row began in the class before it
                const unsigned e = i * (unsigned)nb >= row0 ? 0u : 1u;
                const float v = __ldcg(sums + (int64_t)(2u * i + e) * batch + (live ? col : 0));
                acc[c] += live ? v : 0.f;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < KC; ++c)
        if (c < k) s_dyn[(c * kCsGroups + g) * kGsCols + col] = acc[c];
    __syncthreads();
    for (int idx = tid; idx < k * kGsCols; idx += kCsThreads) {
        const int c = idx / kGsCols, cl = idx % kGsCols;
        float total = 0.f;
#pragma unroll
        for (int gg = 0; gg < kCsGroups; ++gg) total += s_dyn[(c * kCsGroups + gg) * kGsCols + cl];
        s_cta[c][cl] = total;
    }
    cluster.sync();
    if (q == 0) {
        for (int idx = tid; idx < k * kGsCols; idx += kCsThreads) {
            const int c = idx / kGsCols, cl = idx % kGsCols;
            float total = 0.f;
#pragma unroll
            for (int r = 0; r < kCsCluster; ++r) total += *cluster.map_shared_rank(&s_cta[c][cl], r);
            const float sc = total / tau;
            s_dyn[c * kGsCols + cl] = sc;  // the groups' sums are spent: the scores take their place, [class][column]
            if (cl < batch) scores[(int64_t)cl * k + c] = sc;
        }
    }
    cluster.sync();  // the other CTAs' shared memory stays alive until the first one has read it
    if (q != 0 || tid >= kGsCols) return;  // the first CTA's first four warps go on, one sample each
    float local = 0.f;
    if (col < batch) {
        const int64_t t = target[col];
        const float scale = 1.f / (float)batch;
        float mx = -INFINITY;
        for (int c = 0; c < k; ++c) mx = fmaxf(mx, s_dyn[c * kGsCols + col]);
        float sum = 0.f;
        for (int c = 0; c < k; ++c) sum += expf(s_dyn[c * kGsCols + col] - mx);
        const float lse = mx + logf(sum);
        for (int c = 0; c < k; ++c) {
            const float sc = s_dyn[c * kGsCols + col];
            const float p = expf(sc - lse);
            const float gr = (p - (t == c ? 1.f : 0.f)) * scale;
            grad_classes[(int64_t)c * batch + col] = gr / tau;
            if (t == c) local += lse - sc;
        }
    }
    // sum of the samples' losses: shuffle within the warps, then over the four warps in order
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    if (tid % 32 == 0) s_red[tid / 32] = local;
    asm volatile("bar.sync 1, 128;" ::: "memory");  // only these 128 threads are left
    if (tid == 0) loss[0] = (((s_red[0] + s_red[1]) + s_red[2]) + s_red[3]) / (float)batch;
}

// Backward: grad_x[i][:] = grad_out[:, class(i)] / tau.  A CTA takes a run of rows of one class and a block of
// 128 batch columns: the class's 128 gradient values are read once, then row after row is written.
constexpr int kGbkRows = 128;  // rows per CTA

//
// With FROM_LOSS the class gradients are not read but formed from the softmax probabilities of a cross-entropy
// loss (mean over the batch) on the GroupSum's scores: (probs[s][c] - [c == target[s]]) * grad_loss / batch, in the
// same order of operations as the separate loss-backward kernel, so the result is bit-identical to running the two
// kernels one after the other.
template <bool FROM_LOSS>
__global__ void __launch_bounds__(kThreads)
groupsum_backward_kernel(const float *__restrict__ grad_out, const int64_t *__restrict__ target, const float *__restrict__ grad_loss,
                         float *__restrict__ grad_x, int64_t batch, int k, int m, float tau, int pieces) {
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int c = blockIdx.x / pieces, piece = blockIdx.x % pieces;
    const int64_t r0 = (int64_t)c * m + ((int64_t)m * piece) / pieces;
    const int64_t r1 = (int64_t)c * m + ((int64_t)m * (piece + 1)) / pieces;
    const int64_t col = (int64_t)blockIdx.y * kGsCols + lane * 4;
    grid_dependency_wait();  // grad_out comes from the loss' backward just before
    float v[4];
    if (FROM_LOSS) {
        const float scale = grad_loss[0] / (float)batch;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = 0.f;
            if (col + i < batch) {
                const float g = (grad_out[(col + i) * k + c] - (target[col + i] == c ? 1.f : 0.f)) * scale;
                v[i] = g / tau;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = (col + i < batch) ? __ldg(grad_out + (col + i) * k + c) / tau : 0.f;
    }
    if (batch % 4 == 0) {
        if (col >= batch) return;
        const float4 v4 = make_float4(v[0], v[1], v[2], v[3]);
        for (int64_t r = r0 + warp; r < r1; r += kThreads / 32) *reinterpret_cast<float4 *>(grad_x + r * batch + col) = v4;
    } else {
        for (int64_t r = r0 + warp; r < r1; r += kThreads / 32)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (col + i < batch) grad_x[r * batch + col + i] = v[i];
    }
}

}  // namespace dl

using namespace dl;

static int groupsum_check(const char *who, int64_t n, int64_t batch, int64_t k) {
    DL_REQUIRE(n >= 0 && batch >= 0 && k > 0, DL_ERR_INVALID_ARG, "%s: bad size (n=%lld batch=%lld k=%lld)", who,
               (long long)n, (long long)batch, (long long)k);
    DL_REQUIRE(n % k == 0, DL_ERR_NOT_DIVISIBLE, "%s: n (%lld) has to be divisible by k (%lld)", who, (long long)n, (long long)k);
    DL_REQUIRE(k <= 65535 && n / k <= INT32_MAX, DL_ERR_TOO_LARGE, "%s: k or rows per class too large", who);
    return DL_OK;
}

extern "C" DL_API size_t dl_groupsum_workspace_bytes(int64_t n, int64_t batch, int64_t k) {
    if (n <= 0 || batch <= 0 || k <= 0 || n % k != 0) return kGsCounterBytes;
    const int64_t chunks = groupsum_chunks(n, batch, k);
    if (chunks == 1) return kGsCounterBytes;  // one piece per class: no partial sums are stored
    return (size_t)kGsCounterBytes + (size_t)(k * chunks * batch) * sizeof(float);
}

extern "C" DL_API int dl_groupsum_f32(const float *x, float *out, void *workspace, int64_t n, int64_t batch, int64_t k, float tau,
                               void *stream) {
    if (int s = groupsum_check("dl_groupsum_f32", n, batch, k)) return s;
    if (batch == 0) return DL_OK;
    DL_REQUIRE(out && workspace && (x || n == 0), DL_ERR_INVALID_ARG, "dl_groupsum_f32: null pointer");
    DL_REQUIRE(aligned_to(workspace, 256), DL_ERR_INVALID_ARG, "dl_groupsum_f32: workspace must be 256-byte aligned");
    DL_REQUIRE(batch % 4 != 0 || aligned_to(x, 16), DL_ERR_INVALID_ARG, "dl_groupsum_f32: x must be 16-byte aligned");
    const int64_t chunks = groupsum_chunks(n, batch, k);
    const int64_t colblocks = ceil_div(batch, kGsCols);
    // Classes of up to 4096 rows: one cluster of 8 CTAs per (class, column block), no scratch needed.
    const int64_t m_rows = n / k;
    if (groupsum_takes_cluster_kernel(n, batch, k)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)colblocks, (unsigned)k, kGcCluster);
        cfg.blockDim = dim3(kGcThreads);
        cfg.stream = as_stream(stream);
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = kGcCluster;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        cudaLaunchKernelEx(&cfg, groupsum_cluster_kernel, x, out, batch, (int)k, (int)m_rows, tau);
        return launch_status("dl_groupsum_f32");
    }
    DL_REQUIRE(colblocks <= INT32_MAX && chunks <= 65535, DL_ERR_TOO_LARGE, "dl_groupsum_f32: batch too large");
    DL_REQUIRE(chunks == 1 || k * colblocks <= kGsMaxCounters, DL_ERR_TOO_LARGE,
               "dl_groupsum_f32: k * ceil(batch/128) = %lld exceeds %d", (long long)(k * colblocks), kGsMaxCounters);
    unsigned int *counters = reinterpret_cast<unsigned int *>(workspace);
    float *partial = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + kGsCounterBytes);
    const dim3 grid((unsigned)colblocks, (unsigned)k, (unsigned)chunks);
    groupsum_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(x, out, counters, partial, batch, (int)k, (int)(n / k),
                                                              (int)chunks, tau);
    return launch_status("dl_groupsum_f32");
}

extern "C" DL_API int dl_groupsum_backward_f32(const float *grad_out, float *grad_x, int64_t n, int64_t batch, int64_t k,
                                        float tau, void *stream) {
    if (int s = groupsum_check("dl_groupsum_backward_f32", n, batch, k)) return s;
    if (batch == 0 || n == 0) return DL_OK;
    DL_REQUIRE(grad_out && grad_x, DL_ERR_INVALID_ARG, "dl_groupsum_backward_f32: null pointer");
    DL_REQUIRE(batch % 4 != 0 || aligned_to(grad_x, 16), DL_ERR_INVALID_ARG,
               "dl_groupsum_backward_f32: grad_x must be 16-byte aligned");
    const int64_t m = n / k;
    const int64_t pieces = ceil_div(m, kGbkRows);
    const int64_t colblocks = ceil_div(batch, kGsCols);
    DL_REQUIRE(k * pieces <= INT32_MAX && colblocks <= 65535, DL_ERR_TOO_LARGE, "dl_groupsum_backward_f32: problem too large");
    launch_dependent(true, groupsum_backward_kernel<false>, dim3((unsigned)(k * pieces), (unsigned)colblocks), dim3(kThreads), 0,
                     as_stream(stream), grad_out, (const int64_t *)nullptr, (const float *)nullptr, grad_x, batch, (int)k, (int)m, tau,
                     (int)pieces);
    return launch_status("dl_groupsum_backward_f32");
}

// 1 when dl_groupsum_cross_entropy_f32 takes these sizes (classes of 64 .. 4096 rows), else 0.
extern "C" DL_API int dl_groupsum_cross_entropy_applicable(int64_t n, int64_t batch, int64_t k) {
    if (n <= 0 || batch <= 0 || k <= 0 || k > 65535 || n % k != 0) return 0;
    const int64_t m = n / k;
    return m >= 64 && m <= 4096 && ceil_div(batch, kGsCols) <= 65535 ? 1 : 0;
}

// counter: one uint32 on the device, zero before the first call; the kernel leaves it zero.
extern "C" DL_API int dl_groupsum_cross_entropy_f32(const float *x, const int64_t *target, float *scores, float *loss,
                                                    float *grad_classes, void *counter, int64_t n, int64_t batch, int64_t k, float tau,
                                                    void *stream) {
    if (int s = groupsum_check("dl_groupsum_cross_entropy_f32", n, batch, k)) return s;
    DL_REQUIRE(dl_groupsum_cross_entropy_applicable(n, batch, k) == 1, DL_ERR_INVALID_ARG,
               "dl_groupsum_cross_entropy_f32: classes of %lld rows are outside 64 .. 4096", (long long)(k > 0 ? n / k : 0));
    DL_REQUIRE(x && target && scores && loss && grad_classes && counter, DL_ERR_INVALID_ARG,
               "dl_groupsum_cross_entropy_f32: null pointer");
    DL_REQUIRE(batch % 4 != 0 || aligned_to(x, 16), DL_ERR_INVALID_ARG, "dl_groupsum_cross_entropy_f32: x must be 16-byte aligned");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(batch, kGsCols), (unsigned)k, kGcCluster);
    cfg.blockDim = dim3(kGcThreads);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = kGcCluster;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaLaunchKernelEx(&cfg, groupsum_ce_kernel, x, target, scores, loss, grad_classes, reinterpret_cast<unsigned int *>(counter), batch,
                       (int)k, (int)(n / k), tau);
    return launch_status("dl_groupsum_cross_entropy_f32");
}

// Head of a training step from per-CTA class sums (dl_forward_class_sums_f32): scores, loss, grad_classes as
// dl_groupsum_cross_entropy_f32 gives them.  rows_per_run: rows per CTA of the forward kernel, i.e.
// 2 * ceil(n / rows_per_run) == dl_forward_class_sums_rows(n, batch, k).  counter: one zeroed uint32, left zero.
extern "C" DL_API int dl_class_sums_cross_entropy_f32(const float *class_sums, const int64_t *target, float *scores, float *loss,
                                                      float *grad_classes, void *counter, int64_t n, int64_t batch, int64_t k,
                                                      int64_t rows_per_run, float tau, void *stream) {
    if (int s = groupsum_check("dl_class_sums_cross_entropy_f32", n, batch, k)) return s;
    DL_REQUIRE(n <= INT32_MAX, DL_ERR_TOO_LARGE, "dl_class_sums_cross_entropy_f32: more than 2^31 rows");
    DL_REQUIRE(n > 0 && batch > 0 && rows_per_run > 0 && n / k >= rows_per_run && rows_per_run <= INT32_MAX, DL_ERR_INVALID_ARG,
               "dl_class_sums_cross_entropy_f32: classes must be at least as long as a run of rows");
    DL_REQUIRE(class_sums && target && scores && loss && grad_classes && counter, DL_ERR_INVALID_ARG,
               "dl_class_sums_cross_entropy_f32: null pointer");
    const int64_t colblocks = ceil_div(batch, kGsCols);
    DL_REQUIRE(colblocks <= INT32_MAX && k <= 65535, DL_ERR_TOO_LARGE, "dl_class_sums_cross_entropy_f32: batch or k too large");
    constexpr int kSmallClasses = 16, kSmallPieces = 2;
    const size_t small_smem = (size_t)k * kCsGroups * kGsCols * sizeof(float);
    const int64_t pieces = ceil_div(n / k, rows_per_run) + 1;  // runs that can hold rows of one class
    if (colblocks == 1 && k <= kSmallClasses && pieces <= kSmallPieces * kCsGroups * kCsCluster) {
        // one cluster does it all, nothing but the results touches global memory
        auto kernel = class_sums_ce_cluster_kernel<kSmallClasses, kSmallPieces>;
        if (small_smem > 32 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)small_smem) != cudaSuccess)
            return launch_status("dl_class_sums_cross_entropy_f32 (shared memory opt-in)");
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kCsCluster);
        cfg.blockDim = dim3(kCsThreads);
        cfg.dynamicSmemBytes = small_smem;
        cfg.stream = as_stream(stream);
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kCsCluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        cudaLaunchKernelEx(&cfg, kernel, class_sums, target, scores, loss, grad_classes, batch, (int)k, (int)(n / k), (int)rows_per_run, tau);
        return launch_status("dl_class_sums_cross_entropy_f32");
    }
    launch_dependent(true, class_sums_ce_kernel, dim3((unsigned)colblocks, (unsigned)k), dim3(kCsThreads), 0, as_stream(stream), class_sums, target,
                     scores, loss, grad_classes, reinterpret_cast<unsigned int *>(counter), batch, (int)k, (int)(n / k), (int)rows_per_run,
                     tau);
    return launch_status("dl_class_sums_cross_entropy_f32");
}

// Backward of cross_entropy(GroupSum(x)) in one launch: dl_cross_entropy_backward_f32 followed by
// dl_groupsum_backward_f32 without the [batch][k] gradient in between.
extern "C" DL_API int dl_groupsum_cross_entropy_backward_f32(const float *probs, const int64_t *target, const float *grad_loss,
                                                             float *grad_x, int64_t n, int64_t batch, int64_t k, float tau,
                                                             void *stream) {
    if (int s = groupsum_check("dl_groupsum_cross_entropy_backward_f32", n, batch, k)) return s;
    if (batch == 0 || n == 0) return DL_OK;
    DL_REQUIRE(probs && target && grad_loss && grad_x, DL_ERR_INVALID_ARG, "dl_groupsum_cross_entropy_backward_f32: null pointer");
    DL_REQUIRE(batch % 4 != 0 || aligned_to(grad_x, 16), DL_ERR_INVALID_ARG,
               "dl_groupsum_cross_entropy_backward_f32: grad_x must be 16-byte aligned");
    const int64_t m = n / k;
    const int64_t pieces = ceil_div(m, kGbkRows);
    const int64_t colblocks = ceil_div(batch, kGsCols);
    DL_REQUIRE(k * pieces <= INT32_MAX && colblocks <= 65535, DL_ERR_TOO_LARGE,
               "dl_groupsum_cross_entropy_backward_f32: problem too large");
    launch_dependent(true, groupsum_backward_kernel<true>, dim3((unsigned)(k * pieces), (unsigned)colblocks), dim3(kThreads), 0,
                     as_stream(stream), probs, target, grad_loss, grad_x, batch, (int)k, (int)m, tau, (int)pieces);
    return launch_status("dl_groupsum_cross_entropy_backward_f32");
}

// ---------------------------------------------------------------------------------------------
// dl_groupsum_f32_static: the same forward GroupSum for callers that cannot hand over a workspace.
//
// Some callers of this library own no device allocator: a binding from another language that only
// passes through the input and output buffers its framework gave it, or a serving process whose
// memory pool was sized at start-up and is full.  dl_groupsum_f32 is closed to them because it needs
// caller-owned scratch.  This variant keeps that scratch in the library itself, in a fixed device
// array that exists once per GPU for as long as the library is loaded, so the call allocates nothing.
// The price is a size limit (kStaticScratchBytes) and that all calls on a GPU share the array.
// ---------------------------------------------------------------------------------------------
namespace dl {

constexpr size_t kStaticScratchBytes = 256u << 10;  // 256 KiB per GPU: counters + partial sums

static __device__ __align__(256) unsigned char g_groupsum_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void *g_scratch_ptr[kMaxDevices];  // device address of the array, per device; null until looked up

// Device address of this device's copy of the scratch array.  In host code the array's name is only a
// handle; the address a kernel can use has to be asked for, with the device current.
static int static_scratch(void **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return fail(DL_ERR_CUDA, "dl_groupsum_f32_static: cannot tell the current device");
    void *ptr = __atomic_load_n(&g_scratch_ptr[dev], __ATOMIC_ACQUIRE);
    if (ptr == nullptr) {
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_groupsum_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return fail(DL_ERR_CUDA, "dl_groupsum_f32_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        }
        __atomic_store_n(&g_scratch_ptr[dev], ptr, __ATOMIC_RELEASE);  // every thread would store the same value
    }
    *out = ptr;
    return DL_OK;
}

}  // namespace dl

extern "C" DL_API size_t dl_groupsum_static_limit_bytes(void) { return dl::kStaticScratchBytes; }

extern "C" DL_API int dl_groupsum_f32_static(const float *x, float *out, int64_t n, int64_t batch, int64_t k, float tau,
                                             void *stream) {
    if (int s = groupsum_check("dl_groupsum_f32_static", n, batch, k)) return s;
    if (batch == 0) return DL_OK;
    // Shapes that dl_groupsum_f32 sends to its cluster kernel use no scratch at all: no limit applies to them.
    const bool uses_scratch = !groupsum_takes_cluster_kernel(n, batch, k);
    const size_t need = dl_groupsum_workspace_bytes(n, batch, k);
    DL_REQUIRE(!uses_scratch || need <= kStaticScratchBytes, DL_ERR_TOO_LARGE,
               "dl_groupsum_f32_static: this shape needs %zu bytes of scratch, the built-in array holds %zu; "
               "use dl_groupsum_f32 with a workspace of your own",
               need, (size_t)kStaticScratchBytes);
    void *scratch = nullptr;
    if (int s = static_scratch(&scratch)) return s;
    // The array keeps whatever the previous call left.  The partial sums are overwritten before they are
    // read; the counters must start at zero, so they are cleared on the caller's stream first.
    if (uses_scratch && cudaMemsetAsync(scratch, 0, kGsCounterBytes, as_stream(stream)) != cudaSuccess)
        return launch_status("dl_groupsum_f32_static (clearing the counters)");
    return dl_groupsum_f32(x, out, scratch, n, batch, k, tau, stream);
}
