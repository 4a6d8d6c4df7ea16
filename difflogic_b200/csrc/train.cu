// Training kernels of the logic layer: forward, backward_w, backward_x (+ the backward plan).
//
// Activations are feature-major, x[n_in][batch] with the batch contiguous, so one neuron
// reads two whole input rows and writes one output row.  A row is covered by a group of G
// lanes (G a power of two <= 32, picked from the batch size) that each move 16 bytes
// (float4) per access; a CTA of 256 threads holds 256/G such groups.  When the batch is not
// a multiple of four floats, or a base pointer is not 16-byte aligned, the same kernels run
// with scalar accesses.  Columns are split into slabs of G vectors that are walked by
// blockIdx.y, so that all CTAs resident at one time work on the same few slabs and the
// gathered input rows of a slab stay in L2 for their second reader.
//
// No tensor cores: the work is a gather plus a handful of FMAs per element.
#include "adam_math.cuh"
#include "common.cuh"
#include "gates.cuh"

namespace dl {

template <bool VEC4>
struct Vec;
template <>
struct Vec<true> {
    using type = float4;
    static constexpr int width = 4;
};
template <>
struct Vec<false> {
    using type = float;
    static constexpr int width = 1;
};

__device__ __forceinline__ float4 ldv(const float4 *p) { return __ldg(p); }
__device__ __forceinline__ float ldv(const float *p) { return __ldg(p); }

// ---------------------------------------------------------------------------------------------
// forward:  y[j][:] = c0 + ca*x[a_j][:] + cb*x[b_j][:] + cab*x[a_j][:]*x[b_j][:]
// Set-up (before the grid dependency is waited for): connection indices into registers.  Then the
// row loads are issued and, while they are in flight, the four coefficients of each of the CTA's
// neurons are computed into shared memory.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void zero(float4 &v);
__device__ __forceinline__ void zero(float &v);
__device__ __forceinline__ void addv(float4 &acc, const float4 v) { acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w; }
__device__ __forceinline__ void addv(float &acc, const float v) { acc += v; }

// CLASSSUM: the layer's output feeds a GroupSum over classes of `class_rows` consecutive rows (the last layer of a
// network in training).  The rows are then not stored at all: every CTA adds up its NB rows per class -- at most two
// classes, class_rows >= NB -- in a fixed order and stores the sums as two rows of `y`, which then is
// [2 * gridDim.x][batch]: row 2*blockIdx.x for the class of the CTA's first neuron, row 2*blockIdx.x + 1 for the
// next class (zeros when the CTA does not reach it).  class_sums_ce_kernel (groupsum.cu) adds the pieces up.
template <int G, int U, bool VEC4, bool CLASSSUM>
__global__ void __launch_bounds__(kThreads, 4)
forward_kernel(const float *__restrict__ x, const int64_t *__restrict__ a, const int64_t *__restrict__ b,
               const float *__restrict__ w, int w_mode, float *__restrict__ y, float4 *__restrict__ coef_out,
               int64_t n_out, int64_t batch, int64_t ncols, int64_t nslabs, int64_t class_rows) {
    using V = typename Vec<VEC4>::type;
    constexpr int R = kThreads / G;  // neurons per pass
    constexpr int NB = R * U;        // neurons per CTA
    __shared__ float4 s_coef[NB];
    __shared__ V s_acc[CLASSSUM ? 2 * kThreads : 1];  // [class 0 | class 1][row group][lane]

    const int tid = threadIdx.x;
    const int lane = tid % G;
    const int r0 = tid / G;
    const int64_t n0 = (int64_t)blockIdx.x * NB;

    int64_t offa[U], offb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t j = n0 + r0 + u * R;
        if (j < n_out) {
            offa[u] = __ldg(a + j) * batch;
            offb[u] = __ldg(b + j) * batch;
        }
    }
    // the neurons' weights are pulled towards L2 meanwhile (after an L2-cold start they come from DRAM)
    if (tid < NB && n0 + tid < n_out) prefetch_l2(w + (n0 + tid) * 16);
    // Only the connection indices (fixed at construction) are read before this point: the weights may have
    // been written by the kernel just before this one (an optimizer step), the input certainly was.
    grid_dependency_wait();
    grid_dependents_launch();

    bool first = true;
    for (int64_t slab = blockIdx.y; slab < nslabs; slab += gridDim.y) {
        const int64_t col = slab * G + lane;
        const bool incol = col < ncols;
        const int64_t off = col * Vec<VEC4>::width;
        V va[U], vb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (incol && n0 + r0 + u * R < n_out) {
                va[u] = ldv(reinterpret_cast<const V *>(x + offa[u] + off));
                vb[u] = ldv(reinterpret_cast<const V *>(x + offb[u] + off));
            }
        }
        if (first) {
            // coefficients of the CTA's neurons, computed while the row loads are in flight
            for (int t = tid; t < NB * 4; t += kThreads) {  // NB*4 is a multiple of 32: whole warps iterate together
                const int nl = t >> 2, q = t & 3;
                const int64_t j = n0 + nl;
                const float4 c = quad_coef(w + j * 16 + q * 4, j < n_out, q, w_mode);
                if (q == 0 && j < n_out) {
                    s_coef[nl] = c;
                    if (coef_out != nullptr && blockIdx.y == 0) coef_out[j] = c;
                }
            }
            __syncthreads();
            first = false;
        }
        if (!CLASSSUM) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int r = r0 + u * R;
                if (incol && n0 + r < n_out)
                    *reinterpret_cast<V *>(y + (n0 + r) * batch + off) = mixv(s_coef[r], va[u], vb[u]);
            }
        } else {
            // rows below `border` belong to the class of the CTA's first neuron, the others to the next class
            const int64_t border = (n0 / class_rows + 1) * class_rows;
            V acc0, acc1;
            zero(acc0);
            zero(acc1);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int r = r0 + u * R;
                if (incol && n0 + r < n_out) {
                    const V val = mixv(s_coef[r], va[u], vb[u]);
                    if (n0 + r < border)
                        addv(acc0, val);
                    else
                        addv(acc1, val);
                }
            }
            s_acc[tid] = acc0;
            s_acc[kThreads + tid] = acc1;
            __syncthreads();
            if (tid < 2 * G) {  // one thread per (class, lane): the R row groups in a fixed order
                const int e = tid / G, l = tid % G;
                V sum;
                zero(sum);
#pragma unroll
                for (int rr = 0; rr < R; ++rr) addv(sum, s_acc[e * kThreads + rr * G + l]);
                const int64_t c = slab * G + l;
                if (c < ncols) *reinterpret_cast<V *>(y + (2 * (int64_t)blockIdx.x + e) * batch + c * Vec<VEC4>::width) = sum;
            }
            __syncthreads();  // the sums are read before the next slab overwrites them
        }
    }
}

// ---------------------------------------------------------------------------------------------
// backward_w: four batch sums per neuron, reduced over the G lanes of its group by shuffles,
// expanded to the 16 gate gradients and (DL_W_LOGITS) pushed through the softmax in place.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void acc4(float &s0, float &sa, float &sb, float &sab, float4 va, float4 vb, float4 g) {
    s0 += (g.x + g.y) + (g.z + g.w);
    sa += (va.x * g.x + va.y * g.y) + (va.z * g.z + va.w * g.w);
    sb += (vb.x * g.x + vb.y * g.y) + (vb.z * g.z + vb.w * g.w);
    sab += (va.x * vb.x * g.x + va.y * vb.y * g.y) + (va.z * vb.z * g.z + va.w * vb.w * g.w);
}
__device__ __forceinline__ void acc4(float &s0, float &sa, float &sb, float &sab, float va, float vb, float g) {
    s0 += g;
    sa += va * g;
    sb += vb * g;
    sab += va * vb * g;
}

// Optional Adam step in the epilogue of backward_w: a neuron's 16 gradients never leave the registers.  m, v: the
// layer's slices of the moments; state: two ints of this LAYER, {steps done, ticket}: every block reads the count when it
// starts, the last block to finish advances it -- no other kernel touches them, so no kernel has to run in between.
// m == nullptr: off.
struct AdamInBackward {
    float *m, *v;
    int *state;
    float lr, beta1, beta2, eps, grad_scale;
};

// Optional announcement in the epilogue of backward_w (batch-sharded training over peer memory, exchange.cu): when the
// last block of the last backward_w kernel of a gradient bucket is through, it stores the bucket's next epoch into
// every rank's flag words, so the peers learn that this rank's gradients are complete without another launch.
// block_ticket: one int per parameter (zero at rest); kernel_count: one int per bucket (zero at rest), counts the
// backward_w kernels of the bucket that are through; world == 0: off.
struct AnnounceGradients {
    int *flags[16];        // flag words of every rank (index = rank), own entry included
    int world, word;       // number of ranks; index of this rank's "gradients complete" word of the bucket
    const int *epoch_src;  // steps the bucket has done so far: the epoch announced is that + 1
    int *block_ticket, *kernel_count;
    int kernels;           // backward_w kernels per step that write into the bucket
};

// Optional push in the epilogue of backward_w (batch-sharded training, the packet form of the exchange, exchange.cu):
// every gradient that belongs to ANOTHER rank's slice of the bucket goes straight from the registers into that rank's
// inbox, as an 8-byte packet {value, step number} -- one store over NVLink, no fence, no flag -- while the kernel is still
// working on its other neurons; the exchange kernel that follows then has nothing to push.  The gradient is stored
// locally as well (grad_w): the owner of a slice reads its own part from there.  world <= 1: off.
struct PushGradients {
    unsigned long long *inbox[16];  // gradient inbox of every rank (index = rank)
    int rank, world;
    int per4;                       // float4 per slice of the bucket: ceil(float4 of the bucket / world)
    int base4;                      // float4 of the bucket in front of this layer's gradients
    long long region;               // first float4 slot of this bucket in THIS rank's region of an inbox
    long long half;                 // u64 between the two planes of an inbox
    const int *epoch_src;           // steps the bucket has done so far: the packets carry that + 1
};

// Row of grad_y that holds the gradient of output row j.  gy_group == 1: its own row.  gy_group == g > 1: the layer's
// outputs are summed in classes of g consecutive rows (GroupSum) and grad_y has one row per CLASS -- the gradient of
// every row of a class is the same, so it is not expanded to [n_out][batch] in memory.
__device__ __forceinline__ int64_t gy_row(int64_t j, int gy_group) {
    return gy_group == 1 ? j : (int64_t)((int)j / gy_group);
}

template <int G, bool VEC4>
__global__ void __launch_bounds__(kThreads)
backward_w_kernel(const float *__restrict__ x, const int64_t *__restrict__ a, const int64_t *__restrict__ b,
                  const float *__restrict__ gy, const float *w, int w_mode, float *__restrict__ grad_w,
                  int64_t n_out, int64_t batch, int64_t ncols, int gy_group, AdamInBackward adam, AnnounceGradients ann,
                  PushGradients push) {
    using V = typename Vec<VEC4>::type;
    constexpr int R = kThreads / G;
    __shared__ float s_step_size, s_bc2_sqrt;
    // The 16 gates of the neuron are shared by P lanes of its group, K gates each.
    constexpr int P = G < 16 ? G : 16;
    constexpr int K = 16 / P;
    const int tid = threadIdx.x;
    const int lane = tid % G;
    const int gl = lane & (P - 1);
    const int64_t j = (int64_t)blockIdx.x * R + tid / G;
    const bool active = j < n_out;

    // ---- set-up: the connection indices are fixed at construction
    int64_t ia = 0, ib = 0;
    if (active) {
        ia = __ldg(a + j) * batch;
        ib = __ldg(b + j) * batch;
        if (w_mode == DL_W_LOGITS && lane == 0) prefetch_l2(w + j * 16);
    }
    // Adam in the epilogue (adam.m != nullptr): the moments of this neuron's 16 weights are only ever touched by
    // this kernel, one step apart, so they are fetched here, before the wait; the bias corrections likewise.
    float mom1[K], mom2[K];
    if (adam.m != nullptr) {
        if (tid == 0) {
            const float t = (float)(adam.state[0] + 1);
            s_step_size = adam.lr / (1.f - powf(adam.beta1, t));
            s_bc2_sqrt = sqrtf(1.f - powf(adam.beta2, t));
        }
#pragma unroll
        for (int q = 0; q < K; ++q) {
            mom1[q] = (active && lane < P) ? adam.m[j * 16 + gl + q * P] : 0.f;
            mom2[q] = (active && lane < P) ? adam.v[j * 16 + gl + q * P] : 0.f;
        }
        __syncthreads();
    }
    grid_dependency_wait();      // weights, x and grad_y may have been written by the kernels just before
    grid_dependents_launch();

    float prob[K], raw[K];
    if (w_mode == DL_W_LOGITS) {
#pragma unroll
        for (int q = 0; q < K; ++q) raw[q] = prob[q] = active ? w[j * 16 + gl + q * P] : 0.f;
    }

    float s0 = 0.f, sa = 0.f, sb = 0.f, sab = 0.f;
    if (active) {
        const V *xa = reinterpret_cast<const V *>(x + ia);
        const V *xb = reinterpret_cast<const V *>(x + ib);
        const V *g = reinterpret_cast<const V *>(gy + gy_row(j, gy_group) * batch);
#pragma unroll 4
        for (int64_t col = lane; col < ncols; col += G) acc4(s0, sa, sb, sab, ldv(xa + col), ldv(xb + col), ldv(g + col));
    }
#pragma unroll
    for (int off = G / 2; off > 0; off >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, off);
        sa += __shfl_xor_sync(0xffffffffu, sa, off);
        sb += __shfl_xor_sync(0xffffffffu, sb, off);
        sab += __shfl_xor_sync(0xffffffffu, sab, off);
    }

    float out[K];
#pragma unroll
    for (int q = 0; q < K; ++q) out[q] = gate_grad_from_sums(gl + q * P, s0, sa, sb, sab);
    if (w_mode == DL_W_LOGITS) {
        float m = -INFINITY;
#pragma unroll
        for (int q = 0; q < K; ++q) m = fmaxf(m, prob[q]);
#pragma unroll
        for (int off = P / 2; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < K; ++q) {
            prob[q] = expf(prob[q] - m);
            s += prob[q];
        }
#pragma unroll
        for (int off = P / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
#pragma unroll
        for (int q = 0; q < K; ++q) prob[q] = prob[q] / s;
        float dot = 0.f;
#pragma unroll
        for (int q = 0; q < K; ++q) dot += prob[q] * out[q];
#pragma unroll
        for (int off = P / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
#pragma unroll
        for (int q = 0; q < K; ++q) out[q] = prob[q] * (out[q] - dot);
    }
    if (active && lane < P) {
        if (grad_w != nullptr) {
#pragma unroll
            for (int q = 0; q < K; ++q) grad_w[j * 16 + gl + q * P] = out[q];
        }
        if (push.world > 1) {
            const unsigned long long e = (unsigned long long)(unsigned)(*push.epoch_src + 1) << 32;
#pragma unroll
            for (int q = 0; q < K; ++q) {
                const int f = (int)j * 16 + gl + q * P;      // float within the layer
                const int i = push.base4 + (f >> 2);         // float4 within the bucket
                const int owner = i / push.per4;
                if (owner != push.rank) {
                    unsigned long long *dst = push.inbox[owner] + (push.region + (i - owner * push.per4)) * 2 + (f & 1) +
                                              ((f >> 1) & 1) * push.half;
                    const unsigned long long packet = e | __float_as_uint(out[q]);
                    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(packet) : "memory");
                }
            }
        }
        if (adam.m != nullptr) {
            const AdamConsts consts = {1.f - adam.beta1, adam.beta2, 1.f - adam.beta2, s_step_size, s_bc2_sqrt, adam.eps};
            float *wp = const_cast<float *>(w);
#pragma unroll
            for (int q = 0; q < K; ++q) {
                float pw = raw[q];
                adam_update(pw, __fmul_rn(out[q], adam.grad_scale), mom1[q], mom2[q], consts);
                const int64_t at = j * 16 + gl + q * P;
                wp[at] = pw;
                adam.m[at] = mom1[q];
                adam.v[at] = mom2[q];
            }
        }
    }
    if (adam.m != nullptr && tid == 0) {
        // thread 0 of every block has read the step count at its start; the last one to get here advances it
        if (atomicAdd(adam.state + 1, 1) == (int)gridDim.x - 1) {
            adam.state[1] = 0;
            adam.state[0] = adam.state[0] + 1;
        }
    }
    if (ann.world > 0) {
        __syncthreads();  // every thread's gradient stores before thread 0's fence and its block's ticket
        if (tid == 0) __threadfence();
        if (tid == 0 && atomicAdd(ann.block_ticket, 1) == (int)gridDim.x - 1) {
            *ann.block_ticket = 0;
            if (atomicAdd(ann.kernel_count, 1) == ann.kernels - 1) {
                *ann.kernel_count = 0;
                __threadfence_system();  // the whole bucket's gradients before the flags, for observers on other GPUs
                const int epoch = *ann.epoch_src + 1;
                for (int p = 0; p < ann.world; ++p)
                    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(ann.flags[p] + ann.word), "r"(epoch) : "memory");
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// backward_x: each input row gathers from its consumers through the plan (no atomics).  The
// row's first two plan entries and their coefficients are fetched during set-up; with the usual
// fan-out of two nothing but the row loads is left once the previous kernel has finished.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void bx_acc(float4 &acc, float c1, float cab, float4 p, float4 g) {
    acc.x = fmaf(fmaf(cab, p.x, c1), g.x, acc.x);
    acc.y = fmaf(fmaf(cab, p.y, c1), g.y, acc.y);
    acc.z = fmaf(fmaf(cab, p.z, c1), g.z, acc.z);
    acc.w = fmaf(fmaf(cab, p.w, c1), g.w, acc.w);
}
__device__ __forceinline__ void bx_acc(float &acc, float c1, float cab, float p, float g) {
    acc = fmaf(fmaf(cab, p, c1), g, acc);
}
__device__ __forceinline__ float4 scaled(float4 v, float s) { return make_float4(v.x * s, v.y * s, v.z * s, v.w * s); }
__device__ __forceinline__ float scaled(float v, float s) { return v * s; }
__device__ __forceinline__ void zero(float4 &v) { v = make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ void zero(float &v) { v = 0.f; }

template <int G, bool VEC4>
__global__ void __launch_bounds__(kThreads)
backward_x_kernel(const float *__restrict__ x, const float4 *__restrict__ coef, const float *__restrict__ gy,
                  const int64_t *__restrict__ start, const int2 *__restrict__ plan, float scale,
                  float *__restrict__ gx, int64_t n_in, int64_t batch, int64_t ncols, int64_t nslabs, int gy_group) {
    using V = typename Vec<VEC4>::type;
    constexpr int R = kThreads / G;
    constexpr int C = 4;  // columns per lane within a slab: lane, lane+G, lane+2G, lane+3G
    const int tid = threadIdx.x;
    const int lane = tid % G;
    const int64_t i = (int64_t)blockIdx.x * R + tid / G;
    const bool active = i < n_in;

    // ---- set-up: the gather plan is fixed at construction
    int64_t e0 = 0, e1 = 0;
    int2 p0 = make_int2(0, 0), p1 = make_int2(0, 0);
    if (active) {
        e0 = __ldg(start + i);
        e1 = __ldg(start + i + 1);
        if (e0 < e1) p0 = __ldg(plan + e0);
        if (e0 + 1 < e1) p1 = __ldg(plan + e0 + 1);
    }
    grid_dependency_wait();      // coef (forward of this layer) and grad_y (previous kernel) are final from here on
    grid_dependents_launch();
    if (!active) return;
    float4 c0 = make_float4(0.f, 0.f, 0.f, 0.f), c1 = c0;
    if (e0 < e1) c0 = __ldg(coef + (p0.x >> 1));
    if (e0 + 1 < e1) c1 = __ldg(coef + (p1.x >> 1));
    const float k0 = (p0.x & 1) ? c0.z : c0.y, k1 = (p1.x & 1) ? c1.z : c1.y;
    const float *xp0 = x + (int64_t)p0.y * batch, *gp0 = gy + gy_row(p0.x >> 1, gy_group) * batch;
    const float *xp1 = x + (int64_t)p1.y * batch, *gp1 = gy + gy_row(p1.x >> 1, gy_group) * batch;
    const bool has0 = e0 < e1, has1 = e0 + 1 < e1;

    for (int64_t slab = blockIdx.y; slab < nslabs; slab += gridDim.y) {
#pragma unroll 2
        for (int cc = 0; cc < C; ++cc) {
            const int64_t col = slab * (G * C) + cc * G + lane;
            if (col >= ncols) break;
            const int64_t off = col * Vec<VEC4>::width;
            V acc;
            zero(acc);
            if (has1) {
                const V vp = ldv(reinterpret_cast<const V *>(xp0 + off));
                const V vg = ldv(reinterpret_cast<const V *>(gp0 + off));
                const V vp1 = ldv(reinterpret_cast<const V *>(xp1 + off));
                const V vg1 = ldv(reinterpret_cast<const V *>(gp1 + off));
                bx_acc(acc, k0, c0.w, vp, vg);
                bx_acc(acc, k1, c1.w, vp1, vg1);
            } else if (has0) {
                bx_acc(acc, k0, c0.w, ldv(reinterpret_cast<const V *>(xp0 + off)), ldv(reinterpret_cast<const V *>(gp0 + off)));
            }
            for (int64_t e = e0 + 2; e < e1; ++e) {
                const int2 p = __ldg(plan + e);
                const int64_t j = p.x >> 1;
                const float4 c = __ldg(coef + j);
                const V vp = ldv(reinterpret_cast<const V *>(x + (int64_t)p.y * batch + off));
                const V vg = ldv(reinterpret_cast<const V *>(gy + gy_row(j, gy_group) * batch + off));
                bx_acc(acc, (p.x & 1) ? c.z : c.y, c.w, vp, vg);
            }
            *reinterpret_cast<V *>(gx + i * batch + off) = scaled(acc, scale);
        }
    }
}

// y[c][r] = x[r][c]: the batch-major input of a network -> the feature-major layout of the layer kernels, 32 x 32 tiles
// through shared memory.  The kernel that follows may begin its set-up at once (it reads y only after its own dependency
// wait, i.e. after this grid has finished).
__global__ void __launch_bounds__(kThreads)
transpose_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t rows, int64_t cols) {
    __shared__ float tile[32][33];
    grid_dependents_launch();
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
#pragma unroll
    for (int i = 0; i < 32; i += kThreads / 32) {
        const int64_t r = r0 + ty + i, c = c0 + tx;
        if (r < rows && c < cols) tile[ty + i][tx] = x[r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 32; i += kThreads / 32) {
        const int64_t c = c0 + ty + i, r = r0 + tx;
        if (r < rows && c < cols) y[c * rows + r] = tile[tx][ty + i];
    }
}

__global__ void __launch_bounds__(kThreads)
build_plan_kernel(const int64_t *__restrict__ a, const int64_t *__restrict__ b, const int64_t *__restrict__ start,
                  const int64_t *__restrict__ list, int2 *__restrict__ plan, int64_t n_in) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n_in) return;
    const int64_t e0 = start[i], e1 = start[i + 1];
    for (int64_t e = e0; e < e1; ++e) {
        const int64_t j = list[e];
        // A neuron whose inputs are both row i is listed twice in a row: first entry is its
        // a-slot, second its b-slot.
        const bool second = e > e0 && list[e - 1] == j;
        const int slot = second ? 1 : (a[j] == i ? 0 : 1);
        const int64_t partner = slot ? a[j] : b[j];
        plan[e] = make_int2((int)(2 * j + slot), (int)partner);
    }
}

// Every kernel of this library trusts a layer's index arrays: they are fixed when the layer is built, so they are checked
// once, there, instead of on every access.  report: {code, where, value, limit}; the first violation found wins (atomicCAS
// on the code), nothing is accessed through a bad index.  Codes: 1 a[j] or b[j] outside [0, n_in); 2 start[] not
// 0 = start[0] <= ... <= start[n_in] = 2 n_out; 3 list entry outside [0, n_out); 4 plan entry outside its range;
// 5 plan entry does not match the connections (the neuron's input in that slot is not the row that lists it, or the
// partner row is not the neuron's other input).
__device__ __forceinline__ void report_violation(int64_t *report, int64_t code, int64_t where, int64_t value, int64_t limit) {
    if (atomicCAS(reinterpret_cast<unsigned long long *>(report), 0ull, (unsigned long long)code) == 0ull) {
        report[1] = where;
        report[2] = value;
        report[3] = limit;
    }
}

__global__ void __launch_bounds__(kThreads)
check_connections_kernel(const int64_t *__restrict__ a, const int64_t *__restrict__ b, const int64_t *__restrict__ start,
                         const int64_t *__restrict__ list, const int2 *__restrict__ plan, int64_t n_in, int64_t n_out,
                         int64_t *__restrict__ report, int phase) {
    // One launch per phase, in the order of the codes, each phase only when the ones before found nothing: what is
    // reported is the violation with the lowest code, and a later phase may rely on what the earlier ones established.
    if (*reinterpret_cast<volatile int64_t *>(report) != 0) return;
    if (phase == 1) start = nullptr, list = nullptr, plan = nullptr;
    if (phase == 2) list = nullptr, plan = nullptr;
    if (phase == 3) start = nullptr, plan = nullptr;
    if (phase == 4) list = nullptr;
    const bool connections = phase == 1, offsets = phase == 2;
    const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (connections && t < n_out) {
        if (a[t] < 0 || a[t] >= n_in) report_violation(report, 1, t, a[t], n_in);
        if (b[t] < 0 || b[t] >= n_in) report_violation(report, 1, t, b[t], n_in);
    }
    if (offsets && start != nullptr && t <= n_in) {
        const int64_t v = start[t];
        if (v < 0 || v > 2 * n_out || (t == 0 && v != 0) || (t == n_in && v != 2 * n_out) || (t > 0 && start[t - 1] > v))
            report_violation(report, 2, t, v, 2 * n_out);
    }
    if (list != nullptr && t < 2 * n_out && (list[t] < 0 || list[t] >= n_out)) report_violation(report, 3, t, list[t], n_out);
    if (plan != nullptr && start != nullptr && t < n_in) {
        // the entries of input row t, as far as start[] can be trusted
        const int64_t e0 = start[t], e1 = start[t + 1];
        if (e0 >= 0 && e0 <= e1 && e1 <= 2 * n_out) {
            for (int64_t e = e0; e < e1; ++e) {
                const int2 p = plan[e];
                const int64_t j = p.x >> 1;
                const int slot = p.x & 1;
                if (p.x < 0 || j >= n_out || p.y < 0 || p.y >= n_in) {
                    report_violation(report, 4, e, p.x < 0 || j >= n_out ? p.x : p.y, p.x < 0 || j >= n_out ? 2 * n_out : n_in);
                } else {
                    const int64_t mine = slot ? b[j] : a[j], other = slot ? a[j] : b[j];
                    if (mine != t || other != p.y) report_violation(report, 5, e, j, t);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static inline unsigned slab_grid(int64_t nslabs) { return (unsigned)(nslabs < 65535 ? nslabs : 65535); }

constexpr int kForwardU = 4;  // passes of a CTA of the forward kernel over its row groups
static inline int64_t forward_rows_per_cta(int G) { return (kThreads / G) * kForwardU; }

template <bool VEC4, bool CLASSSUM = false>
static int launch_forward(bool overlap, int G, const float *x, const int64_t *a, const int64_t *b, const float *w, int w_mode, float *y,
                          float *coef, int64_t n_out, int64_t batch, int64_t ncols, cudaStream_t st, int64_t class_rows = 0) {
    constexpr int U = kForwardU;
    const int64_t nslabs = ceil_div(ncols, G);
    const int64_t nb = forward_rows_per_cta(G);
    const dim3 grid((unsigned)ceil_div(n_out, nb), slab_grid(nslabs));
    float4 *c4 = reinterpret_cast<float4 *>(coef);
#define DL_FWD(GG)                                                                                              \
    case GG:                                                                                                    \
        launch_dependent(overlap, forward_kernel<GG, U, VEC4, CLASSSUM>, grid, dim3(kThreads), 0, st, x, a, b, w, w_mode, y, c4, n_out, batch, ncols, nslabs, class_rows); \
        break;
    switch (G) {
        DL_FWD(1) DL_FWD(2) DL_FWD(4) DL_FWD(8) DL_FWD(16) DL_FWD(32)
    }
#undef DL_FWD
    return launch_status("dl_forward_f32");
}

template <bool VEC4>
static int launch_backward_w(bool overlap, int G, const float *x, const int64_t *a, const int64_t *b, const float *gy, const float *w,
                             int w_mode, float *grad_w, int64_t n_out, int64_t batch, int64_t ncols, int gy_group,
                             const AdamInBackward &adam, const AnnounceGradients &ann, const PushGradients &push, cudaStream_t st) {
    const unsigned grid = (unsigned)ceil_div(n_out, kThreads / G);
#define DL_BW(GG)                                                                                          \
    case GG:                                                                                               \
        launch_dependent(overlap, backward_w_kernel<GG, VEC4>, dim3(grid), dim3(kThreads), 0, st, x, a, b, gy, w, w_mode, grad_w, n_out, batch, ncols, gy_group, adam, ann, push); \
        break;
    switch (G) {
        DL_BW(1) DL_BW(2) DL_BW(4) DL_BW(8) DL_BW(16) DL_BW(32)
    }
#undef DL_BW
    return launch_status("dl_backward_w_f32");
}

template <bool VEC4>
static int launch_backward_x(bool overlap, int G, const float *x, const float *coef, const float *gy, const int64_t *start,
                             const int32_t *plan, float scale, float *gx, int64_t n_in, int64_t batch, int64_t ncols, int gy_group,
                             cudaStream_t st) {
    const int64_t nslabs = ceil_div(ncols, G * 4);
    const dim3 grid((unsigned)ceil_div(n_in, kThreads / G), slab_grid(nslabs));
    const float4 *c4 = reinterpret_cast<const float4 *>(coef);
    const int2 *p2 = reinterpret_cast<const int2 *>(plan);
#define DL_BX(GG)                                                                                               \
    case GG:                                                                                                    \
        launch_dependent(overlap, backward_x_kernel<GG, VEC4>, grid, dim3(kThreads), 0, st, x, c4, gy, start, p2, scale, gx, n_in, batch, ncols, nslabs, gy_group); \
        break;
    switch (G) {
        DL_BX(1) DL_BX(2) DL_BX(4) DL_BX(8) DL_BX(16) DL_BX(32)
    }
#undef DL_BX
    return launch_status("dl_backward_x_f32");
}

bool forward_tma_applicable(const float *x, const float *y, int64_t n_out, int64_t batch);  // forward_tma.cu
int launch_forward_tma(bool overlap, const float *x, const int64_t *a, const int64_t *b, const float *w, int w_mode, float *y,
                       float *coef, int64_t n_out, int64_t batch, cudaStream_t st);

}  // namespace dl

using namespace dl;

static const int64_t kMaxRows = (int64_t)1 << 30;  // plan entries hold 2*j+slot in an int32

extern "C" DL_API int dl_forward_f32(const float *x, const int64_t *a, const int64_t *b, const float *w, int w_mode, float *y,
                              float *coef, int64_t n_in, int64_t n_out, int64_t batch, int flags, void *stream) {
    DL_REQUIRE(n_in >= 0 && n_out >= 0 && batch >= 0, DL_ERR_INVALID_ARG, "dl_forward_f32: negative size");
    DL_REQUIRE(w_mode >= DL_W_LOGITS && w_mode <= DL_W_ARGMAX, DL_ERR_INVALID_ARG, "dl_forward_f32: unknown w_mode %d", w_mode);
    if (n_out == 0 || batch == 0) return DL_OK;
    DL_REQUIRE(x && a && b && w && y, DL_ERR_INVALID_ARG, "dl_forward_f32: null pointer");
    DL_REQUIRE(n_in > 0, DL_ERR_INVALID_ARG, "dl_forward_f32: n_in is 0 but n_out is %lld", (long long)n_out);
    DL_REQUIRE(coef == nullptr || aligned_to(coef, 16), DL_ERR_INVALID_ARG, "dl_forward_f32: coef must be 16-byte aligned");
    const bool vec = batch % 4 == 0 && aligned_to(x, 16) && aligned_to(y, 16);
    const int64_t ncols = vec ? batch / 4 : batch;
    const int G = pow2_at_least(ncols, 32);
    const bool overlap = (flags & DL_LAUNCH_OVERLAP_SETUP) != 0;
    if (forward_tma_applicable(x, y, n_out, batch))   // long rows: gathered rows staged in shared memory by bulk copies
        return launch_forward_tma(overlap, x, a, b, w, w_mode, y, coef, n_out, batch, as_stream(stream));
    return vec ? launch_forward<true>(overlap, G, x, a, b, w, w_mode, y, coef, n_out, batch, ncols, as_stream(stream))
               : launch_forward<false>(overlap, G, x, a, b, w, w_mode, y, coef, n_out, batch, ncols, as_stream(stream));
}

// Geometry of the class-sum form of the forward kernel for a batch: the lane group G, rows per CTA and whether rows are
// moved as float4 (decided from the batch alone; the pointers must then be 16-byte aligned).
static void forward_class_geometry(int64_t batch, int *G, int64_t *rows_per_cta, bool *vec) {
    *vec = batch % 4 == 0;
    const int64_t ncols = *vec ? batch / 4 : batch;
    *G = pow2_at_least(ncols, 32);
    *rows_per_cta = forward_rows_per_cta(*G);
}

// Rows of the `class_sums` buffer that dl_forward_class_sums_f32 writes: two per CTA (0 when the sizes are outside the
// kernel's range: classes must be at least as long as a CTA's run of rows).
extern "C" DL_API int64_t dl_forward_class_sums_rows(int64_t n_out, int64_t batch, int64_t k) {
    if (n_out <= 0 || batch <= 0 || k <= 0 || n_out % k != 0) return 0;
    int G;
    int64_t nb;
    bool vec;
    forward_class_geometry(batch, &G, &nb, &vec);
    if (n_out / k < nb) return 0;
    return 2 * ceil_div(n_out, nb);
}

// Rows per run (= per CTA of the forward kernel) at this batch size.
extern "C" DL_API int64_t dl_forward_class_sums_run(int64_t batch) {
    if (batch <= 0) return 0;
    int G;
    int64_t nb;
    bool vec;
    forward_class_geometry(batch, &G, &nb, &vec);
    return nb;
}

// Forward of a layer whose output goes into GroupSum(k): instead of y [n_out][batch], per-CTA class sums
// class_sums [dl_forward_class_sums_rows()][batch] are written (see forward_kernel).
extern "C" DL_API int dl_forward_class_sums_f32(const float *x, const int64_t *a, const int64_t *b, const float *w, int w_mode,
                                                float *class_sums, float *coef, int64_t n_in, int64_t n_out, int64_t batch, int64_t k,
                                                int flags, void *stream) {
    DL_REQUIRE(n_in > 0 && n_out > 0 && batch > 0 && k > 0, DL_ERR_INVALID_ARG, "dl_forward_class_sums_f32: sizes must be positive");
    DL_REQUIRE(n_out % k == 0, DL_ERR_NOT_DIVISIBLE, "dl_forward_class_sums_f32: n_out (%lld) has to be divisible by k (%lld)",
               (long long)n_out, (long long)k);
    DL_REQUIRE(w_mode >= DL_W_LOGITS && w_mode <= DL_W_ARGMAX, DL_ERR_INVALID_ARG, "dl_forward_class_sums_f32: unknown w_mode %d", w_mode);
    DL_REQUIRE(x && a && b && w && class_sums, DL_ERR_INVALID_ARG, "dl_forward_class_sums_f32: null pointer");
    DL_REQUIRE(dl_forward_class_sums_rows(n_out, batch, k) > 0, DL_ERR_INVALID_ARG,
               "dl_forward_class_sums_f32: classes of %lld rows are shorter than a CTA's run of rows", (long long)(n_out / k));
    DL_REQUIRE(coef == nullptr || aligned_to(coef, 16), DL_ERR_INVALID_ARG, "dl_forward_class_sums_f32: coef must be 16-byte aligned");
    int G;
    int64_t nb;
    bool vec;
    forward_class_geometry(batch, &G, &nb, &vec);
    DL_REQUIRE(!vec || (aligned_to(x, 16) && aligned_to(class_sums, 16)), DL_ERR_INVALID_ARG,
               "dl_forward_class_sums_f32: x and class_sums must be 16-byte aligned");
    const int64_t ncols = vec ? batch / 4 : batch;
    const bool overlap = (flags & DL_LAUNCH_OVERLAP_SETUP) != 0;
    return vec ? launch_forward<true, true>(overlap, G, x, a, b, w, w_mode, class_sums, coef, n_out, batch, ncols, as_stream(stream), n_out / k)
               : launch_forward<false, true>(overlap, G, x, a, b, w, w_mode, class_sums, coef, n_out, batch, ncols, as_stream(stream), n_out / k);
}

static int backward_w_entry(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, const float *w, int w_mode,
                            float *grad_w, int64_t n_in, int64_t n_out, int64_t batch, int64_t gy_group, int flags, void *stream,
                            const AdamInBackward &adam = AdamInBackward{nullptr, nullptr, nullptr, 0.f, 0.f, 0.f, 0.f, 0.f},
                            const AnnounceGradients &ann = AnnounceGradients{}, const PushGradients &push = PushGradients{}) {
    DL_REQUIRE(gy_group >= 1 && gy_group <= INT32_MAX && n_out % gy_group == 0, DL_ERR_INVALID_ARG,
               "dl_backward_w_f32: n_out (%lld) is not a multiple of the rows per class (%lld)", (long long)n_out, (long long)gy_group);
    DL_REQUIRE(n_in >= 0 && n_out >= 0 && batch >= 0, DL_ERR_INVALID_ARG, "dl_backward_w_f32: negative size");
    DL_REQUIRE(w_mode == DL_W_LOGITS || w_mode == DL_W_PROBS, DL_ERR_INVALID_ARG,
               "dl_backward_w_f32: w_mode must be DL_W_LOGITS or DL_W_PROBS, got %d", w_mode);
    if (n_out == 0) return DL_OK;
    DL_REQUIRE(a && b && (grad_w || adam.m), DL_ERR_INVALID_ARG, "dl_backward_w_f32: null pointer");
    DL_REQUIRE(batch == 0 || (x && grad_y), DL_ERR_INVALID_ARG, "dl_backward_w_f32: null pointer");
    DL_REQUIRE(w_mode != DL_W_LOGITS || w, DL_ERR_INVALID_ARG, "dl_backward_w_f32: DL_W_LOGITS needs the raw weights");
    const bool vec = batch % 4 == 0 && aligned_to(x, 16) && aligned_to(grad_y, 16);
    const int64_t ncols = vec ? batch / 4 : batch;
    const int G = pow2_at_least(ceil_div(ncols, 4), 32);
    const bool overlap = (flags & DL_LAUNCH_OVERLAP_SETUP) != 0;
    return vec ? launch_backward_w<true>(overlap, G, x, a, b, grad_y, w, w_mode, grad_w, n_out, batch, ncols, (int)gy_group, adam, ann, push, as_stream(stream))
               : launch_backward_w<false>(overlap, G, x, a, b, grad_y, w, w_mode, grad_w, n_out, batch, ncols, (int)gy_group, adam, ann, push, as_stream(stream));
}

extern "C" DL_API int dl_backward_w_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, const float *w,
                                 int w_mode, float *grad_w, int64_t n_in, int64_t n_out, int64_t batch, int flags, void *stream) {
    return backward_w_entry(x, a, b, grad_y, w, w_mode, grad_w, n_in, n_out, batch, 1, flags, stream);
}

// grad_y has one row per class of `rows_per_class` consecutive outputs ([n_out / rows_per_class][batch]).
extern "C" DL_API int dl_backward_w_classes_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y_classes,
                                                const float *w, int w_mode, float *grad_w, int64_t n_in, int64_t n_out, int64_t batch,
                                                int64_t rows_per_class, int flags, void *stream) {
    return backward_w_entry(x, a, b, grad_y_classes, w, w_mode, grad_w, n_in, n_out, batch, rows_per_class, flags, stream);
}

static int backward_x_entry(const float *x, const float *coef, const float *grad_y, const int64_t *start, const int32_t *plan,
                            float grad_scale, float *grad_x, int64_t n_in, int64_t n_out, int64_t batch, int64_t gy_group, int flags,
                            void *stream) {
    DL_REQUIRE(gy_group >= 1 && gy_group <= INT32_MAX && n_out % gy_group == 0, DL_ERR_INVALID_ARG,
               "dl_backward_x_f32: n_out (%lld) is not a multiple of the rows per class (%lld)", (long long)n_out, (long long)gy_group);
    DL_REQUIRE(n_in >= 0 && n_out >= 0 && batch >= 0, DL_ERR_INVALID_ARG, "dl_backward_x_f32: negative size");
    DL_REQUIRE(n_out < kMaxRows && n_in < 2 * kMaxRows, DL_ERR_TOO_LARGE, "dl_backward_x_f32: more than 2^30 neurons");
    if (n_in == 0 || batch == 0) return DL_OK;
    DL_REQUIRE(x && grad_x && start, DL_ERR_INVALID_ARG, "dl_backward_x_f32: null pointer");
    DL_REQUIRE(n_out == 0 || (coef && grad_y && plan), DL_ERR_INVALID_ARG, "dl_backward_x_f32: null pointer");
    DL_REQUIRE(aligned_to(coef, 16) && aligned_to(plan, 8), DL_ERR_INVALID_ARG,
               "dl_backward_x_f32: coef must be 16-byte and plan 8-byte aligned");
    const bool vec = batch % 4 == 0 && aligned_to(x, 16) && aligned_to(grad_y, 16) && aligned_to(grad_x, 16);
    const int64_t ncols = vec ? batch / 4 : batch;
    const int G = pow2_at_least(ceil_div(ncols, 4), 32);
    const bool overlap = (flags & DL_LAUNCH_OVERLAP_SETUP) != 0;
    return vec ? launch_backward_x<true>(overlap, G, x, coef, grad_y, start, plan, grad_scale, grad_x, n_in, batch, ncols, (int)gy_group, as_stream(stream))
               : launch_backward_x<false>(overlap, G, x, coef, grad_y, start, plan, grad_scale, grad_x, n_in, batch, ncols, (int)gy_group, as_stream(stream));
}

// backward_w with the Adam step of the layer's weights in its epilogue: w [n_out][16] is UPDATED in place with the
// layer's slices of the moments; grad_w may be null (the gradient is then not stored at all).  state: this layer's own
// {steps done, ticket} pair on the device; the kernel uses steps done + 1 and advances it when it is through.
extern "C" DL_API int dl_backward_w_adam_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, float *w,
                                             float *exp_avg, float *exp_avg_sq, float *grad_w, int64_t n_in, int64_t n_out, int64_t batch,
                                             int64_t rows_per_class, float lr, float beta1, float beta2, float eps, float grad_scale,
                                             int32_t *state, int flags, void *stream) {
    DL_REQUIRE(n_out == 0 || (w && exp_avg && exp_avg_sq && state), DL_ERR_INVALID_ARG, "dl_backward_w_adam_f32: null pointer");
    const AdamInBackward adam = {exp_avg, exp_avg_sq, reinterpret_cast<int *>(state), lr, beta1, beta2, eps, grad_scale};
    return backward_w_entry(x, a, b, grad_y, w, DL_W_LOGITS, grad_w, n_in, n_out, batch, rows_per_class, flags, stream, adam);
}

// backward_w (DL_W_LOGITS) whose last block announces the bucket's gradients to the peers of a peer-memory exchange.
extern "C" DL_API int dl_backward_w_announce_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, const float *w,
                                                 float *grad_w, int64_t n_in, int64_t n_out, int64_t batch, int64_t rows_per_class,
                                                 void *const *flag_ptrs, int rank, int world, int bucket, const int32_t *bucket_state,
                                                 int32_t *block_ticket, int32_t *kernel_count, int kernels_in_bucket, int flags,
                                                 void *stream) {
    DL_REQUIRE(world >= 1 && world <= 16 && rank >= 0 && rank < world && bucket >= 0 && bucket < 32, DL_ERR_INVALID_ARG,
               "dl_backward_w_announce_f32: rank %d of %d, bucket %d", rank, world, bucket);
    DL_REQUIRE(flag_ptrs && bucket_state && block_ticket && kernel_count && kernels_in_bucket >= 1 && grad_w, DL_ERR_INVALID_ARG,
               "dl_backward_w_announce_f32: null pointer");
    AnnounceGradients ann = {};
    for (int p = 0; p < world; ++p) {
        DL_REQUIRE(flag_ptrs[p] != nullptr, DL_ERR_INVALID_ARG, "dl_backward_w_announce_f32: null peer pointer");
        ann.flags[p] = reinterpret_cast<int *>(flag_ptrs[p]);
    }
    ann.world = world;
    ann.word = (bucket * 16 + rank) * 2;
    ann.epoch_src = reinterpret_cast<const int *>(bucket_state);
    ann.block_ticket = reinterpret_cast<int *>(block_ticket);
    ann.kernel_count = reinterpret_cast<int *>(kernel_count);
    ann.kernels = kernels_in_bucket;
    if (n_out == 0) {
        // nothing is launched for an empty layer, so nothing would announce: refuse instead of waiting forever
        return fail(DL_ERR_INVALID_ARG, "dl_backward_w_announce_f32: empty layer");
    }
    return backward_w_entry(x, a, b, grad_y, w, DL_W_LOGITS, grad_w, n_in, n_out, batch, rows_per_class, flags, stream,
                            AdamInBackward{nullptr, nullptr, nullptr, 0.f, 0.f, 0.f, 0.f, 0.f}, ann);
}

// backward_w (DL_W_LOGITS) that also pushes the gradients of the other ranks' slices into their inboxes (PushGradients).
// bucket_offset: floats of the bucket in front of this layer's gradients; bucket_count: floats of the whole bucket;
// inbox_offset / inbox_stride, grad_inbox_ptrs, bucket_state: as for dl_exchange_packets_f32, which follows with pushed = 1.
extern "C" DL_API int dl_backward_w_push_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, const float *w,
                                             float *grad_w, int64_t n_in, int64_t n_out, int64_t batch, int64_t rows_per_class,
                                             void *const *grad_inbox_ptrs, int rank, int world, int64_t bucket_offset,
                                             int64_t bucket_count, int64_t inbox_offset, int64_t inbox_stride,
                                             const int32_t *bucket_state, int flags, void *stream) {
    const char *who = "dl_backward_w_push_f32";
    DL_REQUIRE(world >= 1 && world <= 16 && rank >= 0 && rank < world, DL_ERR_INVALID_ARG, "%s: rank %d of %d", who, rank, world);
    DL_REQUIRE(grad_inbox_ptrs && bucket_state && grad_w, DL_ERR_INVALID_ARG, "%s: null pointer", who);
    DL_REQUIRE(bucket_offset >= 0 && bucket_offset % 4 == 0 && bucket_count % 4 == 0 && bucket_offset + n_out * 16 <= bucket_count &&
                   bucket_count / 4 <= INT32_MAX,
               DL_ERR_INVALID_ARG, "%s: the layer's %lld gradients at %lld do not fit a bucket of %lld floats", who,
               (long long)(n_out * 16), (long long)bucket_offset, (long long)bucket_count);
    PushGradients push = {};
    const int64_t per = ceil_div(bucket_count / 4, (int64_t)world);
    DL_REQUIRE(inbox_offset >= 0 && inbox_stride > 0 && inbox_offset + per <= inbox_stride, DL_ERR_INVALID_ARG,
               "%s: slots %lld + %lld outside a region of %lld", who, (long long)inbox_offset, (long long)per, (long long)inbox_stride);
    for (int p = 0; p < world; ++p) {
        DL_REQUIRE(grad_inbox_ptrs[p] != nullptr && aligned_to(grad_inbox_ptrs[p], 16), DL_ERR_INVALID_ARG,
                   "%s: null or misaligned inbox pointer", who);
        push.inbox[p] = reinterpret_cast<unsigned long long *>(grad_inbox_ptrs[p]);
    }
    push.rank = rank;
    push.world = world;
    push.per4 = (int)(per > 0 ? per : 1);
    push.base4 = (int)(bucket_offset / 4);
    push.region = (long long)rank * inbox_stride + inbox_offset;
    push.half = (long long)world * inbox_stride * 2;
    push.epoch_src = reinterpret_cast<const int *>(bucket_state);
    return backward_w_entry(x, a, b, grad_y, w, DL_W_LOGITS, grad_w, n_in, n_out, batch, rows_per_class, flags, stream,
                            AdamInBackward{nullptr, nullptr, nullptr, 0.f, 0.f, 0.f, 0.f, 0.f}, AnnounceGradients{}, push);
}

extern "C" DL_API int dl_backward_x_f32(const float *x, const float *coef, const float *grad_y, const int64_t *start,
                                 const int32_t *plan, float grad_scale, float *grad_x, int64_t n_in, int64_t n_out,
                                 int64_t batch, int flags, void *stream) {
    return backward_x_entry(x, coef, grad_y, start, plan, grad_scale, grad_x, n_in, n_out, batch, 1, flags, stream);
}

// grad_y has one row per class of `rows_per_class` consecutive outputs ([n_out / rows_per_class][batch]).
extern "C" DL_API int dl_backward_x_classes_f32(const float *x, const float *coef, const float *grad_y_classes, const int64_t *start,
                                                const int32_t *plan, float grad_scale, float *grad_x, int64_t n_in, int64_t n_out,
                                                int64_t batch, int64_t rows_per_class, int flags, void *stream) {
    return backward_x_entry(x, coef, grad_y_classes, start, plan, grad_scale, grad_x, n_in, n_out, batch, rows_per_class, flags, stream);
}

// y [cols][rows] = transpose of x [rows][cols] (a network's input batch -> feature-major).
extern "C" DL_API int dl_transpose_f32(const float *x, float *y, int64_t rows, int64_t cols, void *stream) {
    DL_REQUIRE(rows >= 0 && cols >= 0, DL_ERR_INVALID_ARG, "dl_transpose_f32: negative size");
    if (rows == 0 || cols == 0) return DL_OK;
    DL_REQUIRE(x && y && x != y, DL_ERR_INVALID_ARG, "dl_transpose_f32: null pointer, or in place");
    DL_REQUIRE(ceil_div(rows, 32) <= 65535, DL_ERR_TOO_LARGE, "dl_transpose_f32: more than 2^21 rows");
    const dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)ceil_div(rows, 32));
    transpose_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(x, y, rows, cols);
    return launch_status("dl_transpose_f32");
}

// Checks a layer's index arrays on the device (see check_connections_kernel).  start, list and plan may be null (only a
// and b are checked then).  report: four int64 on the device, zeroed by the caller; stays zero when everything is sound.
extern "C" DL_API int dl_check_connections(const int64_t *a, const int64_t *b, const int64_t *start, const int64_t *list,
                                           const int32_t *plan, int64_t n_in, int64_t n_out, int64_t *report, void *stream) {
    DL_REQUIRE(n_in >= 0 && n_out >= 0, DL_ERR_INVALID_ARG, "dl_check_connections: negative size");
    DL_REQUIRE(report != nullptr && aligned_to(report, 8), DL_ERR_INVALID_ARG, "dl_check_connections: report must be 8-byte aligned");
    if (n_out == 0 && n_in == 0) return DL_OK;
    DL_REQUIRE(n_out == 0 || (a && b), DL_ERR_INVALID_ARG, "dl_check_connections: null pointer");
    DL_REQUIRE(plan == nullptr || aligned_to(plan, 8), DL_ERR_INVALID_ARG, "dl_check_connections: plan must be 8-byte aligned");
    int64_t most = 2 * n_out > n_in + 1 ? 2 * n_out : n_in + 1;
    for (int phase = 1; phase <= 4; ++phase)
        check_connections_kernel<<<(unsigned)ceil_div(most, kThreads), kThreads, 0, as_stream(stream)>>>(
            a, b, start, list, reinterpret_cast<const int2 *>(plan), n_in, n_out, report, phase);
    return launch_status("dl_check_connections");
}

extern "C" DL_API int dl_build_backward_plan(const int64_t *a, const int64_t *b, const int64_t *start, const int64_t *list,
                                      int32_t *plan, int64_t n_in, int64_t n_out, void *stream) {
    DL_REQUIRE(n_in >= 0 && n_out >= 0, DL_ERR_INVALID_ARG, "dl_build_backward_plan: negative size");
    DL_REQUIRE(n_out < kMaxRows && n_in < 2 * kMaxRows, DL_ERR_TOO_LARGE, "dl_build_backward_plan: more than 2^30 neurons");
    if (n_in == 0 || n_out == 0) return DL_OK;
    DL_REQUIRE(a && b && start && list && plan, DL_ERR_INVALID_ARG, "dl_build_backward_plan: null pointer");
    DL_REQUIRE(aligned_to(plan, 8), DL_ERR_INVALID_ARG, "dl_build_backward_plan: plan must be 8-byte aligned");
    build_plan_kernel<<<(unsigned)ceil_div(n_in, kThreads), kThreads, 0, as_stream(stream)>>>(
        a, b, start, list, reinterpret_cast<int2 *>(plan), n_in);
    return launch_status("dl_build_backward_plan");
}
