// Packed-bit inference kernels: per-neuron gate on packed words, bit packing, group bit-sum.
//
// A packed activation is t[n][words]; sample s is bit (s % bit_count) of word (s / bit_count),
// least-significant bit first.  On a little-endian machine that is byte s/8, bit s%8 of the
// row for every word width, so all kernels here treat a row as a string of row_bytes =
// words*bit_count/8 bytes and move it in the widest unit that divides it (16 bytes when they
// can).  The work is bitwise integer logic bounded by HBM traffic; there is nothing for
// tensor cores to do.
#include <stdlib.h>

#include "common.cuh"
#include "gates.cuh"
#include "pack_tile.cuh"
#include "bitcount.cuh"

namespace dl {

// packed_tma.cu: the same eval with the gathered rows staged in shared memory by bulk copies
bool eval_tma_applicable(const void *x, const void *y, int64_t row_bytes, int64_t n_out);
int launch_eval_tma(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, void *y, int64_t n_in, int64_t n_out,
                    int64_t row_bytes, cudaStream_t st, int64_t x_pitch, int64_t y_pitch);
// groupbitsum_tma.cu: the group bit-sum with rows staged the same way
bool groupbitsum_tma_applicable(const void *x, int64_t n, int64_t row_bytes, int64_t k);
int launch_groupbitsum_tma(const void *x, int32_t *out, int64_t n, int64_t row_bytes, int64_t batch, int64_t k, cudaStream_t st);

// ---------------------------------------------------------------------------------------------
// eval:  y[j][c] = gate_j(x[a_j][c], x[b_j][c])
// Same tiling as the float forward: a group of G lanes covers G units of a row, 256/G rows per
// pass, U passes per CTA, slabs of G units walked along blockIdx.y so that concurrently
// resident CTAs gather from the same column slab of x (L2 reuse for the second reader).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 gate_apply(uint4 a, uint4 b, const GateMasks &g) {
    return make_uint4(gate32(a.x, b.x, g), gate32(a.y, b.y, g), gate32(a.z, b.z, g), gate32(a.w, b.w, g));
}
__device__ __forceinline__ unsigned long long gate_apply(unsigned long long a, unsigned long long b, const GateMasks &g) {
    const uint32_t lo = gate32((uint32_t)a, (uint32_t)b, g);
    const uint32_t hi = gate32((uint32_t)(a >> 32), (uint32_t)(b >> 32), g);
    return ((unsigned long long)hi << 32) | lo;
}
__device__ __forceinline__ uint32_t gate_apply(uint32_t a, uint32_t b, const GateMasks &g) { return gate32(a, b, g); }
__device__ __forceinline__ uint16_t gate_apply(uint16_t a, uint16_t b, const GateMasks &g) { return (uint16_t)gate32(a, b, g); }
__device__ __forceinline__ uint8_t gate_apply(uint8_t a, uint8_t b, const GateMasks &g) { return (uint8_t)gate32(a, b, g); }

template <typename V, int G, int U>
__global__ void __launch_bounds__(kThreads)
eval_kernel(const V *__restrict__ x, const int64_t *__restrict__ a, const int64_t *__restrict__ b,
            const uint8_t *__restrict__ gate, V *__restrict__ y, int64_t n_out, int64_t ncols, int64_t nslabs) {
    constexpr int R = kThreads / G;
    const int tid = threadIdx.x;
    const int lane = tid % G;
    const int64_t j0 = (int64_t)blockIdx.x * (R * U) + tid / G;

    const V *xa[U];
    const V *xb[U];
    GateMasks gm[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t j = j0 + u * R;
        if (j < n_out) {
            xa[u] = x + __ldg(a + j) * ncols;
            xb[u] = x + __ldg(b + j) * ncols;
            gm[u] = gate_masks(__ldg(gate + j));
        }
    }
    for (int64_t slab = blockIdx.y; slab < nslabs; slab += gridDim.y) {
        const int64_t col = slab * G + lane;
        if (col >= ncols) continue;
        V va[U], vb[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (j0 + u * R < n_out) {
                va[u] = __ldg(xa[u] + col);
                vb[u] = __ldg(xb[u] + col);
            }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (j0 + u * R < n_out) y[(j0 + u * R) * ncols + col] = gate_apply(va[u], vb[u], gm[u]);
    }
}

template <typename V>
static int launch_eval(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, void *y, int64_t n_out,
                       int64_t row_bytes, cudaStream_t st) {
    constexpr int U = 4;
    const int64_t ncols = row_bytes / (int64_t)sizeof(V);
    const int G = pow2_at_least(ncols, 32);
    const int64_t nslabs = ceil_div(ncols, G);
    const dim3 grid((unsigned)ceil_div(n_out, (kThreads / G) * U), (unsigned)(nslabs < 65535 ? nslabs : 65535));
    const V *xv = reinterpret_cast<const V *>(x);
    V *yv = reinterpret_cast<V *>(y);
#define DL_EV(GG)                                                                                   \
    case GG:                                                                                        \
        eval_kernel<V, GG, U><<<grid, kThreads, 0, st>>>(xv, a, b, gate, yv, n_out, ncols, nslabs); \
        break;
    switch (G) {
        DL_EV(1) DL_EV(2) DL_EV(4) DL_EV(8) DL_EV(16) DL_EV(32)
    }
#undef DL_EV
    return launch_status("dl_eval_packed");
}

// ---------------------------------------------------------------------------------------------
// packbits, feature-major source t[n][batch] (one byte per bool).
// A thread builds one output byte from eight source bytes; the fast variant needs batch % 8 == 0
// and an 8-byte aligned source so that the eight bytes are one load.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t squeeze8(unsigned long long v) {
    // bytes (zero / non-zero) -> 8 bits, byte 0 to bit 0
    const uint32_t lo = __vsetne4((uint32_t)v, 0u), hi = __vsetne4((uint32_t)(v >> 32), 0u);  // 0x01 per non-zero byte
    const uint32_t l = (lo * 0x01020408u) >> 24;  // moves bits 0,8,16,24 to bits 24,25,26,27
    const uint32_t h = (hi * 0x01020408u) >> 24;
    return (l & 0xFu) | ((h & 0xFu) << 4);
}

template <bool FAST>
__global__ void __launch_bounds__(kThreads)
packbits_kernel(const uint8_t *__restrict__ t, uint8_t *__restrict__ out, int64_t n, int64_t batch, int64_t row_bytes) {
    // one thread per output byte; blockIdx.y walks rows
    const int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (q >= row_bytes) return;
    for (int64_t row = blockIdx.y; row < n; row += gridDim.y) {
        const uint8_t *src = t + row * batch + q * 8;
        uint32_t bits = 0;
        if (FAST) {
            if (q * 8 < batch) bits = squeeze8(__ldg(reinterpret_cast<const unsigned long long *>(src)));
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (q * 8 + i < batch) bits |= (uint32_t)(__ldg(src + i) != 0) << i;
        }
        out[row * row_bytes + q] = (uint8_t)bits;
    }
}

// packbits from the batch-major matrix t[batch][n], n % 8 == 0: transpose and pack in one pass, 8-byte loads, bits moved
// eight by eight (pack_tile.cuh).
struct MaskNonZero {
    __device__ __forceinline__ uint32_t operator()(uint32_t lo, uint32_t hi, int) const {
        return squeeze8_ones(nonzero_bytes(lo), nonzero_bytes(hi));
    }
};

__global__ void __launch_bounds__(kThreads)
packbits_bm8_kernel(const uint8_t *__restrict__ t, uint8_t *__restrict__ out, int64_t n, int64_t batch, int64_t row_bytes) {
    __shared__ unsigned long long s_words[8 * kPackRow];
    const int64_t f0 = (int64_t)blockIdx.x * kPackFeatures;
    for (int64_t sblk = blockIdx.y; sblk * kPackSamples < row_bytes * 8; sblk += gridDim.y)
        pack_tile<1>(t, out, 0, n, batch, row_bytes, f0, sblk, s_words, MaskNonZero());
}

// The same for any n (and any alignment): 4-byte or single-byte loads, one bit at a time.
// A CTA takes 128 features x 512 samples.  Warp w owns 64 samples (one 64-bit word); its lanes
// each own four adjacent features, read as one 32-bit load per sample (coalesced along the
// features) and shifted into four words.  The 8 warps' words go through shared memory so that
// a feature's eight words leave as one 64-byte run.
template <bool VEC4>
__global__ void __launch_bounds__(kThreads)
packbits_bm_kernel(const uint8_t *__restrict__ t, uint8_t *__restrict__ out, int64_t n, int64_t batch, int64_t row_bytes) {
    __shared__ unsigned long long s_words[128][9];  // [feature][word], padded
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int64_t f0 = (int64_t)blockIdx.x * 128;
    for (int64_t sblk = blockIdx.y; sblk * 512 < batch; sblk += gridDim.y) {
        const int64_t s0 = sblk * 512 + warp * 64;
        unsigned long long wd[4] = {0ull, 0ull, 0ull, 0ull};
        const int64_t f = f0 + lane * 4;
        if (VEC4) {
            if (f < n) {  // n % 4 == 0, so all four features exist
#pragma unroll 16
                for (int s = 0; s < 64; ++s) {
                    if (s0 + s < batch) {
                        const uint32_t v = __vsetne4(__ldg(reinterpret_cast<const uint32_t *>(t + (s0 + s) * n + f)), 0u);
                        wd[0] |= (unsigned long long)(v & 1u) << s;
                        wd[1] |= (unsigned long long)((v >> 8) & 1u) << s;
                        wd[2] |= (unsigned long long)((v >> 16) & 1u) << s;
                        wd[3] |= (unsigned long long)((v >> 24) & 1u) << s;
                    }
                }
            }
        } else {
            for (int s = 0; s < 64; ++s) {
                if (s0 + s < batch) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (f + q < n) wd[q] |= (unsigned long long)(__ldg(t + (s0 + s) * n + f + q) != 0) << s;
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) s_words[lane * 4 + q][warp] = wd[q];
        __syncthreads();
        // write: byte granularity so that any bit_count / ragged row length works
        const int64_t byte0 = sblk * 64;  // first output byte of this sample block
        for (int idx = threadIdx.x; idx < 128 * 64; idx += kThreads) {
            const int fl = idx / 64, by = idx % 64;
            if (f0 + fl < n && byte0 + by < row_bytes)
                out[(f0 + fl) * row_bytes + byte0 + by] = (uint8_t)(s_words[fl][by / 8] >> (8 * (by % 8)));
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// groupbitsum: out[s][c] = number of set bits of sample s over the n/k rows of class c.
//
// Fast path (row_bytes % 16 == 0, 16-byte aligned rows).  A CTA owns LANES 16-byte columns
// (LANES*128 samples) and a block of KC classes.  Its threads form groups of LANES lanes; a
// group streams the rows of one (class, row chunk) task with 16-byte loads and counts
// vertically in bit-sliced form: a carry-save adder tree turns every 8 rows into one word of
// weight 8 that ripples into the high planes, so a word costs ~2 LOP3 per row instead of one
// add per bit.  The planes are then spread to per-sample integers four samples at a time
// (16-bit fields) and added into a shared-memory tile that leaves as contiguous int32 runs.
// ---------------------------------------------------------------------------------------------
// planes -> integers for the 64 samples of one word: field f of `acc` holds sample s + 16 f.
template <int LANES>
__device__ __forceinline__ void spread_counts(const BitCounter &cn, int *dst, int nplanes) {
#pragma unroll 4
    for (int s = 0; s < 16; ++s) {
        unsigned long long acc = 0ull;
#pragma unroll
        for (int pl = 0; pl < kPlanes; ++pl)
            if (pl < nplanes) acc |= ((cn.plane(pl) >> s) & 0x0001000100010001ull) << pl;
#pragma unroll
        for (int f = 0; f < 4; ++f) {
            const int cnt = (int)((acc >> (16 * f)) & 0xFFFFull);
            if (cnt) atomicAdd(dst + (s + 16 * f) * LANES, cnt);
        }
    }
}

template <int LANES>
__global__ void __launch_bounds__(kThreads)
groupbitsum_kernel(const ulonglong2 *__restrict__ x, int32_t *__restrict__ out, int64_t ncols16, int64_t batch, int k,
                   int rows_per_class, int chunks, int kc, int nplanes) {
    extern __shared__ int s_cnt[];  // [kc][128][LANES] (+1 pad per class)
    constexpr int NG = kThreads / LANES;
    const int pitch = 128 * LANES + 1;
    const int tid = threadIdx.x;
    const int lane = tid % LANES, grp = tid / LANES;
    const int c0 = blockIdx.y * kc;
    const int nc = min(kc, k - c0);
    const int64_t col = (int64_t)blockIdx.x * LANES + lane;

    for (int t = tid; t < kc * pitch; t += kThreads) s_cnt[t] = 0;
    __syncthreads();

    const int tasks = nc * chunks;
    for (int task = grp; task < tasks; task += NG) {
        const int cc = task / chunks, q = task % chunks;
        if (col >= ncols16) continue;
        const int64_t rbeg = (int64_t)(c0 + cc) * rows_per_class + ((int64_t)rows_per_class * q) / chunks;
        const int64_t rend = (int64_t)(c0 + cc) * rows_per_class + ((int64_t)rows_per_class * (q + 1)) / chunks;
        BitCounter cx, cy;
        cx.clear();
        cy.clear();
        const ulonglong2 *p = x + rbeg * ncols16 + col;
        int64_t r = rbeg;
        for (; r + 8 <= rend; r += 8) {
            ulonglong2 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __ldg(p + (int64_t)i * ncols16);
            p += 8 * ncols16;
            unsigned long long vx[8], vy[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { vx[i] = v[i].x; vy[i] = v[i].y; }
            cx.add8(vx);
            cy.add8(vy);
        }
        for (; r < rend; ++r) {
            const ulonglong2 v = __ldg(p);
            p += ncols16;
            cx.add1(v.x);
            cy.add1(v.y);
        }
        spread_counts<LANES>(cx, s_cnt + cc * pitch + lane, nplanes);
        spread_counts<LANES>(cy, s_cnt + cc * pitch + lane + 64 * LANES, nplanes);
    }
    __syncthreads();

    const int64_t sbase = (int64_t)blockIdx.x * LANES * 128;
    const int64_t nsamp = min((int64_t)LANES * 128, batch - sbase);
    for (int64_t t = tid; t < nsamp * nc; t += kThreads) {
        const int sl = (int)(t / nc), cc = (int)(t % nc);
        const int ln = sl / 128, ws = sl % 128;
        out[(sbase + sl) * k + c0 + cc] = s_cnt[cc * pitch + ws * LANES + ln];
    }
}

// Generic path for any row length: one thread per (byte column, class).
__global__ void __launch_bounds__(kThreads)
groupbitsum_bytes_kernel(const uint8_t *__restrict__ x, int32_t *__restrict__ out, int64_t row_bytes, int64_t batch, int k,
                         int rows_per_class) {
    const int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const int c = blockIdx.y;
    if (q >= row_bytes) return;
    int cnt[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const uint8_t *p = x + (int64_t)c * rows_per_class * row_bytes + q;
    for (int r = 0; r < rows_per_class; ++r) {
        const uint32_t v = __ldg(p + (int64_t)r * row_bytes);
#pragma unroll
        for (int i = 0; i < 8; ++i) cnt[i] += (v >> i) & 1u;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (q * 8 + i < batch) out[(q * 8 + i) * k + c] = cnt[i];
}

template <int LANES>
static int launch_groupbitsum(const void *x, int32_t *out, int64_t n, int64_t row_bytes, int64_t batch, int64_t k,
                              cudaStream_t st) {
    const int64_t ncols16 = row_bytes / 16;
    const int64_t m = n / k;
    // shared tile: kc classes x (128*LANES+1) ints; keep it below 96 KB so that two CTAs fit an SM
    const int64_t per_class = (128 * LANES + 1) * 4;
    int64_t kc = (96 * 1024) / per_class;
    if (kc > k) kc = k;
    if (kc < 1) kc = 1;
    // few column blocks (a short batch): spread the classes over more CTAs so that ~600 of them exist
    const int64_t colblocks = ceil_div(ncols16, LANES);
    int64_t class_blocks = ceil_div(592, colblocks);
    if (class_blocks > k) class_blocks = k;
    if (ceil_div(k, class_blocks) < kc) kc = ceil_div(k, class_blocks);
    // row chunks: enough tasks for the 256/LANES groups, and no chunk above the counter's range
    const int ng = kThreads / LANES;
    int64_t chunks = ceil_div(ng, kc);
    if (chunks > m) chunks = m > 0 ? m : 1;
    while (ceil_div(m, chunks) > kMaxChunkRows) ++chunks;
    int nplanes = 1;
    while (nplanes < kPlanes && ((int64_t)1 << nplanes) <= ceil_div(m, chunks)) ++nplanes;
    const size_t smem = (size_t)(kc * per_class);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(groupbitsum_kernel<LANES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
        return launch_status("dl_groupbitsum (shared memory opt-in)");
    const dim3 grid((unsigned)ceil_div(ncols16, LANES), (unsigned)ceil_div(k, kc));
    groupbitsum_kernel<LANES><<<grid, kThreads, smem, st>>>(reinterpret_cast<const ulonglong2 *>(x), out, ncols16, batch,
                                                           (int)k, (int)m, (int)chunks, (int)kc, nplanes);
    return launch_status("dl_groupbitsum");
}

}  // namespace dl

using namespace dl;

static int check_bits(const char *who, int bit_count) {
    if (bit_count == 8 || bit_count == 16 || bit_count == 32 || bit_count == 64) return DL_OK;
    return fail(DL_ERR_BAD_BIT_COUNT, "%s: `bit_count` has to be in { 8, 16, 32, 64 }, got %d", who, bit_count);
}

extern "C" DL_API int dl_eval_packed(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, void *y, int64_t n_in,
                              int64_t n_out, int64_t words, int bit_count, void *stream) {
    if (int s = check_bits("dl_eval_packed", bit_count)) return s;
    DL_REQUIRE(n_in >= 0 && n_out >= 0 && words >= 0, DL_ERR_INVALID_ARG, "dl_eval_packed: negative size");
    if (n_out == 0 || words == 0) return DL_OK;
    DL_REQUIRE(x && a && b && gate && y, DL_ERR_INVALID_ARG, "dl_eval_packed: null pointer");
    DL_REQUIRE(n_in > 0, DL_ERR_INVALID_ARG, "dl_eval_packed: n_in is 0 but n_out is %lld", (long long)n_out);
    const int64_t row_bytes = words * (bit_count / 8);
    cudaStream_t st = as_stream(stream);
    auto fits = [&](int64_t sz) { return row_bytes % sz == 0 && aligned_to(x, sz) && aligned_to(y, sz); };
    // DL_TUNE_EVAL_KERNEL = 1 forces the register-staged kernel (for A/B measurements)
    const bool plain_only = tuning(DL_TUNE_EVAL_KERNEL) == 1;
    if (!plain_only && eval_tma_applicable(x, y, row_bytes, n_out)) return launch_eval_tma(x, a, b, gate, y, n_in, n_out, row_bytes, st, row_bytes, row_bytes);
    if (fits(16)) return launch_eval<uint4>(x, a, b, gate, y, n_out, row_bytes, st);
    if (fits(8)) return launch_eval<unsigned long long>(x, a, b, gate, y, n_out, row_bytes, st);
    if (fits(4)) return launch_eval<uint32_t>(x, a, b, gate, y, n_out, row_bytes, st);
    if (fits(2)) return launch_eval<uint16_t>(x, a, b, gate, y, n_out, row_bytes, st);
    return launch_eval<uint8_t>(x, a, b, gate, y, n_out, row_bytes, st);
}

// dl_eval_packed on column slices: the rows of x and y are `row_bytes` long but lie x_pitch / y_pitch bytes apart (a column
// range of wider matrices, or contiguous ones with pitch == row_bytes).  Staged kernel only: rows of at least 512 bytes,
// row_bytes, both pitches and both pointers multiples of 16.
extern "C" DL_API int dl_eval_packed_pitched(const void *x, int64_t x_pitch, const int64_t *a, const int64_t *b, const uint8_t *gate,
                                             void *y, int64_t y_pitch, int64_t n_in, int64_t n_out, int64_t row_bytes, void *stream) {
    DL_REQUIRE(n_in > 0 && n_out > 0 && row_bytes > 0, DL_ERR_INVALID_ARG, "dl_eval_packed_pitched: sizes must be positive");
    DL_REQUIRE(x && a && b && gate && y, DL_ERR_INVALID_ARG, "dl_eval_packed_pitched: null pointer");
    DL_REQUIRE(x_pitch >= row_bytes && y_pitch >= row_bytes && x_pitch % 16 == 0 && y_pitch % 16 == 0, DL_ERR_INVALID_ARG,
               "dl_eval_packed_pitched: pitches must be multiples of 16 and at least row_bytes");
    DL_REQUIRE(eval_tma_applicable(x, y, row_bytes, n_out), DL_ERR_INVALID_ARG,
               "dl_eval_packed_pitched: rows must be at least 512 bytes, a multiple of 16 and 16-byte aligned");
    return launch_eval_tma(x, a, b, gate, y, n_in, n_out, row_bytes, as_stream(stream), x_pitch, y_pitch);
}

extern "C" DL_API int dl_packbits(const uint8_t *t, void *out, int64_t n, int64_t batch, int bit_count, void *stream) {
    if (int s = check_bits("dl_packbits", bit_count)) return s;
    DL_REQUIRE(n >= 0 && batch >= 0, DL_ERR_INVALID_ARG, "dl_packbits: negative size");
    if (n == 0 || batch == 0) return DL_OK;
    DL_REQUIRE(t && out, DL_ERR_INVALID_ARG, "dl_packbits: null pointer");
    const int64_t row_bytes = ceil_div(batch, bit_count) * (bit_count / 8);
    const dim3 grid((unsigned)ceil_div(row_bytes, kThreads), (unsigned)(n < 65535 ? n : 65535));
    uint8_t *o = reinterpret_cast<uint8_t *>(out);
    if (batch % 8 == 0 && aligned_to(t, 8))
        packbits_kernel<true><<<grid, kThreads, 0, as_stream(stream)>>>(t, o, n, batch, row_bytes);
    else
        packbits_kernel<false><<<grid, kThreads, 0, as_stream(stream)>>>(t, o, n, batch, row_bytes);
    return launch_status("dl_packbits");
}

extern "C" DL_API int dl_packbits_batch_major(const uint8_t *t, void *out, int64_t n, int64_t batch, int bit_count, void *stream) {
    if (int s = check_bits("dl_packbits_batch_major", bit_count)) return s;
    DL_REQUIRE(n >= 0 && batch >= 0, DL_ERR_INVALID_ARG, "dl_packbits_batch_major: negative size");
    if (n == 0 || batch == 0) return DL_OK;
    DL_REQUIRE(t && out, DL_ERR_INVALID_ARG, "dl_packbits_batch_major: null pointer");
    const int64_t row_bytes = ceil_div(batch, bit_count) * (bit_count / 8);
    const int64_t sblocks = ceil_div(row_bytes, 64);  // 512 samples each; covers the pad bytes too
    const dim3 grid((unsigned)ceil_div(n, 128), (unsigned)(sblocks < 65535 ? sblocks : 65535));
    uint8_t *o = reinterpret_cast<uint8_t *>(out);
    if (n % 8 == 0 && aligned_to(t, 8)) {
        const int64_t sb = ceil_div(row_bytes, kPackSamples / 8);
        const dim3 grid8((unsigned)ceil_div(n, kPackFeatures), (unsigned)(sb < 65535 ? sb : 65535));
        packbits_bm8_kernel<<<grid8, kThreads, 0, as_stream(stream)>>>(t, o, n, batch, row_bytes);
    } else if (n % 4 == 0 && aligned_to(t, 4))
        packbits_bm_kernel<true><<<grid, kThreads, 0, as_stream(stream)>>>(t, o, n, batch, row_bytes);
    else
        packbits_bm_kernel<false><<<grid, kThreads, 0, as_stream(stream)>>>(t, o, n, batch, row_bytes);
    return launch_status("dl_packbits_batch_major");
}

extern "C" DL_API int dl_groupbitsum(const void *x, int32_t *out, int64_t n, int64_t words, int64_t pad_len, int64_t k,
                              int bit_count, void *stream) {
    if (int s = check_bits("dl_groupbitsum", bit_count)) return s;
    DL_REQUIRE(n >= 0 && words >= 0 && k > 0, DL_ERR_INVALID_ARG, "dl_groupbitsum: bad size (n=%lld words=%lld k=%lld)",
               (long long)n, (long long)words, (long long)k);
    DL_REQUIRE(n % k == 0, DL_ERR_NOT_DIVISIBLE, "in_dim (%lld) has to be divisible by k (%lld) but it is not", (long long)n,
               (long long)k);
    DL_REQUIRE(pad_len >= 0 && pad_len < bit_count && (words > 0 || pad_len == 0), DL_ERR_INVALID_ARG,
               "dl_groupbitsum: pad_len %lld out of range", (long long)pad_len);
    DL_REQUIRE(k <= 65535 && n / k <= INT32_MAX, DL_ERR_TOO_LARGE, "dl_groupbitsum: k or rows per class too large");
    const int64_t batch = words * bit_count - pad_len;
    if (batch == 0) return DL_OK;
    DL_REQUIRE(out && (x || n == 0), DL_ERR_INVALID_ARG, "dl_groupbitsum: null pointer");
    const int64_t row_bytes = words * (bit_count / 8);
    cudaStream_t st = as_stream(stream);
    // DL_TUNE_GROUPBITSUM_KERNEL = 1 (plain) / 2 (staged) forces one of the two kernels (for A/B measurements)
    const bool plain_only = tuning(DL_TUNE_GROUPBITSUM_KERNEL) == 1;
    const bool staged_only = tuning(DL_TUNE_GROUPBITSUM_KERNEL) == 2;
    // The staged kernel splits a class's rows over several units when (column blocks x classes) alone cannot fill
    // the machine; a split costs a plane expansion and global atomics per unit, which only pays while a unit still
    // streams a few hundred rows.  Shorter pieces go to the register kernel, which splits rows inside a CTA.
    int64_t splits = ceil_div(8 * 148, ceil_div(row_bytes, 1024) * k);
    if (splits < 1) splits = 1;
    const bool enough_units = (n / k) / splits >= 256;
    if (!plain_only && (enough_units || staged_only) && groupbitsum_tma_applicable(x, n, row_bytes, k))
        return launch_groupbitsum_tma(x, out, n, row_bytes, batch, k, st);
    if (n > 0 && row_bytes % 16 == 0 && aligned_to(x, 16)) {
        const int64_t ncols16 = row_bytes / 16;
        // 256-byte row segments when there are enough of them, narrower ones for very short rows
        if (ncols16 >= 16 * 32) return launch_groupbitsum<16>(x, out, n, row_bytes, batch, k, st);
        if (ncols16 >= 8 * 32) return launch_groupbitsum<8>(x, out, n, row_bytes, batch, k, st);
        return launch_groupbitsum<4>(x, out, n, row_bytes, batch, k, st);
    }
    const dim3 grid((unsigned)ceil_div(row_bytes, kThreads), (unsigned)k);
    groupbitsum_bytes_kernel<<<grid, kThreads, 0, st>>>(reinterpret_cast<const uint8_t *>(x), out, row_bytes, batch, (int)k,
                                                        (int)(n / k));
    return launch_status("dl_groupbitsum");
}
