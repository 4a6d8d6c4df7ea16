// Whole-network packed-bit inference in one kernel: all logic layers and the group bit-sum, with the
// activations of a block of 64 samples resident in shared memory from the first layer to the class counts.
//
// Layer by layer, a network of L layers of width n moves 8*(n_in + n) bytes per 64 samples through HBM per
// layer.  Here the only HBM traffic is the packed input (n_0/8 bytes per sample) and the counts (4k bytes per
// sample); the gates read and write shared memory.  The kernel is then bound by shared-memory bandwidth under
// random 8-byte accesses (two reads and one write per gate and word), not by HBM.
//
// Work split: a CTA (1024 threads, one per SM, persistent) takes four adjacent word columns at a time -- the
// 32 bytes per input row are one full DRAM sector --, stages them, and runs the net once per column.  Per layer
// every thread evaluates gates 4t..4t+3 (+4096 i): one 16-byte load of packed gate descriptors
// {a:14 | b:14 | op:4}, eight 8-byte shared loads, four gates, one 32-byte shared store; __syncthreads() between
// layers; the two activation buffers ping-pong.  The group bit-sum adds the last layer's words bit-sliced:
// per-thread ripple counters, a shuffle tree of bit-sliced adders inside each warp, a last pass per sample.
//
// Limits (checked on the host): every layer at most 16384 gates wide, 2*max_width*8 + 32*n_0 bytes of shared
// memory within the 227 KB of an SM, rows a multiple of 8 bytes.  Other networks run layer by layer.
#include "common.cuh"
#include "gates.cuh"

namespace dl {

constexpr int kNetThreads = 1024;
constexpr int kNetMaxWidth = 16384;
constexpr int kNetMaxLayers = 32;

struct NetDesc {
    int n_layers;
    int width[kNetMaxLayers + 1];      // width[0] = input rows, width[l] = gates of layer l
    int meta_off[kNetMaxLayers];       // offset of layer l's descriptors in `meta` (multiple of 4)
};

typedef unsigned long long u64;

__device__ __forceinline__ u64 gate64(u64 a, u64 b, uint32_t op) {
    const GateMasks g = gate_masks((int)op);
    const uint32_t lo = gate32((uint32_t)a, (uint32_t)b, g);
    const uint32_t hi = gate32((uint32_t)(a >> 32), (uint32_t)(b >> 32), g);
    return ((u64)hi << 32) | lo;
}

__device__ __forceinline__ u64 shfl_xor64(u64 v, int off) {
    const uint32_t lo = __shfl_xor_sync(0xffffffffu, (uint32_t)v, off);
    const uint32_t hi = __shfl_xor_sync(0xffffffffu, (uint32_t)(v >> 32), off);
    return ((u64)hi << 32) | lo;
}

constexpr int kSumPlanes = 16;  // bit-sliced counts up to 65535 rows per class

__global__ void __launch_bounds__(kNetThreads, 1)
eval_net_kernel(const u64 *__restrict__ x, const uint32_t *__restrict__ meta, NetDesc desc, int32_t *__restrict__ out,
                int64_t words, int64_t batch, int k, int max_width, int planes_thread, int planes_total) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u64 *buf0 = reinterpret_cast<u64 *>(smem_raw);
    u64 *buf1 = buf0 + max_width;
    u64 *stage = buf1 + max_width;                   // [width0][4]
    __shared__ u64 s_planes[32][kSumPlanes];         // per-warp partial counts (bit-sliced)

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int L = desc.n_layers;
    const int n0 = desc.width[0];
    const int nl = desc.width[L];
    const int m = nl / k;                            // rows per class
    // threads per class for the bit-sum: whole warps, as many as fit
    int tpc = (kNetThreads / k) & ~31;
    if (tpc == 0) tpc = 32;                          // k > 32: classes are handled in rounds of 32 warps
    const int rows_per_thread = (m + tpc - 1) / tpc;
    const int64_t ngroups = (words + 3) / 4;

    for (int64_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x) {
        const int64_t w0 = grp * 4;
        const int nw = (int)min((int64_t)4, words - w0);
        // ---- stage the four input columns
        if (nw == 4 && (words % 4 == 0)) {
            for (int r = tid; r < n0; r += kNetThreads) {
                const ulonglong2 *src = reinterpret_cast<const ulonglong2 *>(x + (int64_t)r * words + w0);
                const ulonglong2 v0 = __ldg(src), v1 = __ldg(src + 1);
                stage[r * 4 + 0] = v0.x; stage[r * 4 + 1] = v0.y; stage[r * 4 + 2] = v1.x; stage[r * 4 + 3] = v1.y;
            }
        } else {
            for (int i = tid; i < n0 * 4; i += kNetThreads) {
                const int r = i >> 2, q = i & 3;
                stage[i] = q < nw ? __ldg(x + (int64_t)r * words + w0 + q) : 0ull;
            }
        }
        __syncthreads();

        for (int q = 0; q < nw; ++q) {
            // ---- the layers
            for (int l = 0; l < L; ++l) {
                const u64 *in = l == 0 ? stage + q : ((l & 1) ? buf0 : buf1);
                const int in_stride = l == 0 ? 4 : 1;
                u64 *dst = (l & 1) ? buf1 : buf0;
                const int n = desc.width[l + 1];
                const uint4 *md = reinterpret_cast<const uint4 *>(meta + desc.meta_off[l]);
                for (int j = tid * 4; j < n; j += kNetThreads * 4) {
                    const uint4 d = __ldg(md + (j >> 2));
                    const uint32_t dd[4] = {d.x, d.y, d.z, d.w};
                    u64 r[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const u64 va = in[(dd[i] & 0x3FFFu) * in_stride];
                        const u64 vb = in[((dd[i] >> 14) & 0x3FFFu) * in_stride];
                        r[i] = gate64(va, vb, dd[i] >> 28);
                    }
                    if (j + 3 < n) {
                        *reinterpret_cast<ulonglong2 *>(dst + j) = make_ulonglong2(r[0], r[1]);
                        *reinterpret_cast<ulonglong2 *>(dst + j + 2) = make_ulonglong2(r[2], r[3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (j + i < n) dst[j + i] = r[i];
                    }
                }
                __syncthreads();
            }
            const u64 *fin = ((L - 1) & 1) ? buf1 : buf0;

            // ---- group bit-sum of the last layer's words, class by class in rounds of (1024 / tpc) classes
            const int classes_per_round = kNetThreads / tpc;
            const int64_t s0 = (w0 + q) * 64;            // first sample of this word column
            for (int c0 = 0; c0 < k; c0 += classes_per_round) {
                const int c = c0 + tid / tpc;
                const int tin = tid % tpc;               // thread within the class
                u64 pl[kSumPlanes];
#pragma unroll
                for (int p = 0; p < kSumPlanes; ++p) pl[p] = 0ull;
                if (c < k && tid / tpc < classes_per_round) {
                    for (int i = 0; i < rows_per_thread; ++i) {
                        const int r = tin + i * tpc;
                        if (r < m) {
                            u64 carry = fin[c * m + r];
#pragma unroll
                            for (int p = 0; p < kSumPlanes; ++p) {
                                const u64 t = pl[p] & carry;
                                pl[p] ^= carry;
                                carry = t;
                                if (carry == 0ull) break;
                            }
                        }
                    }
                }
                // bit-sliced adder tree over the 32 lanes of the warp
                int live = planes_thread;                // planes that can be non-zero so far
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    u64 carry = 0ull;
                    live = min(live + 1, kSumPlanes);
#pragma unroll
                    for (int p = 0; p < kSumPlanes; ++p) {
                        if (p < live) {
                            const u64 other = shfl_xor64(pl[p], off);
                            const u64 a = pl[p];
                            pl[p] = a ^ other ^ carry;
                            carry = (a & other) | (carry & (a ^ other));
                        }
                    }
                }
                if (lane == 0) {
#pragma unroll
                    for (int p = 0; p < kSumPlanes; ++p) s_planes[warp][p] = pl[p];
                }
                __syncthreads();
                // one thread per (class of this round, sample): add the class's warps
                const int wpc = tpc / 32;                // warps per class
                for (int t = tid; t < classes_per_round * 64; t += kNetThreads) {
                    const int cc = t / 64, smp = t % 64;
                    if (c0 + cc < k && s0 + smp < batch) {
                        int cnt = 0;
                        for (int wv = 0; wv < wpc; ++wv)
                            for (int p = 0; p < planes_total; ++p) cnt += (int)((s_planes[cc * wpc + wv][p] >> smp) & 1ull) << p;
                        out[(s0 + smp) * k + c0 + cc] = cnt;
                    }
                }
                __syncthreads();
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads)
pack_meta_kernel(const int64_t *__restrict__ a, const int64_t *__restrict__ b, const uint8_t *__restrict__ gate,
                 uint32_t *__restrict__ meta, int64_t n_out, int64_t n_padded) {
    const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (j >= n_padded) return;
    meta[j] = j < n_out ? ((uint32_t)a[j] | ((uint32_t)b[j] << 14) | ((uint32_t)gate[j] << 28)) : 0u;
}

}  // namespace dl

using namespace dl;

extern "C" DL_API int dl_pack_net_layer(const int64_t *a, const int64_t *b, const uint8_t *gate, uint32_t *meta, int64_t n_in,
                                        int64_t n_out, void *stream) {
    DL_REQUIRE(n_in > 0 && n_out > 0, DL_ERR_INVALID_ARG, "dl_pack_net_layer: bad size");
    DL_REQUIRE(n_in <= kNetMaxWidth && n_out <= kNetMaxWidth, DL_ERR_TOO_LARGE,
               "dl_pack_net_layer: layers wider than %d cannot be fused", kNetMaxWidth);
    DL_REQUIRE(a && b && gate && meta, DL_ERR_INVALID_ARG, "dl_pack_net_layer: null pointer");
    const int64_t padded = (n_out + 3) / 4 * 4;
    pack_meta_kernel<<<(unsigned)ceil_div(padded, kThreads), kThreads, 0, as_stream(stream)>>>(a, b, gate, meta, n_out, padded);
    return launch_status("dl_pack_net_layer");
}

extern "C" DL_API size_t dl_eval_net_shared_bytes(const int64_t *widths, int n_layers) {
    int64_t maxw = 0;
    for (int l = 1; l <= n_layers; ++l) maxw = widths[l] > maxw ? widths[l] : maxw;
    maxw = (maxw + 3) / 4 * 4;
    return (size_t)(2 * maxw * 8 + widths[0] * 32);
}

extern "C" DL_API int dl_eval_net_packed(const void *x, const uint32_t *meta, const int64_t *widths, int n_layers, int32_t *out,
                                         int64_t words, int64_t pad_len, int64_t k, int bit_count, void *stream) {
    DL_REQUIRE(bit_count == 8 || bit_count == 16 || bit_count == 32 || bit_count == 64, DL_ERR_BAD_BIT_COUNT,
               "dl_eval_net_packed: `bit_count` has to be in { 8, 16, 32, 64 }, got %d", bit_count);
    DL_REQUIRE(widths != nullptr && n_layers >= 1 && n_layers <= kNetMaxLayers, DL_ERR_INVALID_ARG,
               "dl_eval_net_packed: between 1 and %d layers", kNetMaxLayers);
    DL_REQUIRE(words >= 0 && k > 0 && pad_len >= 0 && pad_len < bit_count, DL_ERR_INVALID_ARG, "dl_eval_net_packed: bad size");
    NetDesc desc;
    desc.n_layers = n_layers;
    int64_t off = 0, maxw = 0;
    for (int l = 0; l <= n_layers; ++l) {
        DL_REQUIRE(widths[l] > 0 && widths[l] <= kNetMaxWidth, DL_ERR_TOO_LARGE,
                   "dl_eval_net_packed: layer %d has %lld rows; the fused kernel takes at most %d", l, (long long)widths[l],
                   kNetMaxWidth);
        desc.width[l] = (int)widths[l];
        if (l >= 1) {
            desc.meta_off[l - 1] = (int)off;
            off += (widths[l] + 3) / 4 * 4;
            maxw = widths[l] > maxw ? widths[l] : maxw;
        }
    }
    DL_REQUIRE(widths[n_layers] % k == 0, DL_ERR_NOT_DIVISIBLE, "in_dim (%lld) has to be divisible by k (%lld) but it is not",
               (long long)widths[n_layers], (long long)k);
    DL_REQUIRE(widths[n_layers] / k < 65536, DL_ERR_TOO_LARGE, "dl_eval_net_packed: more than 65535 rows per class");
    const int64_t row_bytes = words * (bit_count / 8);
    DL_REQUIRE(row_bytes % 8 == 0, DL_ERR_INVALID_ARG, "dl_eval_net_packed: rows must be a multiple of 8 bytes");
    const int64_t batch = words * bit_count - pad_len;
    if (batch <= 0) return DL_OK;
    DL_REQUIRE(x && meta && out, DL_ERR_INVALID_ARG, "dl_eval_net_packed: null pointer");
    DL_REQUIRE(aligned_to(x, 16) && aligned_to(meta, 16), DL_ERR_INVALID_ARG, "dl_eval_net_packed: x and meta must be 16-byte aligned");
    maxw = (maxw + 3) / 4 * 4;
    const size_t smem = (size_t)(2 * maxw * 8 + widths[0] * 32);
    DL_REQUIRE(smem <= 220 * 1024, DL_ERR_TOO_LARGE, "dl_eval_net_packed: needs %zu bytes of shared memory per CTA", smem);
    if (cudaFuncSetAttribute(eval_net_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return launch_status("dl_eval_net_packed (shared memory opt-in)");
    const int64_t words64 = row_bytes / 8;
    const int64_t ngroups = (words64 + 3) / 4;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned grid = (unsigned)(ngroups < sms ? ngroups : sms);
    // planes a thread's own counter needs, and planes of a whole class's count
    int tpc = (kNetThreads / (int)k) & ~31;
    if (tpc == 0) tpc = 32;
    const int64_t m = widths[n_layers] / k, rows_per_thread = ceil_div(m, tpc);
    int planes_thread = 1, planes_total = 1;
    while (((int64_t)1 << planes_thread) <= rows_per_thread) ++planes_thread;
    while (planes_total < kSumPlanes && ((int64_t)1 << planes_total) <= m) ++planes_total;
    eval_net_kernel<<<grid, kNetThreads, smem, as_stream(stream)>>>(reinterpret_cast<const u64 *>(x), meta, desc, out, words64,
                                                                   batch, (int)k, (int)maxw, planes_thread, planes_total);
    return launch_status("dl_eval_net_packed");
}
