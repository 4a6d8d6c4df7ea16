// Thermometer encoding and bit packing in one pass, straight from uint8 features.
//
// The reference's image pipeline turns every pixel into T binary features (pixel / 255 > (i+1) / (T+1)),
// concatenated threshold-major (experiments/main.py:56-59), then PackBitsTensor transposes and packs the float
// or bool matrix (difflogic/packbitstensor.py:15-16).  For 2^20 samples that is gigabytes of intermediate bools.
// Here the uint8 matrix t[batch][n] is read once (for up to four thresholds at a time) and the packed rows
// out[i*n + f][word] come out directly: bit s of row i*n + f is  t[s][f] > thresholds[i].
//
// n % 8 == 0: the tile packer of pack_tile.cuh (256 features x 512 samples per CTA, 8-byte loads, bits moved eight by
// eight).  Any other n: the 128 x 512 tiling of packbits_bm_kernel, one threshold per pass, one bit at a time.
#include "common.cuh"
#include "pack_tile.cuh"

namespace dl {

constexpr int kMaxThresholds = 16;
struct Thresholds {
    unsigned char v[kMaxThresholds];
};

// n % 8 == 0: 8-byte loads, bits moved eight by eight (pack_tile.cuh); NT thresholds per pass over the source
// (blockIdx.z walks groups of NT thresholds), so the pixels are read once for up to kThresholdsPerPass of them.
constexpr int kThresholdsPerPass = 4;

template <int NT>
struct MaskAbove {
    uint32_t th4[NT];  // the threshold in every byte
    __device__ __forceinline__ uint32_t operator()(uint32_t lo, uint32_t hi, int i) const {
        return squeeze8_ones(__vcmpgtu4(lo, th4[i]) & 0x01010101u, __vcmpgtu4(hi, th4[i]) & 0x01010101u);
    }
};

template <int NT>
__global__ void __launch_bounds__(kThreads, 2)
threshold_pack8_kernel(const uint8_t *__restrict__ t, Thresholds thr, int first, uint8_t *__restrict__ out, int64_t n, int64_t batch,
                       int64_t row_bytes) {
    __shared__ unsigned long long s_words[8 * kPackRow];
    const int64_t f0 = (int64_t)blockIdx.x * kPackFeatures;
    MaskAbove<NT> mask;
#pragma unroll
    for (int i = 0; i < NT; ++i) mask.th4[i] = (uint32_t)thr.v[first + i] * 0x01010101u;
    uint8_t *dst = out + (int64_t)first * n * row_bytes;
    for (int64_t sblk = blockIdx.y; sblk * kPackSamples < row_bytes * 8; sblk += gridDim.y)
        pack_tile<NT>(t, dst, n * row_bytes, n, batch, row_bytes, f0, sblk, s_words, mask);
}

template <bool VEC4>
__global__ void __launch_bounds__(kThreads)
threshold_pack_kernel(const uint8_t *__restrict__ t, Thresholds thr, uint8_t *__restrict__ out, int64_t n, int64_t batch,
                      int64_t row_bytes) {
    __shared__ unsigned long long s_words[128][9];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int64_t f0 = (int64_t)blockIdx.x * 128;
    const uint32_t th = thr.v[blockIdx.z];
    const uint32_t th4 = th * 0x01010101u;
    uint8_t *dst = out + (int64_t)blockIdx.z * n * row_bytes;
    for (int64_t sblk = blockIdx.y; sblk * 512 < batch; sblk += gridDim.y) {
        const int64_t s0 = sblk * 512 + warp * 64;
        unsigned long long wd[4] = {0ull, 0ull, 0ull, 0ull};
        const int64_t f = f0 + lane * 4;
        if (VEC4) {
            if (f < n) {
#pragma unroll 16
                for (int s = 0; s < 64; ++s) {
                    if (s0 + s < batch) {
                        const uint32_t px = __ldg(reinterpret_cast<const uint32_t *>(t + (s0 + s) * n + f));
                        const uint32_t v = __vcmpgtu4(px, th4);  // 0xff in every byte that is above the threshold
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
                        if (f + q < n) wd[q] |= (unsigned long long)(__ldg(t + (s0 + s) * n + f + q) > th) << s;
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) s_words[lane * 4 + q][warp] = wd[q];
        __syncthreads();
        const int64_t byte0 = sblk * 64;
        for (int idx = threadIdx.x; idx < 128 * 64; idx += kThreads) {
            const int fl = idx / 64, by = idx % 64;
            if (f0 + fl < n && byte0 + by < row_bytes)
                dst[(f0 + fl) * row_bytes + byte0 + by] = (uint8_t)(s_words[fl][by / 8] >> (8 * (by % 8)));
        }
        __syncthreads();
    }
}

}  // namespace dl

using namespace dl;

extern "C" DL_API int dl_threshold_packbits_batch_major(const uint8_t *t, const uint8_t *thresholds, int n_thresholds, void *out,
                                                        int64_t n, int64_t batch, int bit_count, void *stream) {
    DL_REQUIRE(bit_count == 8 || bit_count == 16 || bit_count == 32 || bit_count == 64, DL_ERR_BAD_BIT_COUNT,
               "dl_threshold_packbits_batch_major: `bit_count` has to be in { 8, 16, 32, 64 }, got %d", bit_count);
    DL_REQUIRE(n >= 0 && batch >= 0, DL_ERR_INVALID_ARG, "dl_threshold_packbits_batch_major: negative size");
    DL_REQUIRE(thresholds != nullptr && n_thresholds >= 1 && n_thresholds <= kMaxThresholds, DL_ERR_INVALID_ARG,
               "dl_threshold_packbits_batch_major: between 1 and %d thresholds (a host array)", kMaxThresholds);
    if (n == 0 || batch == 0) return DL_OK;
    DL_REQUIRE(t && out, DL_ERR_INVALID_ARG, "dl_threshold_packbits_batch_major: null pointer");
    Thresholds thr;
    for (int i = 0; i < kMaxThresholds; ++i) thr.v[i] = i < n_thresholds ? thresholds[i] : 0;
    const int64_t row_bytes = ceil_div(batch, bit_count) * (bit_count / 8);
    const int64_t sblocks = ceil_div(row_bytes, 64);
    const dim3 grid((unsigned)ceil_div(n, 128), (unsigned)(sblocks < 65535 ? sblocks : 65535), (unsigned)n_thresholds);
    uint8_t *o = reinterpret_cast<uint8_t *>(out);
    if (n % 8 == 0 && aligned_to(t, 8)) {
        const int64_t sb = ceil_div(row_bytes, kPackSamples / 8);
        const dim3 grid8((unsigned)ceil_div(n, kPackFeatures), (unsigned)(sb < 65535 ? sb : 65535));
        for (int first = 0; first < n_thresholds; first += kThresholdsPerPass) {
            switch (n_thresholds - first < kThresholdsPerPass ? n_thresholds - first : kThresholdsPerPass) {
                case 1: threshold_pack8_kernel<1><<<grid8, kThreads, 0, as_stream(stream)>>>(t, thr, first, o, n, batch, row_bytes); break;
                case 2: threshold_pack8_kernel<2><<<grid8, kThreads, 0, as_stream(stream)>>>(t, thr, first, o, n, batch, row_bytes); break;
                case 3: threshold_pack8_kernel<3><<<grid8, kThreads, 0, as_stream(stream)>>>(t, thr, first, o, n, batch, row_bytes); break;
                default: threshold_pack8_kernel<4><<<grid8, kThreads, 0, as_stream(stream)>>>(t, thr, first, o, n, batch, row_bytes); break;
            }
        }
    } else if (n % 4 == 0 && aligned_to(t, 4))
        threshold_pack_kernel<true><<<grid, kThreads, 0, as_stream(stream)>>>(t, thr, o, n, batch, row_bytes);
    else
        threshold_pack_kernel<false><<<grid, kThreads, 0, as_stream(stream)>>>(t, thr, o, n, batch, row_bytes);
    return launch_status("dl_threshold_packbits_batch_major");
}
