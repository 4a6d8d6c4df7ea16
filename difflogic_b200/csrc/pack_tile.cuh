// Transpose-and-pack of a batch-major byte matrix t[batch][n] into feature-major bit rows, shared by the bool packer
// (packed.cu) and the thermometer packer (threshold_pack.cu).
//
// A CTA of 256 threads takes 256 features x 512 samples.  Warp w owns the 64 samples of one output word, lane l eight
// adjacent features: one 8-byte load per sample, so a warp reads 256 contiguous bytes of a sample's row.  No bit is
// moved on its own:
//   * a predicate turns the 8 bytes of a load into 8 bits (bit f = feature f selected): two multiplies and a shift;
//   * 8 samples give an 8 x 8 bit matrix (byte = sample, bit = feature) that is transposed in registers by three delta
//     swaps: byte f then holds the 8 samples' bits of feature f;
//   * after 8 such groups an 8 x 8 BYTE transpose across the 8 registers (byte permutes) gives the 8 output words, one
//     per feature.
// The words of the 8 warps meet in shared memory so that a feature's 64 bytes (512 samples) leave as 16-byte stores
// (words stored straight from the registers, 8 bytes at a time to 8 different rows per thread, measured slower: 382
// against 337 us for 2^20 x 784 bools, and twice as slow with three outputs).
// Needs n % 8 == 0 and an 8-byte aligned source; rows of the output need no alignment (ragged ends go byte by byte).
#pragma once

#include "common.cuh"

namespace dl {

constexpr int kPackFeatures = 256;  // per CTA
constexpr int kPackSamples = 512;   // per CTA and pass
constexpr int kPackRow = 8 * 33 + 1;  // shared-memory row (one per warp): 8 blocks of 32 lanes, padded

// 0x01 in every selected byte of lo / hi -> 8 bits (byte 0 of lo to bit 0): the two products put the bytes' low bits
// next to each other in bits 24..31 and overlap nowhere, so the sum cannot carry
__device__ __forceinline__ uint32_t squeeze8_ones(uint32_t lo_ones, uint32_t hi_ones) {
    return (lo_ones * 0x01020408u + hi_ones * 0x10204080u) >> 24;
}
// 0x01 in every non-zero byte
__device__ __forceinline__ uint32_t nonzero_bytes(uint32_t v) { return ((((v & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | v) >> 7) & 0x01010101u; }

// 8 x 8 bit matrix in a 64-bit word, byte = row: transposed (byte = column)
__device__ __forceinline__ unsigned long long transpose_bits_8x8(unsigned long long x) {
    unsigned long long t;
    t = (x ^ (x >> 7)) & 0x00AA00AA00AA00AAull;
    x ^= t ^ (t << 7);
    t = (x ^ (x >> 14)) & 0x0000CCCC0000CCCCull;
    x ^= t ^ (t << 14);
    t = (x ^ (x >> 28)) & 0x00000000F0F0F0F0ull;
    x ^= t ^ (t << 28);
    return x;
}

// r[i] byte j  <-  v[j] byte i   for four 32-bit values
__device__ __forceinline__ void transpose_bytes_4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t r[4]) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);  // a0 b0 a1 b1 | c0 d0 c1 d1
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);  // a2 b2 a3 b3 | c2 d2 c3 d3
    r[0] = __byte_perm(t0, t1, 0x5410);
    r[1] = __byte_perm(t0, t1, 0x7632);
    r[2] = __byte_perm(t2, t3, 0x5410);
    r[3] = __byte_perm(t2, t3, 0x7632);
}

// MASK: functor (lo, hi: the 8 bytes of one load; i: which of the NT outputs) -> 8 bits, bit f set when feature f is selected
// for output i.  The source is read ONCE for all NT outputs (e.g. NT thermometer thresholds).  Output i goes to the rows
// starting at dst + i * out_stride (row_bytes bytes per feature row); s_words: kPackRow * 8 words.  Samples beyond the
// batch give zero bits.
template <int NT, typename MASK>
__device__ __forceinline__ void pack_tile(const uint8_t *__restrict__ t, uint8_t *__restrict__ dst, int64_t out_stride, int64_t n,
                                          int64_t batch, int64_t row_bytes, int64_t f0, int64_t sblk, unsigned long long *s_words,
                                          MASK mask) {
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int64_t f = f0 + lane * 8;
    const int64_t s0 = sblk * kPackSamples + warp * 64;
    const int live = f < n ? (int)max((int64_t)0, min((int64_t)64, batch - s0)) : 0;  // samples of this thread's item that exist
    const uint8_t *src = t + s0 * n + f;
    unsigned long long grp[NT][8];  // per output and group of 8 samples: byte f = the 8 samples' bits of feature f
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        uint2 v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            v[r] = make_uint2(0u, 0u);
            if (g * 8 + r < live) v[r] = __ldg(reinterpret_cast<const uint2 *>(src + (int64_t)(g * 8 + r) * n));
        }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            uint32_t xlo = 0u, xhi = 0u;  // byte r = the mask of sample r
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                xlo |= (g * 8 + r < live ? mask(v[r].x, v[r].y, i) : 0u) << (8 * r);
                xhi |= (g * 8 + 4 + r < live ? mask(v[4 + r].x, v[4 + r].y, i) : 0u) << (8 * r);
            }
            grp[i][g] = transpose_bits_8x8((unsigned long long)xlo | ((unsigned long long)xhi << 32));
        }
    }
    const int64_t byte0 = sblk * (kPackSamples / 8);
    const bool wide = row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(dst) % 16) == 0 && out_stride % 16 == 0;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        // word of feature q: byte g = grp[g] byte q
        uint32_t lo_a[4], lo_b[4], hi_a[4], hi_b[4];
        transpose_bytes_4x4((uint32_t)grp[i][0], (uint32_t)grp[i][1], (uint32_t)grp[i][2], (uint32_t)grp[i][3], lo_a);  // features 0..3, groups 0..3
        transpose_bytes_4x4((uint32_t)grp[i][4], (uint32_t)grp[i][5], (uint32_t)grp[i][6], (uint32_t)grp[i][7], lo_b);  // features 0..3, groups 4..7
        transpose_bytes_4x4((uint32_t)(grp[i][0] >> 32), (uint32_t)(grp[i][1] >> 32), (uint32_t)(grp[i][2] >> 32),
                            (uint32_t)(grp[i][3] >> 32), hi_a);                                                       // features 4..7
        transpose_bytes_4x4((uint32_t)(grp[i][4] >> 32), (uint32_t)(grp[i][5] >> 32), (uint32_t)(grp[i][6] >> 32),
                            (uint32_t)(grp[i][7] >> 32), hi_b);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            s_words[warp * kPackRow + q * 33 + lane] = (unsigned long long)lo_a[q] | ((unsigned long long)lo_b[q] << 32);
            s_words[warp * kPackRow + (q + 4) * 33 + lane] = (unsigned long long)hi_a[q] | ((unsigned long long)hi_b[q] << 32);
        }
        __syncthreads();
        // a feature's eight words (64 bytes) leave as four 16-byte stores; ragged ends and unaligned rows byte by byte
        uint8_t *rows = dst + (int64_t)i * out_stride;
        for (int idx = threadIdx.x; idx < kPackFeatures * 4; idx += kThreads) {
            const int fl = idx / 4, piece = idx % 4;
            if (f0 + fl >= n) continue;
            const int at = (fl % 8) * 33 + fl / 8;
            const unsigned long long w0 = s_words[(2 * piece) * kPackRow + at], w1 = s_words[(2 * piece + 1) * kPackRow + at];
            uint8_t *o = rows + (f0 + fl) * row_bytes + byte0 + 16 * piece;
            const int64_t left = row_bytes - (byte0 + 16 * piece);
            if (left >= 16 && wide) {
                *reinterpret_cast<uint4 *>(o) = make_uint4((uint32_t)w0, (uint32_t)(w0 >> 32), (uint32_t)w1, (uint32_t)(w1 >> 32));
            } else {
                for (int by = 0; by < 16 && by < left; ++by) o[by] = (uint8_t)((by < 8 ? w0 : w1) >> (8 * (by % 8)));
            }
        }
        __syncthreads();
    }
}

}  // namespace dl
