// Bit-sliced vertical counter: counts, for each of the 64 bit positions of a word, how many of the
// words fed to it have that bit set.  A carry-save adder tree turns every 8 input words into one
// word of weight 8 that ripples into the high planes, so a word costs about two LOP3 per input
// instead of one add per bit.
#pragma once

#include <stdint.h>

namespace dl {

#define DL_CSA(h, l, a, b, c)               \
    {                                       \
        const unsigned long long u_ = (a) ^ (b); \
        const unsigned long long c_ = (c);  \
        h = ((a) & (b)) | (u_ & c_);        \
        l = u_ ^ c_;                        \
    }

constexpr int kHiPlanes = 9;                      // weights 8 .. 2048
constexpr int kPlanes = 3 + kHiPlanes;            // ones, twos, fours + high planes
constexpr int kMaxChunkRows = 8 * (1 << kHiPlanes) - 1;  // 4095

// HI = number of planes above ones / twos / fours: counts up to 8 * 2^HI - 1.
template <int HI>
struct BitCounterT {
    unsigned long long ones, twos, fours, hi[HI];
    __device__ __forceinline__ void clear() {
        ones = twos = fours = 0ull;
#pragma unroll
        for (int q = 0; q < HI; ++q) hi[q] = 0ull;
    }
    __device__ __forceinline__ void add8(const unsigned long long (&v)[8]) {
        unsigned long long t2a, t2b, t4a, t4b, e8;
        DL_CSA(t2a, ones, ones, v[0], v[1]);
        DL_CSA(t2b, ones, ones, v[2], v[3]);
        DL_CSA(t4a, twos, twos, t2a, t2b);
        DL_CSA(t2a, ones, ones, v[4], v[5]);
        DL_CSA(t2b, ones, ones, v[6], v[7]);
        DL_CSA(t4b, twos, twos, t2a, t2b);
        DL_CSA(e8, fours, fours, t4a, t4b);
        unsigned long long carry = e8;
#pragma unroll
        for (int q = 0; q < HI; ++q) {
            const unsigned long long t = hi[q] & carry;
            hi[q] ^= carry;
            carry = t;
        }
    }
    __device__ __forceinline__ void add1(unsigned long long v) {
        unsigned long long carry = v, t;
        t = ones & carry; ones ^= carry; carry = t;
        t = twos & carry; twos ^= carry; carry = t;
        t = fours & carry; fours ^= carry; carry = t;
#pragma unroll
        for (int q = 0; q < HI; ++q) {
            t = hi[q] & carry;
            hi[q] ^= carry;
            carry = t;
        }
    }
    __device__ __forceinline__ unsigned long long plane(int p) const {
        return p == 0 ? ones : p == 1 ? twos : p == 2 ? fours : hi[p - 3];
    }
};

using BitCounter = BitCounterT<kHiPlanes>;

}  // namespace dl
