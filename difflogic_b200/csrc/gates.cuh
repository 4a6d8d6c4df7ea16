// The 16 two-input gates: truth-table algebra shared by the training and the packed kernels.
//
// Gate id i encodes its truth table as  i = 8*f(0,0) + 4*f(0,1) + 2*f(1,0) + f(1,1)
// (reference: difflogic/functional.py:7-24).  Every real-valued relaxation of the reference
// (functional.py:31-62) is the multilinear extension of that table,
//     f(A,B) = t00 + (t10-t00) A + (t01-t00) B + (t00-t01-t10+t11) A B,
// so a probability mix over the gates collapses to four coefficients per neuron.
#pragma once

#include "common.cuh"

namespace dl {

__device__ __forceinline__ int first_argmax16(const float *__restrict__ w) {
    int best = 0;
    float m = __ldg(w);
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        const float v = __ldg(w + i);
        if (v > m) { m = v; best = i; }
    }
    return best;
}

// ---------------------------------------------------------------------------------------------
// Coefficients of one neuron computed by four adjacent lanes (a "quad"), lane q holding gates
// 4q .. 4q+3: softmax / pass-through / arg-max one-hot over the 16 weights, then the sum over
// the gates of p_i times the gate's multilinear coefficients.  All 32 lanes of the warp call it.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

__device__ __forceinline__ float4 quad_coef(const float *__restrict__ wq, bool live, int q, int w_mode) {
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = live ? __ldg(wq + i) : 0.f;
    if (w_mode == DL_W_LOGITS) {
        float m = fmaxf(fmaxf(p[0], p[1]), fmaxf(p[2], p[3]));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) { p[i] = expf(p[i] - m); s += p[i]; }
        s = quad_sum(s);
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = p[i] / s;
    } else if (w_mode == DL_W_ARGMAX) {
        int best = 0;
        float m = p[0];
#pragma unroll
        for (int i = 1; i < 4; ++i) if (p[i] > m) { m = p[i]; best = i; }
        int gbest = 4 * q + best;
#pragma unroll
        for (int off = 1; off <= 2; off <<= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, off);
            const int og = __shfl_xor_sync(0xffffffffu, gbest, off);
            if (om > m || (om == m && og < gbest)) { m = om; gbest = og; }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = (4 * q + i == gbest) ? 1.f : 0.f;
    }
    // gate 4q+i has truth table t00 = q>>1, t01 = q&1, t10 = i>>1, t11 = i&1
    const int t00 = q >> 1, t01 = q & 1;
    float c0 = 0.f, ca = 0.f, cb = 0.f, cab = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t10 = i >> 1, t11 = i & 1;
        c0 += p[i] * (float)t00;
        ca += p[i] * (float)(t10 - t00);
        cb += p[i] * (float)(t01 - t00);
        cab += p[i] * (float)(t00 - t01 - t10 + t11);
    }
    return make_float4(quad_sum(c0), quad_sum(ca), quad_sum(cb), quad_sum(cab));
}

// The layer's output from the four coefficients c = {c0, ca, cb, cab}: c0 + ca A + cb B + cab A B, in one fixed order of
// fused multiply-adds (every forward kernel uses this function, so they agree to the bit).
__device__ __forceinline__ float4 mixv(const float4 c, const float4 a, const float4 b) {
    float4 r;
    r.x = fmaf(c.w, a.x * b.x, fmaf(c.y, a.x, fmaf(c.z, b.x, c.x)));
    r.y = fmaf(c.w, a.y * b.y, fmaf(c.y, a.y, fmaf(c.z, b.y, c.x)));
    r.z = fmaf(c.w, a.z * b.z, fmaf(c.y, a.z, fmaf(c.z, b.z, c.x)));
    r.w = fmaf(c.w, a.w * b.w, fmaf(c.y, a.w, fmaf(c.z, b.w, c.x)));
    return r;
}
__device__ __forceinline__ float mixv(const float4 c, const float a, const float b) {
    return fmaf(c.w, a * b, fmaf(c.y, a, fmaf(c.z, b, c.x)));
}

// dL/dp_i from the four batch sums S = {sum g, sum A g, sum B g, sum A B g}.
__device__ __forceinline__ float gate_grad_from_sums(int i, float s0, float sa, float sb, float sab) {
    const int t00 = (i >> 3) & 1, t01 = (i >> 2) & 1, t10 = (i >> 1) & 1, t11 = i & 1;
    return (float)t00 * s0 + (float)(t10 - t00) * sa + (float)(t01 - t00) * sb + (float)(t00 - t01 - t10 + t11) * sab;
}

// Bitwise gate in algebraic normal form: y = m0 ^ (ma & A) ^ (mb & B) ^ (mab & A & B),
// each mask all-ones or zero (reference gate list: difflogic_kernel.cu:437-472).
struct GateMasks {
    uint32_t m0, ma, mb, mab;
};
__device__ __forceinline__ GateMasks gate_masks(int op) {
    const uint32_t t00 = (op >> 3) & 1, t01 = (op >> 2) & 1, t10 = (op >> 1) & 1, t11 = op & 1;
    GateMasks g;
    g.m0 = 0u - t00;
    g.ma = 0u - (t00 ^ t10);
    g.mb = 0u - (t00 ^ t01);
    g.mab = 0u - (t00 ^ t01 ^ t10 ^ t11);
    return g;
}
// Whether gate `op` depends on its first (which = 0) or second (which = 1) input at all.  Six of the sixteen gates do not
// need both: false and true need none, A, not A, B and not B need one.  The masks above are zero for an input that
// is not needed, so whatever stands in its place is ignored.
__device__ __forceinline__ bool gate_needs_input(uint32_t op, int which) {
    const uint32_t t00 = (op >> 3) & 1, t01 = (op >> 2) & 1, t10 = (op >> 1) & 1, t11 = op & 1;
    return which == 0 ? ((t00 ^ t10) | (t01 ^ t11)) != 0 : ((t00 ^ t01) | (t10 ^ t11)) != 0;
}
__device__ __forceinline__ uint32_t gate32(uint32_t a, uint32_t b, const GateMasks &g) {
    return g.m0 ^ (g.ma & a) ^ (g.mb & b) ^ (g.mab & a & b);
}

}  // namespace dl
