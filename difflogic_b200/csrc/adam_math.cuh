// The Adam update of one element, with every rounding spelled out so that each kernel that applies it (the
// single-GPU step and the multi-GPU exchange) produces the same bits whatever the compiler makes of the code around it
// (left to itself it contracts a * b + c * d into one of two different fused multiply-adds).
//
// torch.optim.Adam without weight decay or amsgrad (as used at experiments/main.py:169):
//   m <- m + (g - m)(1 - beta1);  v <- v beta2 + g g (1 - beta2);  p <- p - step_size * m / (sqrt(v) / bc2_sqrt + eps)
// with step_size = lr / (1 - beta1^t) and bc2_sqrt = sqrt(1 - beta2^t).
#pragma once

#include <cuda_runtime.h>

namespace dl {

struct AdamConsts {
    float omb1, beta2, omb2, step_size, bc2_sqrt, eps;
};

__device__ __forceinline__ void adam_update(float &p, float g, float &m, float &v, const AdamConsts &c) {
    m = __fmaf_rn(__fsub_rn(g, m), c.omb1, m);
    v = __fmaf_rn(v, c.beta2, __fmul_rn(__fmul_rn(g, g), c.omb2));
    const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), c.bc2_sqrt), c.eps);
    p = __fmaf_rn(-c.step_size, __fdiv_rn(m, denom), p);
}

__device__ __forceinline__ void adam_update4(float4 &p, const float4 &g, float4 &m, float4 &v, const AdamConsts &c) {
    adam_update(p.x, g.x, m.x, v.x, c);
    adam_update(p.y, g.y, m.y, v.y, c);
    adam_update(p.z, g.z, m.z, v.z, c);
    adam_update(p.w, g.w, m.w, v.w, c);
}

}  // namespace dl
