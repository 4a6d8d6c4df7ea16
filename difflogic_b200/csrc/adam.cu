// One Adam step over a flat parameter vector, in a single kernel.
//
// The gate weights of all layers live in one flat fp32 buffer (and so do their gradients, first and
// second moments), so the optimizer step of a whole network is one elementwise pass with 16-byte
// accesses instead of one multi-tensor launch sequence.  The step counter stays on the device, which
// keeps the kernel capturable in a CUDA graph: every block reads it, the last block to finish
// increments it.
#include "common.cuh"

namespace dl {

__global__ void __launch_bounds__(kThreads)
adam_kernel(float *__restrict__ p, const float *__restrict__ g, float *__restrict__ m, float *__restrict__ v, int64_t n, float lr,
            float beta1, float beta2, float eps, float grad_scale, int *__restrict__ state) {
    __shared__ float s_step_size, s_bc2_sqrt;
    {
        // set-up: pull this thread's slices of the parameters and moments towards L2 (128-byte lines) while the
        // last backward kernel is still running
        const int64_t lines = (n * 4 + 127) / 128;
        for (int64_t l = (int64_t)blockIdx.x * kThreads + threadIdx.x; l < lines; l += (int64_t)gridDim.x * kThreads) {
            prefetch_l2(reinterpret_cast<const char *>(p) + l * 128);
            prefetch_l2(reinterpret_cast<const char *>(m) + l * 128);
            prefetch_l2(reinterpret_cast<const char *>(v) + l * 128);
        }
    }
    grid_dependency_wait();  // gradients come from the kernels just before
    if (threadIdx.x == 0) {
        const float t = (float)(state[0] + 1);
        s_step_size = lr / (1.f - powf(beta1, t));
        s_bc2_sqrt = sqrtf(1.f - powf(beta2, t));
    }
    __syncthreads();
    const float step_size = s_step_size, bc2_sqrt = s_bc2_sqrt;
    const float omb1 = 1.f - beta1, omb2 = 1.f - beta2;
    const int64_t n4 = n / 4;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride) {
        float4 pp = reinterpret_cast<float4 *>(p)[i];
        float4 gg = __ldg(reinterpret_cast<const float4 *>(g) + i);
        float4 mm = reinterpret_cast<float4 *>(m)[i];
        float4 vv = reinterpret_cast<float4 *>(v)[i];
#define DL_ADAM1(c)                                          \
    {                                                        \
        const float gr = gg.c * grad_scale;                  \
        mm.c = mm.c + (gr - mm.c) * omb1;                    \
        vv.c = vv.c * beta2 + gr * gr * omb2;                \
        const float denom = sqrtf(vv.c) / bc2_sqrt + eps;    \
        pp.c = pp.c - step_size * (mm.c / denom);            \
    }
        DL_ADAM1(x) DL_ADAM1(y) DL_ADAM1(z) DL_ADAM1(w)
#undef DL_ADAM1
        reinterpret_cast<float4 *>(p)[i] = pp;
        reinterpret_cast<float4 *>(m)[i] = mm;
        reinterpret_cast<float4 *>(v)[i] = vv;
    }
    for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float gr = g[i] * grad_scale;
        const float mi = m[i] + (gr - m[i]) * omb1;
        const float vi = v[i] * beta2 + gr * gr * omb2;
        m[i] = mi;
        v[i] = vi;
        p[i] = p[i] - step_size * (mi / (sqrtf(vi) / bc2_sqrt + eps));
    }
    // the last block to get here advances the step counter and re-arms the ticket
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const int done = atomicAdd(state + 1, 1);
        if (done == (int)gridDim.x - 1) {
            state[1] = 0;
            state[0] = state[0] + 1;
        }
    }
}

}  // namespace dl

extern "C" DL_API int dl_adam_step_f32(float *param, const float *grad, float *exp_avg, float *exp_avg_sq, int64_t n, float lr,
                                       float beta1, float beta2, float eps, float grad_scale, int32_t *state, void *stream) {
    using namespace dl;
    DL_REQUIRE(n >= 0, DL_ERR_INVALID_ARG, "dl_adam_step_f32: negative size");
    DL_REQUIRE(state != nullptr, DL_ERR_INVALID_ARG, "dl_adam_step_f32: null state");
    DL_REQUIRE(n == 0 || (param && grad && exp_avg && exp_avg_sq), DL_ERR_INVALID_ARG, "dl_adam_step_f32: null pointer");
    DL_REQUIRE(aligned_to(param, 16) && aligned_to(grad, 16) && aligned_to(exp_avg, 16) && aligned_to(exp_avg_sq, 16),
               DL_ERR_INVALID_ARG, "dl_adam_step_f32: buffers must be 16-byte aligned");
    int64_t blocks = ceil_div(n / 4 > 0 ? n / 4 : 1, kThreads);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (launch_dependent(true, adam_kernel, dim3((unsigned)blocks), dim3(kThreads), 0, as_stream(stream), param, grad, exp_avg,
                         exp_avg_sq, n, lr, beta1, beta2, eps, grad_scale, reinterpret_cast<int *>(state)) != cudaSuccess)
        return launch_status("dl_adam_step_f32");
    return launch_status("dl_adam_step_f32");
}
