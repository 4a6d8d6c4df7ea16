// One Adam step over a flat parameter vector, in a single kernel.
//
// The gate weights of all layers live in one flat fp32 buffer (and so do their gradients, first and
// second moments), so the optimizer step of a whole network is one elementwise pass with 16-byte
// accesses instead of one multi-tensor launch sequence.  The step counter stays on the device, which
// keeps the kernel capturable in a CUDA graph: every block reads it, the last block to finish
// increments it.
#include "adam_math.cuh"
#include "common.cuh"

namespace dl {

__global__ void __launch_bounds__(kThreads)
adam_kernel(float *__restrict__ p, const float *__restrict__ g, float *__restrict__ m, float *__restrict__ v, int64_t n, float lr,
            float beta1, float beta2, float eps, float grad_scale, int *__restrict__ state) {
    __shared__ float s_step_size, s_bc2_sqrt;
    // Everything that does not depend on the gradients happens BEFORE the wait for the kernels that write them, i.e.
    // while the last backward kernel is still running: the bias corrections (two powf), and this thread's first
    // elements of the parameters and moments, which only this kernel ever writes.
    if (threadIdx.x == 0) {
        const float t = (float)(state[0] + 1);
        s_step_size = lr / (1.f - powf(beta1, t));
        s_bc2_sqrt = sqrtf(1.f - powf(beta2, t));
    }
    const int64_t n4 = n / 4;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t first = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    float4 p0 = make_float4(0.f, 0.f, 0.f, 0.f), m0 = p0, v0 = p0;
    if (first < n4) {
        p0 = reinterpret_cast<float4 *>(p)[first];
        m0 = reinterpret_cast<float4 *>(m)[first];
        v0 = reinterpret_cast<float4 *>(v)[first];
    }
    // later passes (when the grid does not cover the vector): pull their elements towards L2
    for (int64_t i = first + stride; i < n4; i += stride) {
        prefetch_l2(reinterpret_cast<const char *>(p) + i * 16);
        prefetch_l2(reinterpret_cast<const char *>(m) + i * 16);
        prefetch_l2(reinterpret_cast<const char *>(v) + i * 16);
    }
    __syncthreads();
    const float step_size = s_step_size, bc2_sqrt = s_bc2_sqrt;
    const float omb1 = 1.f - beta1, omb2 = 1.f - beta2;
    grid_dependency_wait();  // gradients come from the kernels just before
    const AdamConsts consts = {omb1, beta2, omb2, step_size, bc2_sqrt, eps};
    for (int64_t i = first; i < n4; i += stride) {
        float4 pp, mm, vv;
        if (i == first) {
            pp = p0; mm = m0; vv = v0;
        } else {
            pp = reinterpret_cast<float4 *>(p)[i];
            mm = reinterpret_cast<float4 *>(m)[i];
            vv = reinterpret_cast<float4 *>(v)[i];
        }
        float4 gg = __ldg(reinterpret_cast<const float4 *>(g) + i);
        gg.x = __fmul_rn(gg.x, grad_scale); gg.y = __fmul_rn(gg.y, grad_scale);
        gg.z = __fmul_rn(gg.z, grad_scale); gg.w = __fmul_rn(gg.w, grad_scale);
        adam_update4(pp, gg, mm, vv, consts);
        reinterpret_cast<float4 *>(p)[i] = pp;
        reinterpret_cast<float4 *>(m)[i] = mm;
        reinterpret_cast<float4 *>(v)[i] = vv;
    }
    for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        float pi = p[i], mi = m[i], vi = v[i];
        adam_update(pi, __fmul_rn(g[i], grad_scale), mi, vi, consts);
        p[i] = pi;
        m[i] = mi;
        v[i] = vi;
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

// Pulls a range of memory towards L2, one 128-byte line per thread and pass.  Used to warm the optimizer's moments
// while the backward pass is still running: they are touched once per step, so they are never in L2 by themselves.
__global__ void __launch_bounds__(kThreads) prefetch_l2_kernel(const char *__restrict__ p, int64_t lines) {
    for (int64_t l = (int64_t)blockIdx.x * kThreads + threadIdx.x; l < lines; l += (int64_t)gridDim.x * kThreads)
        prefetch_l2(p + l * 128);
}

}  // namespace dl

extern "C" DL_API int dl_prefetch_l2(const void *ptr, size_t bytes, void *stream) {
    using namespace dl;
    if (bytes == 0) return DL_OK;
    DL_REQUIRE(ptr != nullptr, DL_ERR_INVALID_ARG, "dl_prefetch_l2: null pointer");
    const int64_t lines = (int64_t)((bytes + 127) / 128);
    int64_t blocks = ceil_div(lines, kThreads);
    if (blocks > 148 * 2) blocks = 148 * 2;  // a small grid: it runs beside other kernels
    prefetch_l2_kernel<<<(unsigned)blocks, kThreads, 0, as_stream(stream)>>>(reinterpret_cast<const char *>(ptr), lines);
    return launch_status("dl_prefetch_l2");
}

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
