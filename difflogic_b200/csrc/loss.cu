// Cross-entropy loss on the class scores of a GroupSum: [batch][k] fp32 logits, int64 class targets, mean over
// the batch -- the loss the reference's training loop applies to the network output
// (torch.nn.CrossEntropyLoss, experiments/main.py:167,175).  torch runs it as six small kernels; for the few
// kilobytes involved one kernel each way is enough, and with programmatic dependent launch its set-up
// overlaps the GroupSum kernel before it.
//
// forward : p = softmax(logits[s]);  loss = -(1/B) sum_s log p[s][target_s];  probs (= p) is kept for backward
// backward: grad_logits[s][c] = (p[s][c] - [c == target_s]) * grad_loss / B
#include "common.cuh"

namespace dl {

constexpr int kCeThreads = 1024;

__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(const float *__restrict__ logits, const int64_t *__restrict__ target, float *__restrict__ loss,
                     float *__restrict__ probs, int64_t batch, int k) {
    __shared__ float s_partial[kCeThreads / 32];
    grid_dependency_wait();
    float local = 0.f;
    for (int64_t s = threadIdx.x; s < batch; s += kCeThreads) {
        const float *row = logits + s * k;
        float m = -INFINITY;
        for (int c = 0; c < k; ++c) m = fmaxf(m, row[c]);
        float sum = 0.f;
        for (int c = 0; c < k; ++c) sum += expf(row[c] - m);
        const float lse = m + logf(sum);
        for (int c = 0; c < k; ++c) probs[s * k + c] = expf(row[c] - lse);
        const int64_t t = target[s];
        if (t >= 0 && t < k) local += lse - row[t];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    if (threadIdx.x % 32 == 0) s_partial[threadIdx.x / 32] = local;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < kCeThreads / 32 ? s_partial[threadIdx.x] : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (threadIdx.x == 0) loss[0] = v / (float)batch;
    }
}

__global__ void __launch_bounds__(kThreads)
cross_entropy_backward_kernel(const float *__restrict__ probs, const int64_t *__restrict__ target,
                              const float *__restrict__ grad_loss, float *__restrict__ grad_logits, int64_t batch, int k) {
    grid_dependency_wait();
    const float scale = grad_loss[0] / (float)batch;
    const int64_t total = batch * k;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kThreads) {
        const int64_t s = i / k;
        const int c = (int)(i % k);
        grad_logits[i] = (probs[i] - (target[s] == c ? 1.f : 0.f)) * scale;
    }
}

}  // namespace dl

using namespace dl;

extern "C" DL_API int dl_cross_entropy_f32(const float *logits, const int64_t *target, float *loss, float *probs, int64_t batch,
                                           int64_t k, void *stream) {
    DL_REQUIRE(batch > 0 && k > 0 && k <= INT32_MAX, DL_ERR_INVALID_ARG, "dl_cross_entropy_f32: bad size");
    DL_REQUIRE(logits && target && loss && probs, DL_ERR_INVALID_ARG, "dl_cross_entropy_f32: null pointer");
    launch_dependent(true, cross_entropy_kernel, dim3(1), dim3(kCeThreads), 0, as_stream(stream), logits, target, loss, probs,
                     batch, (int)k);
    return launch_status("dl_cross_entropy_f32");
}

extern "C" DL_API int dl_cross_entropy_backward_f32(const float *probs, const int64_t *target, const float *grad_loss,
                                                    float *grad_logits, int64_t batch, int64_t k, void *stream) {
    DL_REQUIRE(batch > 0 && k > 0 && k <= INT32_MAX, DL_ERR_INVALID_ARG, "dl_cross_entropy_backward_f32: bad size");
    DL_REQUIRE(probs && target && grad_loss && grad_logits, DL_ERR_INVALID_ARG, "dl_cross_entropy_backward_f32: null pointer");
    int64_t blocks = ceil_div(batch * k, kThreads);
    if (blocks > 148 * 4) blocks = 148 * 4;
    launch_dependent(true, cross_entropy_backward_kernel, dim3((unsigned)blocks), dim3(kThreads), 0, as_stream(stream), probs,
                     target, grad_loss, grad_logits, batch, (int)k);
    return launch_status("dl_cross_entropy_backward_f32");
}
