// Training forward for long rows (batch >= 256): the two gathered input rows of every neuron staged in shared memory by
// bulk asynchronous copies (TMA), warp-specialised -- the float counterpart of the staged packed-bit eval kernel.
//
// Why: the register-staged forward kernel holds its loads in registers (two float4 per row and lane, four rows per
// thread); at batch sizes in the hundreds and thousands that caps the bytes in flight per SM well below what HBM3e
// needs (measured 0.63-0.75 of the copy bandwidth on 64000 x 64000 x 1024 and 128000 x 128000 x 256).  Here two
// producer warps issue one 1-D bulk copy per gathered 2 KB row segment into a ring of two 64 KB stages -- no registers
// held -- and eight consumer warps turn finished stages into output rows: c0 + ca A + cb B + cab A B with 16-byte
// shared loads and 16-byte global stores.  A consumer warp first computes the four coefficients of its two neurons
// (softmax over the 16 gate weights, four lanes per neuron) while the stage is still landing.
//
// Tiling as in the eval kernel: a tile is 16 neurons x `chunk` bytes of their rows, tiles numbered column chunk major so
// that the persistent grid (one CTA per SM) works on one column chunk of x at a time and the second reader of an input
// row finds it in L2.  Every wait is bounded; a wait that runs out raises the flag that dl_async_error() reads.
#include <stdlib.h>

#include "common.cuh"
#include "gates.cuh"
#include "tma.cuh"

namespace dl {

constexpr int kFwRows = 16;
constexpr int kFwStages = 2;
constexpr int kFwProducers = 2;
constexpr int kFwConsumerWarps = 8;
constexpr int kFwThreads = 32 * (kFwProducers + kFwConsumerWarps);
constexpr int kFwMaxChunk = 2048;  // bytes of a row per tile: 512 floats

__device__ int g_fw_async_error = 0;

__device__ __forceinline__ bool fw_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

__global__ void __launch_bounds__(kFwThreads, 1)
forward_tma_kernel(const float *__restrict__ x, const int64_t *__restrict__ a, const int64_t *__restrict__ b,
                   const float *__restrict__ w, int w_mode, float *__restrict__ y, float4 *__restrict__ coef_out, uint32_t n_out,
                   int64_t row_bytes, int chunk, uint32_t row_blocks, uint32_t ntiles) {
    extern __shared__ __align__(128) uint8_t smem[];
    const size_t stage_bytes = (size_t)2 * kFwRows * chunk;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kFwStages * stage_bytes);
    uint64_t *empty = full + kFwStages;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    if (tid == 0) {
        for (int s = 0; s < kFwStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kFwConsumerWarps);
        }
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    volatile int *abort_flag = &s_abort;
    const uint32_t G = gridDim.x;
    const uint8_t *xb = reinterpret_cast<const uint8_t *>(x);

    if (warp < kFwProducers) {
        // ---------------- producers: lane l copies input (l / 16) of neuron (l % 16) of the tile ----------------
        const int r = lane % kFwRows, which = lane / kFwRows;
        uint32_t it = warp;
        uint32_t t = blockIdx.x + warp * G;
        uint32_t issued = 0;
        bool ok = true;
        int64_t idx = 0;
        if (t < ntiles) {  // the connection indices are fixed at construction: read them before the dependency wait
            const uint32_t j = (t % row_blocks) * kFwRows + r;
            if (j < n_out) idx = __ldg((which ? b : a) + j);
        }
        grid_dependency_wait();  // x is the output of the kernel just before
        grid_dependents_launch();
        for (; t < ntiles; t += kFwProducers * G, it += kFwProducers) {
            const int s = (int)(it % kFwStages);
            const uint32_t use = it / kFwStages;
            int64_t idx_next = 0;
            const uint32_t tn = t + kFwProducers * G;
            if (tn < ntiles) {
                const uint32_t jn = (tn % row_blocks) * kFwRows + r;
                if (jn < n_out) idx_next = __ldg((which ? b : a) + jn);
            }
            if (!fw_wait(empty + s, (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t cb = t / row_blocks, nb = t % row_blocks;
            const int64_t col0 = (int64_t)cb * chunk;
            const uint32_t bytes = (uint32_t)min((int64_t)chunk, row_bytes - col0);
            const bool valid = nb * kFwRows + r < n_out;
            const uint32_t nvalid = min((uint32_t)kFwRows, n_out - nb * kFwRows);
            if (lane == 0) mbar_arrive_expect_tx(full + s, 2u * nvalid * bytes);
            __syncwarp();
            if (valid)
                bulk_load(smem + s * stage_bytes + (size_t)(which * kFwRows + r) * chunk, xb + idx * row_bytes + col0, bytes, full + s);
            ++issued;
            idx = idx_next;
        }
        if (!ok || *abort_flag) {
            if (lane == 0) {
                g_fw_async_error = 1;
                s_abort = 1;
            }
            __syncwarp();
            if (issued > 0) {
                const uint32_t last = it - kFwProducers;
                mbar_wait(full + (last % kFwStages), (last / kFwStages) & 1u);
            }
        }
    } else {
        // ---------------- consumers: warp cw turns rows cw and cw + 8 of every finished stage into output rows ----------
        const int cw = warp - kFwProducers;
        const int q = lane & 3;           // four lanes share a neuron's 16 weights
        const int mine = lane >> 2;       // 0: row cw, 1: row cw + 8, others: no neuron
        grid_dependency_wait();           // the weights may have been updated by the kernels just before
        uint32_t it = 0;
        for (uint32_t t = blockIdx.x; t < ntiles; t += G, ++it) {
            const int s = (int)(it % kFwStages);
            const uint32_t use = it / kFwStages;
            const uint32_t cb = t / row_blocks, nb = t % row_blocks;
            // coefficients of this warp's two neurons, while the stage is landing
            const uint32_t jq = nb * kFwRows + cw + 8 * mine;
            const bool live = mine < 2 && jq < n_out;
            const float4 cq = quad_coef(w + (int64_t)(live ? jq : 0) * 16 + q * 4, live, q, w_mode);
            if (live && q == 0 && cb == 0 && coef_out != nullptr) coef_out[jq] = cq;
            if (!fw_wait(full + s, use & 1u, abort_flag)) {
                if (lane == 0) {
                    g_fw_async_error = 1;
                    s_abort = 1;
                }
                break;
            }
            const int64_t col0 = (int64_t)cb * chunk;
            const int vecs = (int)(min((int64_t)chunk, row_bytes - col0) / 16);
            const int nvalid = (int)min((uint32_t)kFwRows, n_out - nb * kFwRows);
            const float4 *sa = reinterpret_cast<const float4 *>(smem + s * stage_bytes);
            const float4 *sb = reinterpret_cast<const float4 *>(smem + s * stage_bytes + (size_t)kFwRows * chunk);
            const int pitch = chunk / 16;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = cw + 8 * half;
                float4 c;
                c.x = __shfl_sync(0xffffffffu, cq.x, 4 * half);
                c.y = __shfl_sync(0xffffffffu, cq.y, 4 * half);
                c.z = __shfl_sync(0xffffffffu, cq.z, 4 * half);
                c.w = __shfl_sync(0xffffffffu, cq.w, 4 * half);
                if (r < nvalid) {
                    float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(y) + ((int64_t)nb * kFwRows + r) * row_bytes + col0);
#pragma unroll 4
                    for (int v = lane; v < vecs; v += 32) dst[v] = mixv(c, sa[r * pitch + v], sb[r * pitch + v]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);
        }
    }
}

int forward_tma_async_error() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, g_fw_async_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return flag;
}

// True when the staged kernel applies and pays: rows of whole float4s and at least 1 KB (batch >= 256), 16-byte aligned
// buffers.  Opt-in: DL_TUNE_FORWARD_KERNEL = 2 (staged) selects it from 512-byte rows on (for A/B timing).
bool forward_tma_applicable(const float *x, const float *y, int64_t n_out, int64_t batch) {
    if (tuning(DL_TUNE_FORWARD_KERNEL) != 2) return false;  // opt-in for now
    const int64_t row_bytes = batch * 4;
    const int64_t least = 512;
    if (!(batch % 4 == 0 && row_bytes >= least && n_out >= kFwRows && aligned_to(x, 16) && aligned_to(y, 16))) return false;
    const int64_t chunk = row_bytes < kFwMaxChunk ? row_bytes : kFwMaxChunk;
    return n_out < ((int64_t)1 << 31) && ceil_div(row_bytes, chunk) * ceil_div(n_out, kFwRows) < ((int64_t)1 << 31) - 4096;
}

int launch_forward_tma(bool overlap, const float *x, const int64_t *a, const int64_t *b, const float *w, int w_mode, float *y,
                       float *coef, int64_t n_out, int64_t batch, cudaStream_t st) {
    const int64_t row_bytes = batch * 4;
    const int chunk = (int)(row_bytes < kFwMaxChunk ? row_bytes : kFwMaxChunk);
    const int64_t row_blocks = ceil_div(n_out, kFwRows);
    const int64_t ntiles = ceil_div(row_bytes, chunk) * row_blocks;
    const size_t smem = (size_t)kFwStages * 2 * kFwRows * chunk + 2 * kFwStages * sizeof(uint64_t);
    if (cudaFuncSetAttribute(forward_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return launch_status("dl_forward_f32 (shared memory opt-in)");
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const unsigned grid = (unsigned)(ntiles < sms ? ntiles : sms);
    launch_dependent(overlap, forward_tma_kernel, dim3(grid), dim3(kFwThreads), smem, st, x, a, b, w, w_mode, y,
                     reinterpret_cast<float4 *>(coef), (uint32_t)n_out, row_bytes, chunk, (uint32_t)row_blocks, (uint32_t)ntiles);
    return launch_status("dl_forward_f32");
}

}  // namespace dl
