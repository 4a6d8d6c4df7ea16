// Packed-bit eval for long rows: gathered input rows staged in shared memory by bulk asynchronous
// copies (TMA), warp-specialised.
//
// Why: the plain eval kernel keeps its loads in registers, and at 16 bytes per lane the register
// file caps the bytes in flight per SM well below what HBM3e needs (ncu: 91 registers, 2 CTAs per SM,
// 42 % of DRAM peak).  Here two producer warps issue one 1-D bulk copy per gathered row segment --
// no registers held, 64 KB per stage -- and eight consumer warps turn finished stages into output
// rows with 16-byte shared loads, LOP3s and 16-byte global stores.  One producer warp alone was the
// bottleneck (about 1 us of issue work per tile); two alternate over the tiles.
//
// Tiling: a tile is kTileRows neurons x `chunk` bytes of their rows.  Tiles are numbered column
// chunk major, so the CTAs of the persistent grid (one per SM) work on the same column chunk of x at
// the same time and the second reader of an input row finds it in L2; DRAM reads stay at one pass
// over x.
#include <stdlib.h>

#include "common.cuh"
#include "gates.cuh"
#include "tma.cuh"

namespace dl {

// Two shapes of the same kernel (template parameters kTileRows x kStages):
//   16 x 2, one CTA per SM  -- square layers: every input row is read about twice, HBM reads dominate;
//    8 x 3, two CTAs per SM -- layers at least twice as wide as their input (e.g. 784 -> 8000): the input rows are
//                              read many times out of L2 and the output writes dominate; four producer warps
//                              per SM and smaller tiles keep more independent copies in flight (measured on
//                              2^20 samples: 784 -> 8000 221 us against 288 us, 4000 -> 8000 254 against 327,
//                              but 6000 -> 8000 391 against 346).  Also used when the 16 x 2 shape would give a
//                              CTA fewer than 64 tiles (8000 -> 8000 on 2^17 samples: 48 us against 53 us).
constexpr int kProducers = 2;       // producer warps; tile i is issued by warp i % kProducers
constexpr int kConsumerWarps = 8;
constexpr int kTmaThreads = 32 * (kProducers + kConsumerWarps);
constexpr int kMaxChunk = 2048;     // bytes of a row per tile

__device__ int g_async_error = 0;   // set when a bounded wait ran out; read by dl_async_error()

__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

template <int kTileRows, int kStages>
__global__ void __launch_bounds__(kTmaThreads)
eval_tma_kernel(const uint8_t *__restrict__ x, const int64_t *__restrict__ a, const int64_t *__restrict__ b,
                const uint8_t *__restrict__ gate, uint8_t *__restrict__ y, uint32_t n_out, int64_t row_bytes, int chunk,
                uint32_t row_blocks, uint32_t ntiles, int64_t x_pitch, int64_t y_pitch) {
    extern __shared__ __align__(128) uint8_t smem[];
    const size_t stage_bytes = (size_t)2 * kTileRows * chunk;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kStages * stage_bytes);
    uint64_t *empty = full + kStages;
    uint8_t *meta = reinterpret_cast<uint8_t *>(empty + kStages);  // [kStages][kTileRows] gate ids
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kConsumerWarps);
        }
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    volatile int *abort_flag = &s_abort;
    const uint32_t G = gridDim.x;

    if (warp < kProducers) {
        // ---------------- producers: one bulk copy per (neuron, input) of the tile ----------------
        // Lane l owns input (l / kTileRows) of neuron (l % kTileRows).  The connection indices of this warp's
        // NEXT tile are fetched while the current stage is still being waited for.
        const int r = lane % kTileRows, which = (lane / kTileRows) & 1;
        const bool copier = lane < 2 * kTileRows;
        uint32_t it = warp;
        uint32_t t = blockIdx.x + warp * G;
        uint32_t issued = 0;
        bool ok = true;
        int64_t idx = 0;
        uint32_t op = 0;
        if (copier && t < ntiles) {
            const uint32_t j = (t % row_blocks) * kTileRows + r;
            if (j < n_out) {
                idx = __ldg((which ? b : a) + j);
                op = __ldg(gate + j);
            }
        }
        for (; t < ntiles; t += kProducers * G, it += kProducers) {
            const int s = (int)(it % kStages);
            const uint32_t use = it / kStages;
            int64_t idx_next = 0;
            uint32_t op_next = 0;
            const uint32_t tn = t + kProducers * G;
            if (copier && tn < ntiles) {
                const uint32_t jn = (tn % row_blocks) * kTileRows + r;
                if (jn < n_out) {
                    idx_next = __ldg((which ? b : a) + jn);
                    op_next = __ldg(gate + jn);
                }
            }
            if (!wait_or_abort(empty + s, (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t cb = t / row_blocks, nb = t % row_blocks;
            const int64_t col0 = (int64_t)cb * chunk;
            const uint32_t bytes = (uint32_t)min((int64_t)chunk, row_bytes - col0);
            const bool valid = copier && nb * kTileRows + r < n_out;
            if (valid && which == 0) meta[s * kTileRows + r] = (uint8_t)op;
            // an input that the neuron's gate ignores is not fetched: its mask is zero, whatever the stage holds there
            const bool needed = valid && gate_needs_input(op, which);
            const uint32_t copies = (uint32_t)__popc(__ballot_sync(0xffffffffu, needed));
            __syncwarp();  // the masks / gate ids written above are ordered before lane 0's arrival
            if (lane == 0) mbar_arrive_expect_tx(full + s, copies * bytes);
            __syncwarp();
            if (needed)
                bulk_load(smem + s * stage_bytes + (size_t)(which * kTileRows + r) * chunk, x + idx * x_pitch + col0, bytes,
                          full + s);
            ++issued;
            idx = idx_next;
            op = op_next;
        }
        if (!ok || *abort_flag) {
            // something went wrong: flag it, stop everybody, and give this warp's last copies time to land
            if (lane == 0) {
                g_async_error = 1;
                s_abort = 1;
            }
            __syncwarp();
            if (issued > 0) {
                const uint32_t last = it - kProducers;  // iteration of this warp's latest fill
                mbar_wait(full + (last % kStages), (last / kStages) & 1u);
            }
        }
    } else {
        // ---------------- consumers: finished stages -> output rows ------------------------------
        const int cw = warp - kProducers;
        uint32_t it = 0;
        for (uint32_t t = blockIdx.x; t < ntiles; t += G, ++it) {
            const int s = (int)(it % kStages);
            const uint32_t use = it / kStages;
            if (!wait_or_abort(full + s, use & 1u, abort_flag)) {
                if (lane == 0) {
                    g_async_error = 1;
                    s_abort = 1;
                }
                break;
            }
            const uint32_t cb = t / row_blocks, nb = t % row_blocks;
            const int64_t col0 = (int64_t)cb * chunk;
            const int vecs = (int)(min((int64_t)chunk, row_bytes - col0) / 16);
            const int nvalid = (int)min((uint32_t)kTileRows, n_out - nb * kTileRows);
            const uint4 *sa = reinterpret_cast<const uint4 *>(smem + s * stage_bytes);
            const uint4 *sb = reinterpret_cast<const uint4 *>(smem + s * stage_bytes + (size_t)kTileRows * chunk);
            const int pitch = chunk / 16;
            for (int r = cw; r < nvalid; r += kConsumerWarps) {
                const GateMasks gm = gate_masks(meta[s * kTileRows + r]);
                uint4 *dst = reinterpret_cast<uint4 *>(y + ((int64_t)nb * kTileRows + r) * y_pitch + col0);
#pragma unroll 4
                for (int c = lane; c < vecs; c += 32) {
                    const uint4 va = sa[r * pitch + c], vb = sb[r * pitch + c];
                    dst[c] = make_uint4(gate32(va.x, vb.x, gm), gate32(va.y, vb.y, gm), gate32(va.z, vb.z, gm),
                                        gate32(va.w, vb.w, gm));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);
        }
    }
}

int groupbitsum_async_error();       // groupbitsum_tma.cu
int eval_groupbitsum_async_error();  // eval_groupbitsum.cu
int forward_tma_async_error();       // forward_tma.cu

static int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

constexpr int kMinTileRows = 8;

// True when the staged kernel applies: 16-byte aligned rows of at least 512 bytes, tile count within 32 bits.
bool eval_tma_applicable(const void *x, const void *y, int64_t row_bytes, int64_t n_out) {
    if (!(row_bytes % 16 == 0 && row_bytes >= 512 && n_out >= 16 && aligned_to(x, 16) && aligned_to(y, 16))) return false;
    const int64_t chunk = row_bytes < kMaxChunk ? row_bytes : kMaxChunk;
    return n_out < ((int64_t)1 << 31) && ceil_div(row_bytes, chunk) * ceil_div(n_out, kMinTileRows) < ((int64_t)1 << 31) - 4096;
}

template <int ROWS, int STAGES>
static int launch_eval_tma_shape(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, void *y, int64_t n_out,
                                 int64_t row_bytes, int ctas_per_sm, cudaStream_t st, int64_t x_pitch, int64_t y_pitch) {
    const int chunk = (int)(row_bytes < kMaxChunk ? row_bytes : kMaxChunk);
    const int64_t col_chunks = ceil_div(row_bytes, chunk);
    const int64_t row_blocks = ceil_div(n_out, ROWS);
    const int64_t ntiles = col_chunks * row_blocks;
    const size_t smem = (size_t)STAGES * 2 * ROWS * chunk + 2 * STAGES * sizeof(uint64_t) + STAGES * ROWS;
    if (cudaFuncSetAttribute(eval_tma_kernel<ROWS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return launch_status("dl_eval_packed (shared memory opt-in)");
    const int64_t slots = (int64_t)sm_count() * ctas_per_sm;
    const unsigned grid = (unsigned)(ntiles < slots ? ntiles : slots);
    eval_tma_kernel<ROWS, STAGES><<<grid, kTmaThreads, smem, st>>>(reinterpret_cast<const uint8_t *>(x), a, b, gate,
                                                                  reinterpret_cast<uint8_t *>(y), (uint32_t)n_out, row_bytes, chunk,
                                                                  (uint32_t)row_blocks, (uint32_t)ntiles, x_pitch, y_pitch);
    return launch_status("dl_eval_packed");
}

// x_pitch / y_pitch: bytes from one row of x / y to the next (row_bytes for contiguous matrices; larger when the rows
// are a column slice of wider rows).  Multiples of 16.
int launch_eval_tma(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, void *y, int64_t n_in, int64_t n_out,
                    int64_t row_bytes, cudaStream_t st, int64_t x_pitch, int64_t y_pitch) {
    // fan-out of an input row: 2 * n_out / n_in.  DL_TUNE_EVAL_SHAPE = 1 (wide) | 2 (square) overrides the choice.
    const int force = tuning(DL_TUNE_EVAL_SHAPE);
    const int64_t chunk = row_bytes < kMaxChunk ? row_bytes : kMaxChunk;
    const bool few_tiles = ceil_div(row_bytes, chunk) * ceil_div(n_out, 16) < (int64_t)64 * sm_count();
    const bool wide = force == 1 ? true : force == 2 ? false : (n_out >= 2 * n_in || few_tiles);
    if (wide) return launch_eval_tma_shape<8, 3>(x, a, b, gate, y, n_out, row_bytes, 2, st, x_pitch, y_pitch);
    return launch_eval_tma_shape<16, 2>(x, a, b, gate, y, n_out, row_bytes, 1, st, x_pitch, y_pitch);
}

}  // namespace dl

// Self-test of the bounded mbarrier wait that every staged kernel relies on: one thread waits, with mbar_wait() and a
// poll limit given by the caller, for a barrier phase that nobody completes -- the wait must run out and the kernel must
// return -- and then for a phase that its own arrival completes.  result[0]: 1 = the first wait ran out as it should,
// 2 = it reported completion; result[1]: 1 = the second wait succeeded.  Touches none of the library's state.
__global__ void bounded_wait_selftest_kernel(int *result, uint32_t polls) {
    __shared__ uint64_t bar[2];
    if (threadIdx.x == 0) {
        dl::mbar_init(bar, 1);
        dl::mbar_init(bar + 1, 1);
        dl::mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        result[0] = dl::mbar_wait(bar, 0, polls) ? 2 : 1;
        dl::mbar_arrive(bar + 1);
        result[1] = dl::mbar_wait(bar + 1, 0, polls) ? 1 : 0;
    }
}

extern "C" DL_API int dl_selftest_bounded_wait(int32_t *result, uint32_t polls, void *stream) {
    DL_REQUIRE(result != nullptr && polls > 0 && polls <= dl::kSpinLimit, DL_ERR_INVALID_ARG, "dl_selftest_bounded_wait: bad argument");
    bounded_wait_selftest_kernel<<<1, 32, 0, dl::as_stream(stream)>>>(reinterpret_cast<int *>(result), polls);
    return dl::launch_status("dl_selftest_bounded_wait");
}

// 1 if a bounded wait inside a kernel of this library ever ran out on the current device (the affected
// launch produced incomplete output), else 0; negative on a CUDA error.  Synchronises the device.
extern "C" DL_API int dl_async_error(void) {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, dl::g_async_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    const int other = dl::groupbitsum_async_error();
    if (other < 0) return other;
    const int fused = dl::eval_groupbitsum_async_error();
    if (fused < 0) return fused;
    const int fwd = dl::forward_tma_async_error();
    if (fwd < 0) return fwd;
    return flag | other | fused | fwd;
}
