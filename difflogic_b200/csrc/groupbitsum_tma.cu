// Group bit-sum for long rows, rows staged in shared memory by bulk asynchronous copies (TMA).
//
// A work unit is (column block of kColBytes bytes, class, row split).  One producer warp streams the
// unit's rows, 32 at a time (one bulk copy per lane), into a ring of shared-memory stages; 128
// consumer threads own one 64-bit word column each and feed the rows of every finished stage to a
// bit-sliced counter that lives in registers for the whole unit.  At the end of the unit the planes
// are spread to 64 integers per thread and stored to out[sample][class] (added atomically when a
// class's rows were split over several units).  The copy engine keeps ~100 KB in flight per SM
// without using registers, and the expansion of one unit overlaps the loads of the next.
#include "bitcount.cuh"
#include "common.cuh"
#include "tma.cuh"

namespace dl {

constexpr int kGbRows = 32;         // rows per stage: one copy per producer lane
constexpr int kGbColBytes = 1024;   // column block: 128 words of 64 bits
constexpr int kGbStages = 3;        // 3 x 32 KB per CTA; two CTAs share an SM, so two producer warps issue copies per SM
constexpr int kGbConsumers = 128;
constexpr int kGbThreads = 32 + kGbConsumers;

__device__ int g_gb_async_error = 0;  // set when a bounded wait ran out; read by groupbitsum_async_error()

__device__ __forceinline__ bool gb_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

struct GbUnit {
    int64_t col0;   // first byte of the column block within a row
    int64_t row0;   // first row
    int rows;       // number of rows
    int cls;
    uint32_t bytes; // bytes per row segment
};

__device__ __forceinline__ GbUnit gb_unit(int64_t u, int64_t row_bytes, int k, int m, int splits) {
    GbUnit g;
    const int q = (int)(u % splits);
    const int64_t rest = u / splits;
    g.cls = (int)(rest % k);
    const int64_t cb = rest / k;
    g.col0 = cb * kGbColBytes;
    g.bytes = (uint32_t)min((int64_t)kGbColBytes, row_bytes - g.col0);
    const int64_t r0 = ((int64_t)m * q) / splits, r1 = ((int64_t)m * (q + 1)) / splits;
    g.row0 = (int64_t)g.cls * m + r0;
    g.rows = (int)(r1 - r0);
    return g;
}

__global__ void __launch_bounds__(kGbThreads, 2)
groupbitsum_tma_kernel(const uint8_t *__restrict__ x, int32_t *__restrict__ out, int64_t row_bytes, int64_t batch, int k, int m,
                       int splits, int nplanes, int64_t nunits) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr size_t stage_bytes = (size_t)kGbRows * kGbColBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kGbStages * stage_bytes);
    uint64_t *empty = full + kGbStages;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    if (tid == 0) {
        for (int s = 0; s < kGbStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, kGbConsumers / 32);
        }
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    volatile int *abort_flag = &s_abort;

    if (warp == 0) {
        // ---------------- producer ----------------
        int64_t it = 0;
        bool ok = true;
        for (int64_t u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
            const GbUnit g = gb_unit(u, row_bytes, k, m, splits);
            for (int r = 0; r < g.rows; r += kGbRows, ++it) {
                const int s = (int)(it % kGbStages);
                const uint32_t use = (uint32_t)(it / kGbStages);
                if (!gb_wait(empty + s, (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                const int nr = min(kGbRows, g.rows - r);
                if (lane == 0) mbar_arrive_expect_tx(full + s, (uint32_t)nr * g.bytes);
                __syncwarp();
                if (lane < nr)
                    bulk_load(smem + s * stage_bytes + (size_t)lane * kGbColBytes, x + (g.row0 + r + lane) * row_bytes + g.col0,
                              g.bytes, full + s);
            }
        }
        if (!ok || *abort_flag) {
            if (lane == 0) {
                g_gb_async_error = 1;
                s_abort = 1;
            }
            __syncwarp();
            for (int s = 0; s < kGbStages; ++s) {
                const int64_t fills = (it + kGbStages - 1 - s) / kGbStages;
                if (fills > 0) mbar_wait(full + s, (uint32_t)(fills - 1) & 1u);
            }
        }
    } else {
        // ---------------- consumers: one 64-bit word column per thread ----------------
        const int ct = tid - 32;
        int64_t it = 0;
        bool ok = true;
        for (int64_t u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
            const GbUnit g = gb_unit(u, row_bytes, k, m, splits);
            const bool mine = (uint32_t)ct * 8u < g.bytes;
            BitCounter cn;
            cn.clear();
            for (int r = 0; r < g.rows; r += kGbRows, ++it) {
                const int s = (int)(it % kGbStages);
                const uint32_t use = (uint32_t)(it / kGbStages);
                if (!gb_wait(full + s, use & 1u, abort_flag)) {
                    if (lane == 0) {
                        g_gb_async_error = 1;
                        s_abort = 1;
                    }
                    ok = false;
                    break;
                }
                const int nr = min(kGbRows, g.rows - r);
                if (mine) {
                    const unsigned long long *col = reinterpret_cast<const unsigned long long *>(smem + s * stage_bytes) + ct;
                    int rr = 0;
                    for (; rr + 8 <= nr; rr += 8) {
                        unsigned long long v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = col[(size_t)(rr + i) * (kGbColBytes / 8)];
                        cn.add8(v);
                    }
                    for (; rr < nr; ++rr) cn.add1(col[(size_t)rr * (kGbColBytes / 8)]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + s);
            }
            if (!ok) break;
            if (mine) {
                // planes -> integers, four samples at a time (16-bit fields: sample s + 16 f)
                const int64_t s0 = (g.col0 + (int64_t)ct * 8) * 8;  // first sample of this word
                int32_t *dst = out + s0 * k + g.cls;
#pragma unroll 2
                for (int sft = 0; sft < 16; ++sft) {
                    unsigned long long acc = 0ull;
#pragma unroll
                    for (int pl = 0; pl < kPlanes; ++pl)
                        if (pl < nplanes) acc |= ((cn.plane(pl) >> sft) & 0x0001000100010001ull) << pl;
#pragma unroll
                    for (int f = 0; f < 4; ++f) {
                        const int smp = sft + 16 * f;
                        const int cnt = (int)((acc >> (16 * f)) & 0xFFFFull);
                        if (s0 + smp < batch) {
                            if (splits == 1)
                                dst[(int64_t)smp * k] = cnt;
                            else if (cnt)
                                atomicAdd(dst + (int64_t)smp * k, cnt);
                        }
                    }
                }
            }
        }
    }
}

static int gb_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    return n;
}

int groupbitsum_async_error() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, g_gb_async_error, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return flag;
}

bool groupbitsum_tma_applicable(const void *x, int64_t n, int64_t row_bytes, int64_t k) {
    return n > 0 && row_bytes % 16 == 0 && row_bytes >= 256 && aligned_to(x, 16) && n / k >= 8;
}

int launch_groupbitsum_tma(const void *x, int32_t *out, int64_t n, int64_t row_bytes, int64_t batch, int64_t k, cudaStream_t st) {
    const int64_t m = n / k;
    const int64_t colblocks = ceil_div(row_bytes, kGbColBytes);
    const int64_t sms = gb_sm_count();
    // split a class's rows when columns x classes alone cannot occupy every SM a few times over
    int64_t splits = ceil_div(8 * sms, colblocks * k);
    if (splits > m / 64) splits = m / 64;
    if (splits < 1) splits = 1;
    while (ceil_div(m, splits) > kMaxChunkRows) ++splits;
    int nplanes = 1;
    while (nplanes < kPlanes && ((int64_t)1 << nplanes) <= ceil_div(m, splits)) ++nplanes;
    const int64_t nunits = colblocks * k * splits;
    if (splits > 1 && cudaMemsetAsync(out, 0, (size_t)batch * k * sizeof(int32_t), st) != cudaSuccess)
        return launch_status("dl_groupbitsum (clearing the output)");
    const size_t smem = (size_t)kGbStages * kGbRows * kGbColBytes + 2 * kGbStages * sizeof(uint64_t);
    if (cudaFuncSetAttribute(groupbitsum_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return launch_status("dl_groupbitsum (shared memory opt-in)");
    const unsigned grid = (unsigned)(nunits < 2 * sms ? nunits : 2 * sms);
    groupbitsum_tma_kernel<<<grid, kGbThreads, smem, st>>>(reinterpret_cast<const uint8_t *>(x), out, row_bytes, batch, (int)k,
                                                          (int)m, (int)splits, nplanes, nunits);
    return launch_status("dl_groupbitsum");
}

}  // namespace dl
