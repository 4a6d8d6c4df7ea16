// Version, error reporting and the two per-neuron helper kernels (coefficients, arg-max gate).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "gates.cuh"

namespace dl {

static thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

// Kernel-choice switches for A/B measurements (dl_set_tuning).  They are plain ints read on the hot entry points; their
// initial values are taken from the environment ONCE, when the library is loaded.
static int g_tuning[DL_TUNE_COUNT];

static int env_choice(const char *name, const char *letters, const int *values, int n) {
    const char *v = getenv(name);
    if (v == nullptr) return 0;
    for (int i = 0; i < n; ++i)
        if (v[0] == letters[i]) return values[i];
    return 0;
}

static const bool g_tuning_loaded = [] {
    const int pdl[] = {1}, ek[] = {1}, es[] = {1, 2}, gb[] = {1, 2}, gs[] = {1}, fc[] = {2, 4, 8}, fk[] = {1, 2};
    g_tuning[DL_TUNE_NO_PDL] = env_choice("DL_PDL", "0", pdl, 1);
    g_tuning[DL_TUNE_EVAL_KERNEL] = env_choice("DL_EVAL_KERNEL", "p", ek, 1);
    g_tuning[DL_TUNE_EVAL_SHAPE] = env_choice("DL_EVAL_SHAPE", "ws", es, 2);
    g_tuning[DL_TUNE_GROUPBITSUM_KERNEL] = env_choice("DL_GROUPBITSUM_KERNEL", "ps", gb, 2);
    g_tuning[DL_TUNE_GROUPSUM_KERNEL] = env_choice("DL_GROUPSUM_KERNEL", "t", gs, 1);
    g_tuning[DL_TUNE_FUSED_CLUSTER] = env_choice("DL_FUSED_CLUSTER", "248", fc, 3);
    g_tuning[DL_TUNE_FORWARD_KERNEL] = env_choice("DL_FORWARD_KERNEL", "ps", fk, 2);
    return true;
}();

int tuning(int key) { return __atomic_load_n(&g_tuning[key], __ATOMIC_RELAXED); }

bool pdl_enabled() { return tuning(DL_TUNE_NO_PDL) == 0; }

int launch_status(const char *what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();  // clear the sticky launch error so that later calls are not blamed
        return fail(DL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
    return DL_OK;
}

__global__ void __launch_bounds__(kThreads) coefs_kernel(const float *__restrict__ w, int w_mode,
                                                         float4 *__restrict__ coef, int64_t n_out) {
    // four lanes per neuron, the same arithmetic (and rounding) as inside the forward kernel
    const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const int64_t j = t >> 2;
    const int q = (int)(t & 3);
    const float4 c = quad_coef(w + j * 16 + q * 4, j < n_out, q, w_mode);
    if (q == 0 && j < n_out) coef[j] = c;
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const float *__restrict__ w, uint8_t *__restrict__ gate,
                                                          int64_t n_out) {
    const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (j < n_out) gate[j] = (uint8_t)first_argmax16(w + j * 16);
}

}  // namespace dl

extern "C" DL_API int dl_version(void) { return 100; }

extern "C" DL_API const char *dl_last_error_string(void) { return dl::g_error; }

extern "C" DL_API int dl_set_tuning(int key, int value) {
    DL_REQUIRE(key >= 0 && key < DL_TUNE_COUNT, DL_ERR_INVALID_ARG, "dl_set_tuning: unknown key %d", key);
    (void)dl::g_tuning_loaded;
    __atomic_store_n(&dl::g_tuning[key], value, __ATOMIC_RELAXED);
    return DL_OK;
}

extern "C" DL_API int dl_get_tuning(int key) { return key >= 0 && key < DL_TUNE_COUNT ? dl::tuning(key) : -1; }

extern "C" DL_API int dl_coefs_f32(const float *w, int w_mode, float *coef, int64_t n_out, void *stream) {
    DL_REQUIRE(w && coef, DL_ERR_INVALID_ARG, "dl_coefs_f32: null pointer");
    DL_REQUIRE(n_out >= 0, DL_ERR_INVALID_ARG, "dl_coefs_f32: negative size");
    DL_REQUIRE(w_mode >= DL_W_LOGITS && w_mode <= DL_W_ARGMAX, DL_ERR_INVALID_ARG, "dl_coefs_f32: unknown w_mode %d", w_mode);
    DL_REQUIRE(dl::aligned_to(coef, 16), DL_ERR_INVALID_ARG, "dl_coefs_f32: coef must be 16-byte aligned");
    if (n_out == 0) return DL_OK;
    dl::coefs_kernel<<<(unsigned)dl::ceil_div(4 * n_out, dl::kThreads), dl::kThreads, 0, dl::as_stream(stream)>>>(
        w, w_mode, reinterpret_cast<float4 *>(coef), n_out);
    return dl::launch_status("dl_coefs_f32");
}

extern "C" DL_API int dl_argmax_gate_u8(const float *w, uint8_t *gate, int64_t n_out, void *stream) {
    DL_REQUIRE(w && gate, DL_ERR_INVALID_ARG, "dl_argmax_gate_u8: null pointer");
    DL_REQUIRE(n_out >= 0, DL_ERR_INVALID_ARG, "dl_argmax_gate_u8: negative size");
    if (n_out == 0) return DL_OK;
    dl::argmax_kernel<<<(unsigned)dl::ceil_div(n_out, dl::kThreads), dl::kThreads, 0, dl::as_stream(stream)>>>(w, gate, n_out);
    return dl::launch_status("dl_argmax_gate_u8");
}
