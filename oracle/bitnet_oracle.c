/*
 * CPU oracle of the packed-bit path, in C.  TEST INFRASTRUCTURE ONLY: a checker for the CUDA
 * kernels and the timed CPU baseline of the benchmark; nothing in the shipped package links it.
 *
 * It restates what the reference's CompiledLogicNet C code does for one block of 64 samples
 * (difflogic/compiled_model.py:159-239): pack 64 boolean samples into one int64 per feature,
 * LSB = first sample (:191-198); apply every gate of every layer bitwise (:94-137, one of the 16
 * operators per gate); count per class with a bit-sliced ripple counter (:204-219); unpack to
 * int32 [sample][class] (:222-230).  The reference emits one C statement per gate and compiles
 * it; this file walks the same gates from tables, so that it can travel without a compiler run.
 * Parity is pinned in tests/test_oracle_golden.py against class counts produced by the
 * reference's own compiled code (tests/golden/).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline uint64_t gate64(uint64_t a, uint64_t b, int op) {
    switch (op) {
    case 0: return 0;
    case 1: return a & b;
    case 2: return a & ~b;
    case 3: return a;
    case 4: return b & ~a;
    case 5: return b;
    case 6: return a ^ b;
    case 7: return a | b;
    case 8: return ~(a | b);
    case 9: return ~(a ^ b);
    case 10: return ~b;
    case 11: return ~b | a;
    case 12: return ~a;
    case 13: return ~a | b;
    case 14: return ~(a & b);
    default: return ~(uint64_t)0;
    }
}

/* One layer on packed rows: y[j][w] = gate_j(x[a_j][w], x[b_j][w])  (difflogic_kernel.cu:474-501). */
void oracle_eval_layer(const uint64_t *x, const int64_t *a, const int64_t *b, const uint8_t *op, uint64_t *y,
                       int64_t n_out, int64_t words) {
    for (int64_t j = 0; j < n_out; ++j)
        for (int64_t w = 0; w < words; ++w)
            y[j * words + w] = gate64(x[a[j] * words + w], x[b[j] * words + w], op[j]);
}

/*
 * Whole net on boolean samples, 64 at a time, as CompiledLogicNet.forward does.
 *   inp    bool  [n_blocks*64][n_in]   (sample-major; the caller pads the batch to a multiple of 64)
 *   out    int32 [n_blocks*64][k]
 *   a,b,op concatenated over the layers; widths[l] = gates of layer l
 * Blocks are independent; they are spread over `threads` OpenMP threads (1 = the reference's
 * single-threaded behaviour).
 */
void oracle_apply_net(const uint8_t *inp, int32_t *out, int64_t n_blocks, int64_t n_in, int n_layers, const int64_t *widths,
                      const int64_t *a, const int64_t *b, const uint8_t *op, int64_t k, int threads) {
    int64_t max_w = n_in;
    for (int l = 0; l < n_layers; ++l)
        if (widths[l] > max_w) max_w = widths[l];
    const int64_t n_last = widths[n_layers - 1];
    const int64_t per_class = n_last / k;
    int planes = 0;
    while (((int64_t)1 << planes) <= per_class) ++planes;

#pragma omp parallel num_threads(threads)
    {
        uint64_t *cur = malloc(sizeof(uint64_t) * max_w);
        uint64_t *nxt = malloc(sizeof(uint64_t) * max_w);
        uint64_t count[64];
#pragma omp for schedule(static)
        for (int64_t blk = 0; blk < n_blocks; ++blk) {
            const uint8_t *src = inp + blk * 64 * n_in;
            for (int64_t d = 0; d < n_in; ++d) {
                uint64_t w = 0;
                for (int s = 0; s < 64; ++s) w |= (uint64_t)(src[(int64_t)s * n_in + d] != 0) << s;
                cur[d] = w;
            }
            int64_t off = 0;
            for (int l = 0; l < n_layers; ++l) {
                const int64_t n = widths[l];
                for (int64_t j = 0; j < n; ++j) nxt[j] = gate64(cur[a[off + j]], cur[b[off + j]], op[off + j]);
                off += n;
                uint64_t *t = cur; cur = nxt; nxt = t;
            }
            for (int64_t c = 0; c < k; ++c) {
                memset(count, 0, sizeof(count));
                for (int64_t g = 0; g < per_class; ++g) {
                    uint64_t carry = cur[c * per_class + g];
                    for (int p = 0; p < planes && carry; ++p) {
                        const uint64_t t = count[p] & carry;
                        count[p] ^= carry;
                        carry = t;
                    }
                }
                for (int s = 0; s < 64; ++s) {
                    int32_t v = 0;
                    for (int p = 0; p < planes; ++p) v |= (int32_t)((count[p] >> s) & 1) << p;
                    out[(blk * 64 + s) * k + c] = v;
                }
            }
        }
        free(cur);
        free(nxt);
    }
}
