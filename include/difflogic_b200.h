/*
 * difflogic_b200 -- C ABI of the logic-layer hot path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, launches asynchronously on the
 * stream it is given (a cudaStream_t passed as void*; NULL is the legacy default stream),
 * never allocates or frees device memory (the dl_comm_* set-up helpers excepted), never
 * synchronises the device and never exits the process.  The return value is a status code (DL_OK == 0).  After a non-zero status,
 * dl_last_error_string() gives a message for the calling thread.
 *
 * Layouts.  Float activations are feature-major: x[n_in][batch], y[n_out][batch], batch is
 * the fastest dimension.  Packed activations are feature-major rows of words along the batch:
 * t[n][words], word = bit_count bits (8, 16, 32 or 64), sample s is bit (s % bit_count) of
 * word (s / bit_count), least-significant bit first.  Connection indices a[], b[] are int64,
 * as the Python API stores them.
 *
 * Each declaration names the interface of the reference implementation
 * (Felix-Petersen/difflogic) that it replaces, as file:line within that project.
 */
#ifndef DIFFLOGIC_B200_H
#define DIFFLOGIC_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define DL_API __attribute__((visibility("default")))
#else
#define DL_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
enum {
    DL_OK = 0,
    DL_ERR_INVALID_ARG = 1,   /* null pointer, negative size, unknown mode  -> RuntimeError   */
    DL_ERR_BAD_BIT_COUNT = 2, /* bit_count not in {8,16,32,64}              -> ValueError     */
    DL_ERR_NOT_DIVISIBLE = 3, /* rows not divisible by the number of groups -> ValueError     */
    DL_ERR_CUDA = 4,          /* a CUDA runtime call or launch failed       -> RuntimeError   */
    DL_ERR_TOO_LARGE = 5      /* size beyond a documented limit             -> RuntimeError   */
};

/* How the [n_out][16] weight matrix handed to a training kernel is to be read. */
enum {
    DL_W_LOGITS = 0, /* raw parameters; the kernel applies softmax over the 16 gates          */
    DL_W_PROBS = 1,  /* mixing weights used as they are (already soft-maxed by the caller)    */
    DL_W_ARGMAX = 2  /* raw parameters; only the arg-max gate is used (first max on ties)     */
};

/* Launch flags of the training entry points.
 * DL_LAUNCH_OVERLAP_SETUP: launch with programmatic stream serialisation, so that the kernel may
 * read its connection indices (a, b, start, plan) while the previous kernel in the stream is still
 * running.  The caller promises that those index arrays were final before the previous kernel in
 * the stream was launched (they are fixed when a layer is built).  All other operands -- x, grad_y,
 * w, coef -- are read only after the previous kernel has completed, as under a plain launch. */
enum { DL_LAUNCH_PLAIN = 0, DL_LAUNCH_OVERLAP_SETUP = 1 };

DL_API int dl_version(void);
DL_API const char *dl_last_error_string(void);

/* Kernel-choice switches for A/B measurements; 0 = the library chooses (the default).  Process-wide.  Their initial
 * values come from the environment once, when the library is loaded (DL_PDL=0, DL_EVAL_KERNEL=plain,
 * DL_EVAL_SHAPE=wide|square, DL_GROUPBITSUM_KERNEL=plain|staged, DL_GROUPSUM_KERNEL=ticket, DL_FUSED_CLUSTER=2|4|8,
 * DL_FORWARD_KERNEL=plain|staged); no entry point reads the environment afterwards.  No counterpart in the reference. */
enum {
    DL_TUNE_NO_PDL = 0,             /* 1: never launch with programmatic stream serialisation                    */
    DL_TUNE_EVAL_KERNEL = 1,        /* 1: dl_eval_packed always takes the register-staged kernel                 */
    DL_TUNE_EVAL_SHAPE = 2,         /* staged eval kernel: 1 = 8 neurons x 3 stages, 2 = 16 neurons x 2 stages   */
    DL_TUNE_GROUPBITSUM_KERNEL = 3, /* 1: register kernel, 2: staged kernel                                      */
    DL_TUNE_GROUPSUM_KERNEL = 4,    /* 1: dl_groupsum_f32 always takes the workspace (ticket) kernel             */
    DL_TUNE_FUSED_CLUSTER = 5,      /* dl_eval_groupbitsum: CTAs per class, 2, 4 or 8                            */
    DL_TUNE_FORWARD_KERNEL = 6,     /* dl_forward_f32: 1 = register kernel, 2 = staged (bulk-copy) kernel        */
    DL_TUNE_COUNT = 7
};
DL_API int dl_set_tuning(int key, int value);
DL_API int dl_get_tuning(int key);

/* Kernels that stage data with asynchronous copies poll their barriers a bounded number of times
 * instead of waiting forever.  Returns 1 if such a wait ever ran out on the current device (the
 * launch it happened in wrote incomplete output), 0 if not, negative on a CUDA error.  This call
 * synchronises the device; it is a diagnostic, not part of the hot path.  The reference has no
 * counterpart: its kernels never wait on anything (difflogic_kernel.cu). */
DL_API int dl_async_error(void);
/* Self-test of the bounded mbarrier wait that the staged kernels rely on: one thread waits for a barrier phase that
 * nobody completes, for at most `polls` polls (at most 2^24, the limit the kernels use); the wait must run out and the
 * kernel return.  result (two int32 on the device): [0] = 1 when the wait ran out as it should (2: it reported
 * completion), [1] = 1 when a second wait, which the thread's own arrival completes, succeeded.  Changes no state of the
 * library.  No reference counterpart. */
DL_API int dl_selftest_bounded_wait(int32_t *result, uint32_t polls, void *stream);

/* ------------------------------------------------------------------------------------------
 * Training forward.
 * Replaces logic_layer_cuda_forward, difflogic/cuda/difflogic_kernel.cu:259-297 (kernel
 * :90-135), bound as difflogic_cuda.forward at difflogic/cuda/difflogic.cpp:46-51, together
 * with the softmax / one_hot(argmax) that LogicLayer.forward_cuda applies before it
 * (difflogic/difflogic.py:123,128).
 *
 *   y[j][s] = sum_i  p[j][i] * gate_i(x[a[j]][s], x[b[j]][s])
 *
 * coef (optional, may be NULL) receives per neuron the four numbers {c0, ca, cb, cab} with
 * y = c0 + ca*A + cb*B + cab*A*B; dl_backward_x_f32 consumes it.
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_forward_f32(const float *x, const int64_t *a, const int64_t *b, const float *w, int w_mode,
                   float *y, float *coef, int64_t n_in, int64_t n_out, int64_t batch, int flags, void *stream);

/* y [cols][rows] = transpose of x [rows][cols]: a network's batch-major input -> the feature-major layout above, in
 * front of the first layer (the reference transposes with ATen, difflogic/difflogic.py:115-116).  The kernel lets a
 * DL_LAUNCH_OVERLAP_SETUP kernel launched behind it begin its set-up at once. */
DL_API int dl_transpose_f32(const float *x, float *y, int64_t rows, int64_t cols, void *stream);

/* The coefficient table alone (w [n_out][16] -> coef [n_out][4]); used when a caller hands
 * dl_backward_x_f32 weights that did not pass through dl_forward_f32.  No counterpart in the
 * reference, which re-reads 12 of the 16 weights per consumer (difflogic_kernel.cu:215-251). */
DL_API int dl_coefs_f32(const float *w, int w_mode, float *coef, int64_t n_out, void *stream);

/* ------------------------------------------------------------------------------------------
 * backward_w.
 * Replaces logic_layer_cuda_backward_w, difflogic_kernel.cu:300-364 (kernel :138-178 and the
 * ATen epilogue :337-360), bound as difflogic_cuda.backward_w at difflogic.cpp:52-56.
 *
 * w_mode == DL_W_PROBS : grad_w[j][i] = dL/dp[j][i] (the reference's result; w may be NULL).
 * w_mode == DL_W_LOGITS: w holds the raw parameters and grad_w receives dL/dw, i.e. the
 *                        softmax backward of difflogic.py:123 is applied in the same kernel.
 * grad_w is [n_out][16], fully written (column 0 of the DL_W_PROBS result is exactly zero).
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_backward_w_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y,
                      const float *w, int w_mode, float *grad_w,
                      int64_t n_in, int64_t n_out, int64_t batch, int flags, void *stream);

/* ------------------------------------------------------------------------------------------
 * backward_x.
 * Replaces logic_layer_cuda_backward_x, difflogic_kernel.cu:367-410 (kernel :181-256), bound
 * as difflogic_cuda.backward_x at difflogic.cpp:57-62, and folds in GradFactor's scaling
 * (difflogic/functional.py:130-138) through grad_scale.
 *
 *   grad_x[i][s] = grad_scale * sum over consumers j of input i of
 *                    (d y_j / d input)(partner value) * grad_y[j][s]
 *
 * plan is the inverse connection index in the form produced by dl_build_backward_plan:
 * 2*n_out entries of two int32 {2*j + slot, partner row}, grouped by input row; start
 * [n_in+1] (int64) are the group offsets (LogicLayer.given_x_indices_of_y_start,
 * difflogic/difflogic.py:66-67).  A neuron whose two inputs are the same row contributes
 * d/da + d/db (the reference kernel adds 2*d/da there; its python path gives d/da + d/db).
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_backward_x_f32(const float *x, const float *coef, const float *grad_y, const int64_t *start,
                      const int32_t *plan, float grad_scale, float *grad_x,
                      int64_t n_in, int64_t n_out, int64_t batch, int flags, void *stream);

/* Builds `plan` [2*n_out][2] int32 from the reference's inverse index: start [n_in+1] and
 * list [2*n_out] (LogicLayer.given_x_indices_of_y_start / given_x_indices_of_y,
 * difflogic/difflogic.py:56-69).  One-time set-up per layer. */
DL_API int dl_build_backward_plan(const int64_t *a, const int64_t *b, const int64_t *start, const int64_t *list,
                           int32_t *plan, int64_t n_in, int64_t n_out, void *stream);

/* Debug aid: checks a layer's index arrays on the device, once, instead of bounds checks on every access (the arrays
 * are fixed when a layer is built, and every kernel here trusts them).  Checked: a[j], b[j] in [0, n_in);
 * 0 = start[0] <= ... <= start[n_in] = 2 n_out; list entries in [0, n_out); plan entries in range and consistent with
 * a and b.  start, list, plan may be NULL.  report: four int64 on the device, zeroed by the caller:
 * {code (0 = sound), position, offending value, limit}; nothing is read through an unchecked index and nothing traps.
 * The reference checks only contiguity and device of its tensors (CHECK_INPUT, difflogic_kernel.cu:13-17); an index
 * out of range there is an out-of-bounds access.  LogicLayer runs this check at construction when DIFFLOGIC_DEBUG=1. */
DL_API int dl_check_connections(const int64_t *a, const int64_t *b, const int64_t *start, const int64_t *list,
                                const int32_t *plan, int64_t n_in, int64_t n_out, int64_t *report, void *stream);

/* ------------------------------------------------------------------------------------------
 * Packed-bit eval.
 * Replaces logic_layer_cuda_eval, difflogic_kernel.cu:503-541 (kernel :474-501, gates
 * :437-472), bound as difflogic_cuda.eval at difflogic.cpp:63-68.
 *   y[j][c] = gate_{gate[j]}(x[a[j]][c], x[b[j]][c])   bitwise, c over the words of a row.
 * Every word of y is written (no memset needed).  gate is uint8 [n_out].
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_eval_packed(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, void *y,
                   int64_t n_in, int64_t n_out, int64_t words, int bit_count, void *stream);

/* dl_eval_packed on column slices: the rows of x and y are row_bytes long but lie x_pitch / y_pitch bytes apart (a
 * column range of wider matrices; pitch == row_bytes for contiguous ones).  For running a network over a batch in
 * slices whose activations stay in the L2 cache while the packed input and the counts stay whole.  Rows of at least
 * 512 bytes; row_bytes, pitches and pointers multiples of 16 (else DL_ERR_INVALID_ARG).  Same kernel, same results. */
DL_API int dl_eval_packed_pitched(const void *x, int64_t x_pitch, const int64_t *a, const int64_t *b, const uint8_t *gate,
                                  void *y, int64_t y_pitch, int64_t n_in, int64_t n_out, int64_t row_bytes, void *stream);

/* argmax over the 16 gate weights -> uint8 gate id, first maximum on ties
 * (weights.argmax(-1).to(uint8), difflogic/difflogic.py:146). */
DL_API int dl_argmax_gate_u8(const float *w, uint8_t *gate, int64_t n_out, void *stream);

/* ------------------------------------------------------------------------------------------
 * Bit packing.
 * Replaces tensor_packbits_cuda, difflogic_kernel.cu:583-625 (kernel :547-581), bound at
 * difflogic.cpp:69-74.  t is bool (one byte, non-zero = true) feature-major [n][batch];
 * out is [n][ceil(batch/bit_count)] words, every word fully written, pad bits zero.
 * pad_len = (bit_count - batch % bit_count) % bit_count is the caller's to compute.
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_packbits(const uint8_t *t, void *out, int64_t n, int64_t batch, int bit_count, void *stream);

/* Same result from the batch-major matrix t[batch][n] the user holds: the transpose that
 * PackBitsTensor.__init__ does first (difflogic/packbitstensor.py:15) is folded in. */
DL_API int dl_packbits_batch_major(const uint8_t *t, void *out, int64_t n, int64_t batch, int bit_count,
                            void *stream);

/* Thermometer encoding + packing from uint8 features (the step in front of the packed path).
 * t[batch][n] uint8 -> out[n_thresholds*n][words]: bit s of row (i*n + f) is t[s][f] > thresholds[i].
 * thresholds is a HOST array (at most 16 entries).  Replaces the thermometer features of
 * experiments/main.py:56-59 (pixel/255 > (i+1)/4 for i = 0..2, i.e. thresholds {63, 127, 191}) followed by
 * PackBitsTensor(...) (difflogic/packbitstensor.py:15-16). */
DL_API int dl_threshold_packbits_batch_major(const uint8_t *t, const uint8_t *thresholds, int n_thresholds, void *out,
                                             int64_t n, int64_t batch, int bit_count, void *stream);

/* ------------------------------------------------------------------------------------------
 * Group bit-sum.
 * Replaces groupbitsum, difflogic_kernel.cu:666-700 (kernel :631-664), bound at
 * difflogic.cpp:75-83 (whose n % k check is DL_ERR_NOT_DIVISIBLE here).
 * x [n][words] -> out [batch][k] int32, batch = words*bit_count - pad_len, contiguous.
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_groupbitsum(const void *x, int32_t *out, int64_t n, int64_t words, int64_t pad_len, int64_t k,
                   int bit_count, void *stream);

/* ------------------------------------------------------------------------------------------
 * Last logic layer + group bit-sum in one launch: out equals dl_groupbitsum applied to the y of
 * dl_eval_packed(x, a, b, gate), but y is never written.  Replaces the last logic_layer_cuda_eval
 * (difflogic_kernel.cu:503-541) together with groupbitsum (:666-700) in the chain
 * model(PackBitsTensor) of experiments/main.py:198-210; bit-identical results.
 * dl_eval_groupbitsum_applicable returns 1 when the sizes are in the kernel's range (rows of at least
 * 512 bytes and a multiple of 16, x 16-byte aligned, n_out % k == 0, 32 <= n_out/k <= 2040), else 0;
 * dl_eval_groupbitsum returns DL_ERR_INVALID_ARG outside that range.  out [batch][k] int32,
 * batch = words*bit_count - pad_len.
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_eval_groupbitsum_applicable(const void *x, int64_t n_in, int64_t n_out, int64_t words, int bit_count, int64_t k);
DL_API int dl_eval_groupbitsum(const void *x, const int64_t *a, const int64_t *b, const uint8_t *gate, int32_t *out,
                               int64_t n_in, int64_t n_out, int64_t words, int64_t pad_len, int64_t k, int bit_count,
                               void *stream);

/* ------------------------------------------------------------------------------------------
 * Float GroupSum, forward and backward, on the feature-major activation of the last layer.
 * Replaces the torch expression of GroupSum.forward, difflogic/difflogic.py:195-196
 * (reshape -> sum -> / tau) and its autograd.
 *   out[s][c]    = (sum_{r < n/k} x[c*n/k + r][s]) / tau
 *   grad_x[i][s] = grad_out[s][i / (n/k)] / tau      (a true division, as the reference does)
 * The forward needs scratch memory: dl_groupsum_workspace_bytes(n, batch, k) bytes, 256-byte
 * aligned, owned by the caller.  Its first 4096 bytes hold counters that must be zero before
 * the first use; the kernel leaves them zero again.  Calls that share a workspace must not
 * overlap on the GPU.
 * ---------------------------------------------------------------------------------------- */
DL_API size_t dl_groupsum_workspace_bytes(int64_t n, int64_t batch, int64_t k);
DL_API int dl_groupsum_f32(const float *x, float *out, void *workspace, int64_t n, int64_t batch, int64_t k,
                    float tau, void *stream);
DL_API int dl_groupsum_backward_f32(const float *grad_out, float *grad_x, int64_t n, int64_t batch, int64_t k,
                             float tau, void *stream);

/* ------------------------------------------------------------------------------------------
 * dl_groupsum_f32 without a caller-owned workspace.  No counterpart in the reference (its GroupSum
 * is a torch expression that allocates through torch).
 *
 * For callers that cannot allocate device memory: a foreign-language binding that only forwards the
 * buffers its own framework handed it, or a process whose device memory pool is fixed and full.  The
 * scratch lives in a device array inside the library: dl_groupsum_static_limit_bytes() bytes (256 KiB)
 * per GPU, held from the first use of the library on that GPU until the process exits.  The call
 * allocates and frees nothing.  Limits and rules:
 *   - shapes that need more scratch than the limit (dl_groupsum_workspace_bytes(n, batch, k)) get
 *     DL_ERR_TOO_LARGE; shapes that dl_groupsum_f32 computes without scratch (several pieces per class and
 *     classes of 64 .. 4096 rows) are never refused;
 *   - the first call on a device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture;
 *   - every call on a GPU uses the same array: calls that may overlap on the GPU (different
 *     streams) race with each other and must be ordered by the caller.
 * Results are identical to dl_groupsum_f32.
 * ---------------------------------------------------------------------------------------- */
DL_API size_t dl_groupsum_static_limit_bytes(void);
DL_API int dl_groupsum_f32_static(const float *x, float *out, int64_t n, int64_t batch, int64_t k, float tau,
                                  void *stream);

/* ------------------------------------------------------------------------------------------
 * Cross-entropy loss (mean over the batch, int64 class targets) on the [batch][k] scores of a
 * GroupSum, and its backward.  Replaces torch.nn.CrossEntropyLoss as the reference's training
 * loop uses it (experiments/main.py:167,175: loss_fn(model(x), y), loss.backward()).
 *   forward : loss[0] = -(1/B) sum_s log softmax(logits[s])[target[s]];  probs[s][:] = softmax(logits[s])
 *   backward: grad_logits[s][c] = (probs[s][c] - [c == target[s]]) * grad_loss[0] / B
 * loss and grad_loss are device scalars.  Targets outside [0, k) contribute nothing.
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_cross_entropy_f32(const float *logits, const int64_t *target, float *loss, float *probs, int64_t batch,
                                int64_t k, void *stream);
DL_API int dl_cross_entropy_backward_f32(const float *probs, const int64_t *target, const float *grad_loss,
                                         float *grad_logits, int64_t batch, int64_t k, void *stream);
/* The head of a training step in one launch: GroupSum (difflogic/difflogic.py:195-196), the cross-entropy loss on
 * its scores (experiments/main.py:167,175) and the gradient of the loss w.r.t. the scores, laid out as one row per
 * CLASS: grad_classes [k][batch] = ((softmax(scores) - onehot(target)) / batch) / tau, i.e. the gradient of every
 * output row of that class (for loss.backward() with unit gradient).  The last layer's backward then runs as
 * dl_backward_w_classes_f32 / dl_backward_x_classes_f32, which take grad_classes in place of grad_y [n_out][batch].
 * scores [batch][k], loss a device scalar, counter one zeroed uint32 on the device (left zero).  Sizes:
 * dl_groupsum_cross_entropy_applicable (classes of 64 .. 4096 rows), else use the separate entry points. */
DL_API int dl_groupsum_cross_entropy_applicable(int64_t n, int64_t batch, int64_t k);
DL_API int dl_groupsum_cross_entropy_f32(const float *x, const int64_t *target, float *scores, float *loss, float *grad_classes,
                                         void *counter, int64_t n, int64_t batch, int64_t k, float tau, void *stream);
/* The same head in two launches that never form the last layer's output.  dl_forward_class_sums_f32 is the layer's
 * forward (as dl_forward_f32), but its CTAs add up their rows per class and store only those sums: class_sums
 * [dl_forward_class_sums_rows(n_out, batch, k)][batch] holds two rows per run of dl_forward_class_sums_run(batch)
 * consecutive neurons -- the sum over the run's rows that belong to the class of its first row, and the sum over those of
 * the next class (zero when the run does not reach it).  dl_class_sums_cross_entropy_f32 adds the runs of each class in
 * a fixed order and gives scores, loss and grad_classes as above.  Replaces logic_layer_cuda_forward
 * (difflogic_kernel.cu:259-297) of the last layer + GroupSum (difflogic/difflogic.py:195-196) + CrossEntropyLoss
 * (experiments/main.py:167,175) in training, where the layer's output itself is never needed (its backward reads the
 * layer's INPUT and grad_classes).  dl_forward_class_sums_rows returns 0 when a class is shorter than a run (use the
 * separate entry points then). */
DL_API int64_t dl_forward_class_sums_rows(int64_t n_out, int64_t batch, int64_t k);
DL_API int64_t dl_forward_class_sums_run(int64_t batch);
DL_API int dl_forward_class_sums_f32(const float *x, const int64_t *a, const int64_t *b, const float *w, int w_mode,
                                     float *class_sums, float *coef, int64_t n_in, int64_t n_out, int64_t batch, int64_t k,
                                     int flags, void *stream);
DL_API int dl_class_sums_cross_entropy_f32(const float *class_sums, const int64_t *target, float *scores, float *loss,
                                           float *grad_classes, void *counter, int64_t n, int64_t batch, int64_t k,
                                           int64_t rows_per_run, float tau, void *stream);
/* backward_w with the Adam step (update rule of dl_adam_step_f32) of the layer's weights in its epilogue: the 16
 * gradients of a neuron go from the registers straight into the update of w [n_out][16], exp_avg and exp_avg_sq (the
 * layer's slices, same layout as w); grad_w may be null, the gradient is then not stored.  state: two int32 on the
 * device that belong to THIS layer, {steps done, 0}, zero at first; the kernel takes the step number steps done + 1 and
 * advances the count when it is through (so each layer needs its own pair, and nothing has to run between the steps).
 * rows_per_class as in dl_backward_w_classes_f32 (1: grad_y has a row
 * per output).  Replaces logic_layer_cuda_backward_w (difflogic_kernel.cu:300-364) + softmax backward +
 * torch.optim.Adam.step for that layer (experiments/main.py:179). */
DL_API int dl_backward_w_adam_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, float *w, float *exp_avg,
                                  float *exp_avg_sq, float *grad_w, int64_t n_in, int64_t n_out, int64_t batch,
                                  int64_t rows_per_class, float lr, float beta1, float beta2, float eps, float grad_scale,
                                  int32_t *state, int flags, void *stream);
/* backward_w / backward_x of a layer whose output feeds a GroupSum: grad_y_classes has one row per class of
 * rows_per_class consecutive outputs, [n_out / rows_per_class][batch]; otherwise as dl_backward_w_f32 / dl_backward_x_f32. */
DL_API int dl_backward_w_classes_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y_classes,
                                     const float *w, int w_mode, float *grad_w, int64_t n_in, int64_t n_out, int64_t batch,
                                     int64_t rows_per_class, int flags, void *stream);
DL_API int dl_backward_x_classes_f32(const float *x, const float *coef, const float *grad_y_classes, const int64_t *start,
                                     const int32_t *plan, float grad_scale, float *grad_x, int64_t n_in, int64_t n_out,
                                     int64_t batch, int64_t rows_per_class, int flags, void *stream);
/* Backward of loss_fn(GroupSum(x), y) in one launch: dl_cross_entropy_backward_f32 followed by
 * dl_groupsum_backward_f32 (GroupSum of difflogic/difflogic.py:195-196 under the loss of experiments/main.py:167,175)
 * without the [batch][k] gradient in between; bit-identical to the two calls.  grad_x is feature-major [n][batch]. */
DL_API int dl_groupsum_cross_entropy_backward_f32(const float *probs, const int64_t *target, const float *grad_loss,
                                                  float *grad_x, int64_t n, int64_t batch, int64_t k, float tau, void *stream);

/* ------------------------------------------------------------------------------------------
 * Adam step over a flat fp32 parameter vector (all layers' gate weights in one buffer).
 * Replaces torch.optim.Adam(model.parameters(), lr).step() of the reference's training loop
 * (experiments/main.py:169,179), same update rule (no weight decay, no amsgrad):
 *   m = m + (g - m)(1 - beta1);  v = v beta2 + g g (1 - beta2);
 *   p = p - lr / (1 - beta1^t) * m / (sqrt(v) / sqrt(1 - beta2^t) + eps),     g = grad * grad_scale
 * state is two int32 on the device: {t (steps done so far), 0}; the kernel advances t, so the
 * launch can be replayed from a CUDA graph.  All buffers 16-byte aligned.
 * The kernel is launched with programmatic stream serialisation and reads param, exp_avg, exp_avg_sq and
 * state BEFORE it waits for the kernel in front of it in the stream; only grad is read after that wait.
 * The caller promises that the kernel just before this one in the stream writes none of the four (in a
 * training step it is a backward kernel, which writes gradients only).  dl_backward_w_adam_f32 makes the
 * same assumption for exp_avg, exp_avg_sq and state (w itself is read after the wait).
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_adam_step_f32(float *param, const float *grad, float *exp_avg, float *exp_avg_sq, int64_t n, float lr,
                            float beta1, float beta2, float eps, float grad_scale, int32_t *state, void *stream);
/* Pulls [ptr, ptr + bytes) towards L2 (prefetch.global.L2, 128-byte lines); no result, no reference counterpart.
 * Used on a side stream during the backward pass to warm the Adam moments, which are touched once per step. */
DL_API int dl_prefetch_l2(const void *ptr, size_t bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * Batch-sharded training: gradient exchange and Adam over peer memory, bucket by bucket.
 * No counterpart in the reference (it has no multi-GPU code); these kernels take the place of an
 * NCCL all-reduce of the [out_dim,16] gradients followed by dl_adam_step_f32 on every rank.
 *
 * Set-up (these DO allocate, once): every rank allocates its flat parameter buffer, flat gradient
 * buffer and dl_exchange_flag_bytes() bytes of flag words with dl_comm_alloc (zero-filled), exports
 * them with dl_comm_export (64-byte handles, to be passed to the other processes of the machine by
 * any means) and maps its peers' with dl_comm_import; dl_comm_close / dl_comm_free undo that.
 *
 * Per step and bucket -- a bucket is the range [offset, offset + count) of the flat buffers (floats,
 * multiples of 4), e.g. one layer's weights, numbered 0 .. 31:
 *   1. the rank's gradients of the bucket are announced to every peer (its "gradients complete" flag
 *      word in every rank's flag array is set to the bucket's step number): by the last block of
 *      dl_backward_w_announce_f32, i.e. by the kernel that writes them, or by dl_exchange_announce, or by
 *      dl_exchange_bucket_f32 itself (announce_here = 1);
 *   2. dl_exchange_bucket_f32, typically on a stream of its own as soon as the bucket's backward_w is in
 *      the queue, beside the rest of the backward pass: waits until all ranks have announced, averages
 *      slice `rank` of the bucket over all ranks' gradient buffers (peer loads), applies Adam to that
 *      slice (exp_avg / exp_avg_sq: buffers of the flat layout, of which every rank touches only its
 *      slices), writes the new parameters into its own parameter buffer and tells the peers; waits until
 *      all ranks' slices are complete, fetches the other ranks' slices (peer loads) into this rank's
 *      parameter buffer and advances the bucket's step count.  With whole_bucket = 1 every rank averages
 *      and updates the WHOLE bucket instead (identical arithmetic on every rank, full moments on every
 *      rank), nothing is fetched, and the kernel ends when all ranks have finished reading: one flag round
 *      trip less at (N-1) times the bucket over NVLink per rank -- for a small bucket that nothing else can
 *      hide.  A bucket keeps its form from step to step.
 * The pointer arguments are HOST arrays of `world` device pointers (index = rank, own entry = own
 * buffers).  state: sixteen int32 on the device PER BUCKET, zero at first: {steps done, ticket, error,
 * ticket} and six 64-bit nanosecond time stamps of the latest step (%globaltimer: kernel entered, all
 * ranks' gradients seen, own slice complete, unused, all ranks' slices seen, done).  A wait for the
 * peers takes at most wait_limit_us microseconds (0: the default of 20 seconds); when a wait runs out
 * the kernel sets `error` to 1, leaves parameters, moments and step count untouched and returns -- the
 * run cannot continue, but nothing hangs and nothing is corrupted.  flags: DL_LAUNCH_OVERLAP_SETUP when the
 * kernel is launched right behind the kernel that wrote this rank's gradients of the bucket, in the
 * same stream.  All ranks must launch the same buckets, one rank per GPU (the kernels of one step
 * must be able to run at the same time on their GPUs).  The kernel waits for other GPUs only.
 *
 * dl_backward_w_announce_f32: dl_backward_w_classes_f32 with DL_W_LOGITS whose last block does step 1.
 * bucket_state: the bucket's sixteen int32 (the step number announced is steps done + 1);
 * block_ticket: one zeroed int32 per parameter; kernel_count: one zeroed int32 per bucket, shared by the
 * kernels_in_bucket backward_w kernels per step that write into the bucket (the last one announces).
 * ---------------------------------------------------------------------------------------- */
DL_API int dl_comm_alloc(size_t bytes, void **ptr);
DL_API int dl_comm_free(void *ptr);
DL_API int dl_comm_export(void *ptr, unsigned char *handle);
DL_API int dl_comm_import(const unsigned char *handle, void **ptr);
DL_API int dl_comm_close(void *ptr);
DL_API size_t dl_exchange_flag_bytes(void);
DL_API int dl_exchange_flag_word(int bucket, int rank, int which);
DL_API int dl_exchange_announce(void *const *flag_ptrs, int rank, int world, int bucket, const int32_t *state, void *stream);
/* A barrier of the ranks on the device: the kernel raises this rank's word (bucket, rank, 0) in every rank's flags to
 * state[0] + 1 and waits (wait_limit_us, 0: 20 s) until all ranks' words in its own flags are there; then state[0]
 * advances, else state[2] is set.  `bucket`: a bucket number that no exchange uses; state: sixteen int32, zero at first.
 * For aligning the ranks in front of a timed step, or wherever a host-side barrier would stall the launch queue. */
DL_API int dl_rank_barrier(void *const *flag_ptrs, int rank, int world, int bucket, int32_t *state, uint32_t wait_limit_us,
                           void *stream);
DL_API int dl_exchange_bucket_f32(void *const *param_ptrs, void *const *grad_ptrs, void *const *flag_ptrs, int rank, int world,
                                  float *exp_avg, float *exp_avg_sq, int64_t offset, int64_t count, int bucket, float lr,
                                  float beta1, float beta2, float eps, int32_t *state, int announce_here, int whole_bucket,
                                  uint32_t wait_limit_us, int flags, void *stream);
/* The exchange of one SMALL bucket with the flags inside the data: every float crosses NVLink as an 8-byte packet
 * {value, step number} stored into the receiver's inbox, so a packet announces itself and there is no flag round trip, no
 * fence and no pull: gradients of the other ranks' slices are pushed to their owners; the owner adds up its slice in rank
 * order (the same sums as dl_exchange_bucket_f32), applies Adam and pushes the new parameters to every peer; the peers take
 * them out of their inboxes.  NVLink carries 4 (N-1)/N times the bucket per rank.  param, grad, exp_avg, exp_avg_sq: this
 * rank's flat buffers; grad_inbox_ptrs / param_inbox_ptrs: host arrays of `world` device pointers (index = rank) to every
 * rank's two inboxes, 32 * world * inbox_stride bytes each, zero at first, peer-mapped (dl_comm_*); inbox_offset: the
 * bucket's first float4 slot inside a sender's region of inbox_stride slots (a bucket needs ceil(count / 4 / world)).
 * state, wait_limit_us, flags: as for dl_exchange_bucket_f32 (no flag words are used); after a wait that ran out the
 * error word is set and part of the bucket may have been updated.  pushed = 1: the gradients of the other ranks' slices
 * are in their inboxes already (dl_backward_w_push_f32) and are not pushed again. */
DL_API int dl_exchange_packets_f32(float *param, const float *grad, void *const *grad_inbox_ptrs, void *const *param_inbox_ptrs,
                                   int rank, int world, float *exp_avg, float *exp_avg_sq, int64_t offset, int64_t count,
                                   int64_t inbox_offset, int64_t inbox_stride, float lr, float beta1, float beta2, float eps,
                                   int32_t *state, int pushed, uint32_t wait_limit_us, int flags, void *stream);
/* backward_w and the first half of that exchange in ONE kernel: dl_backward_w_classes_f32 with DL_W_LOGITS whose epilogue
 * also sends every gradient that belongs to another rank's slice of the bucket straight from the registers into that
 * rank's gradient inbox, as a packet, while the kernel is still working on its other neurons -- the transfer over
 * NVLink runs beside the arithmetic, and dl_exchange_packets_f32 (then called with pushed = 1) finds most packets
 * there.  The gradient is stored into grad_w as well.  bucket_offset: floats of the bucket in front of this layer's
 * gradients (0 when the bucket is the layer); bucket_count: floats of the whole bucket; bucket_state: the bucket's state
 * (read only: the packets carry steps done + 1).  Every kernel that writes into the bucket must push, or none.
 * Measured on config 2 with two ranks: the exchange kernel gets 2 us shorter and every backward_w kernel longer by more
 * (93.9 against 91.1 us per step), so FlatAdam leaves it off unless asked. */
DL_API int dl_backward_w_push_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, const float *w,
                                  float *grad_w, int64_t n_in, int64_t n_out, int64_t batch, int64_t rows_per_class,
                                  void *const *grad_inbox_ptrs, int rank, int world, int64_t bucket_offset,
                                  int64_t bucket_count, int64_t inbox_offset, int64_t inbox_stride,
                                  const int32_t *bucket_state, int flags, void *stream);
DL_API int dl_backward_w_announce_f32(const float *x, const int64_t *a, const int64_t *b, const float *grad_y, const float *w,
                                      float *grad_w, int64_t n_in, int64_t n_out, int64_t batch, int64_t rows_per_class,
                                      void *const *flag_ptrs, int rank, int world, int bucket, const int32_t *bucket_state,
                                      int32_t *block_ticket, int32_t *kernel_count, int kernels_in_bucket, int flags,
                                      void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DIFFLOGIC_B200_H */
