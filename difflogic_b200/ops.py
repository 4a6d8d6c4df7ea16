"""Tensor-level operators over the C ABI (include/difflogic_b200.h).

Each function checks its tensors, lets torch allocate the output on the inputs' device and
launches the kernel on torch's current stream.  Nothing here computes on the CPU; a missing
library raises (see _native.lib()).

Layouts: float activations are feature-major `[features, batch]` contiguous; packed
activations are `[features, words]`; indices are int64, as LogicLayer stores them.
"""
import torch

from . import _native as N
from ._native import W_ARGMAX, W_LOGITS, W_PROBS  # noqa: F401  (re-exported)

_BITS_TO_DTYPE = {8: torch.int8, 16: torch.int16, 32: torch.int32, 64: torch.int64}
_DTYPE_TO_BITS = {v: k for k, v in _BITS_TO_DTYPE.items()}
_DTYPE_TO_BITS[torch.uint8] = 8


def _need(cond, msg):
    if not cond:
        raise RuntimeError("difflogic_b200: " + msg)


def _f32_matrix(t, name):
    N.require_cuda(t)
    _need(t.dtype == torch.float32, "%s must be float32, got %s (the CUDA path computes in fp32)" % (name, t.dtype))
    _need(t.dim() == 2 and t.is_contiguous(), "%s must be a contiguous 2-D tensor" % name)


def _index(t, name, n=None):
    N.require_cuda(t)
    _need(t.dtype == torch.int64 and t.dim() == 1 and t.is_contiguous(), "%s must be a contiguous int64 vector" % name)
    if n is not None:
        _need(t.numel() == n, "%s has %d entries, expected %d" % (name, t.numel(), n))


# ------------------------------------------------------------------------------------------------
# training
# ------------------------------------------------------------------------------------------------

def logic_forward(x, a, b, w, w_mode=W_LOGITS, want_coef=False, overlap=False):
    """y[j,:] = sum_i p[j,i] gate_i(x[a_j,:], x[b_j,:]);  returns (y [n_out,batch], coef or None).

    overlap=True lets the kernel read `a`, `b` while the previous kernel in the stream is still running; pass
    it only when those index tensors were complete before that kernel was launched (see DL_LAUNCH_OVERLAP_SETUP)."""
    _f32_matrix(x, "x")
    _f32_matrix(w, "w")
    n_in, batch = x.shape
    n_out = w.shape[0]
    _need(w.shape[1] == 16, "w must be [n_out, 16]")
    _index(a, "a", n_out)
    _index(b, "b", n_out)
    y = torch.empty((n_out, batch), dtype=torch.float32, device=x.device)
    coef = torch.empty((n_out, 4), dtype=torch.float32, device=x.device) if want_coef else None
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_forward_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), w.data_ptr(), w_mode, y.data_ptr(),
                                       N.ptr(coef), n_in, n_out, batch, int(overlap), N.stream_of(x)))
    return y, coef


def logic_coefs(w, w_mode=W_LOGITS):
    _f32_matrix(w, "w")
    _need(w.shape[1] == 16, "w must be [n_out, 16]")
    coef = torch.empty((w.shape[0], 4), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        N.check(N.lib().dl_coefs_f32(w.data_ptr(), w_mode, coef.data_ptr(), w.shape[0], N.stream_of(w)))
    return coef


def transpose(x):
    """[rows, cols] float32 -> its transpose as a new contiguous tensor (dl_transpose_f32)."""
    _f32_matrix(x, "x")
    y = torch.empty((x.shape[1], x.shape[0]), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_transpose_f32(x.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], N.stream_of(x)))
    return y


def logic_backward_w(x, a, b, grad_y, w=None, w_mode=W_PROBS, out=None, overlap=False, rows_per_class=1):
    """[n_out,16] gradient: w_mode=W_PROBS w.r.t. the mixing weights, W_LOGITS w.r.t. the raw
    parameters `w` (softmax backward applied in the kernel).  rows_per_class > 1: grad_y holds one row per class of
    that many consecutive outputs (the gradient that comes back through a GroupSum), [n_out / rows_per_class, batch]."""
    _f32_matrix(x, "x")
    _f32_matrix(grad_y, "grad_y")
    n_in, batch = x.shape
    rows_per_class = int(rows_per_class)
    _need(rows_per_class >= 1, "rows_per_class must be positive")
    n_out = grad_y.shape[0] * rows_per_class
    _need(grad_y.shape[1] == batch, "grad_y and x disagree on the batch size")
    _index(a, "a", n_out)
    _index(b, "b", n_out)
    if w_mode == W_LOGITS:
        _need(w is not None, "W_LOGITS needs the raw weights")
        _f32_matrix(w, "w")
        _need(tuple(w.shape) == (n_out, 16), "w must be [n_out, 16]")
    if out is None:
        out = torch.empty((n_out, 16), dtype=torch.float32, device=x.device)
    else:
        _f32_matrix(out, "out")
        _need(tuple(out.shape) == (n_out, 16), "out must be [n_out, 16]")
    with torch.cuda.device(x.device):
        if rows_per_class == 1:
            N.check(N.lib().dl_backward_w_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), grad_y.data_ptr(), N.ptr(w), w_mode,
                                              out.data_ptr(), n_in, n_out, batch, int(overlap), N.stream_of(x)))
        else:
            N.check(N.lib().dl_backward_w_classes_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), grad_y.data_ptr(), N.ptr(w), w_mode,
                                                      out.data_ptr(), n_in, n_out, batch, rows_per_class, int(overlap),
                                                      N.stream_of(x)))
    return out


def logic_backward_w_adam(x, a, b, grad_y, w, exp_avg, exp_avg_sq, state, lr, beta1, beta2, eps, grad_scale=1.0, grad_out=None,
                          overlap=False, rows_per_class=1):
    """backward_w of a layer with the Adam step of its weights in the kernel's epilogue: `w` [n_out, 16] and its moment
    slices are updated in place; the gradient is stored only when `grad_out` is given.  `state`: two int32 on the device
    that belong to this layer, {steps done, 0}; the kernel advances the count."""
    _f32_matrix(x, "x")
    _f32_matrix(grad_y, "grad_y")
    _f32_matrix(w, "w")
    n_in, batch = x.shape
    rows_per_class = int(rows_per_class)
    n_out = grad_y.shape[0] * rows_per_class
    _need(grad_y.shape[1] == batch, "grad_y and x disagree on the batch size")
    _need(tuple(w.shape) == (n_out, 16), "w must be [n_out, 16]")
    _index(a, "a", n_out)
    _index(b, "b", n_out)
    for t, name in ((exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        _need(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.numel() >= n_out * 16 and t.device == x.device,
              "%s must be a contiguous float32 CUDA tensor of at least n_out * 16 elements" % name)
    _need(state.is_cuda and state.dtype == torch.int32 and state.numel() >= 2 and state.is_contiguous(),
          "state must be a contiguous int32 CUDA tensor of two elements")
    if grad_out is not None:
        _f32_matrix(grad_out, "grad_out")
        _need(tuple(grad_out.shape) == (n_out, 16), "grad_out must be [n_out, 16]")
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_backward_w_adam_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), grad_y.data_ptr(), w.data_ptr(),
                                               exp_avg.data_ptr(), exp_avg_sq.data_ptr(), N.ptr(grad_out), n_in, n_out, batch,
                                               rows_per_class, float(lr), float(beta1), float(beta2), float(eps), float(grad_scale),
                                               state.data_ptr(), int(overlap), N.stream_of(x)))
    return grad_out


def logic_backward_w_announce(x, a, b, grad_y, w, out, rows_per_class, flag_ptrs, rank, world, bucket, bucket_state, block_ticket,
                              kernel_count, kernels_in_bucket):
    """logic_backward_w (W_LOGITS) into `out` [n_out, 16] whose last block announces the gradients of exchange bucket
    `bucket` to the peers (dl_backward_w_announce_f32).  flag_ptrs: ctypes array of the ranks' flag words;
    bucket_state / block_ticket / kernel_count: int32 device tensors (see the header)."""
    _f32_matrix(x, "x")
    _f32_matrix(grad_y, "grad_y")
    _f32_matrix(w, "w")
    _f32_matrix(out, "out")
    n_in, batch = x.shape
    rows_per_class = int(rows_per_class)
    n_out = grad_y.shape[0] * rows_per_class
    _need(grad_y.shape[1] == batch, "grad_y and x disagree on the batch size")
    _need(tuple(w.shape) == (n_out, 16) and tuple(out.shape) == (n_out, 16), "w and out must be [n_out, 16]")
    _index(a, "a", n_out)
    _index(b, "b", n_out)
    for t in (bucket_state, block_ticket, kernel_count):
        _need(t.is_cuda and t.dtype == torch.int32 and t.numel() >= 1, "state words must be int32 CUDA tensors")
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_backward_w_announce_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), grad_y.data_ptr(), w.data_ptr(),
                                                   out.data_ptr(), n_in, n_out, batch, rows_per_class, flag_ptrs, rank, world, bucket,
                                                   bucket_state.data_ptr(), block_ticket.data_ptr(), kernel_count.data_ptr(),
                                                   int(kernels_in_bucket), N.LAUNCH_OVERLAP_SETUP, N.stream_of(x)))
    return out


def inverse_index(a, b, n_in):
    """The reference's inverse connection index (difflogic/difflogic.py:56-69) built with device
    ops: for every input row the consumer neurons in increasing order, a neuron whose two inputs
    are the same row listed twice.  Returns (start [n_in+1] int64, list [2*n_out] int64)."""
    keys = torch.stack([a, b], dim=1).reshape(-1)           # position 2*j + slot
    order = torch.argsort(keys, stable=True)
    counts = torch.bincount(keys, minlength=n_in)
    start = torch.zeros(n_in + 1, dtype=torch.int64, device=a.device)
    start[1:] = torch.cumsum(counts, 0)
    return start, (order // 2).contiguous()


def build_backward_plan(a, b, start, lst):
    n_out = a.numel()
    n_in = start.numel() - 1
    _index(a, "a")
    _index(b, "b", n_out)
    _index(start, "start")
    _index(lst, "list", 2 * n_out)
    plan = torch.empty((2 * n_out, 2), dtype=torch.int32, device=a.device)
    with torch.cuda.device(a.device):
        N.check(N.lib().dl_build_backward_plan(a.data_ptr(), b.data_ptr(), start.data_ptr(), lst.data_ptr(),
                                               plan.data_ptr(), n_in, n_out, N.stream_of(a)))
    return plan


_VIOLATIONS = {1: "connection index outside [0, in_dim)", 2: "inverse-index offsets are not 0 = start[0] <= ... <= start[in_dim] = 2 * out_dim",
               3: "inverse-index entry outside [0, out_dim)", 4: "gather-plan entry out of range",
               5: "gather-plan entry does not match the connections"}


def logic_backward_w_push(x, a, b, grad_y, w, out, rows_per_class, grad_inbox_ptrs, rank, world, bucket_offset, bucket_count,
                          inbox_offset, inbox_stride, bucket_state):
    """logic_backward_w (W_LOGITS) into `out` [n_out, 16] that also pushes the gradients of the other ranks' slices of the
    exchange bucket into their inboxes as packets (dl_backward_w_push_f32).  grad_inbox_ptrs: ctypes array of the ranks'
    gradient inboxes; bucket_offset / bucket_count: floats in front of this layer inside the bucket / of the bucket."""
    _f32_matrix(x, "x")
    _f32_matrix(grad_y, "grad_y")
    _f32_matrix(w, "w")
    _f32_matrix(out, "out")
    n_in, batch = x.shape
    rows_per_class = int(rows_per_class)
    n_out = grad_y.shape[0] * rows_per_class
    _need(grad_y.shape[1] == batch, "grad_y and x disagree on the batch size")
    _need(tuple(w.shape) == (n_out, 16) and tuple(out.shape) == (n_out, 16), "w and out must be [n_out, 16]")
    _index(a, "a", n_out)
    _index(b, "b", n_out)
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_backward_w_push_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), grad_y.data_ptr(), w.data_ptr(), out.data_ptr(),
                                               n_in, n_out, batch, rows_per_class, grad_inbox_ptrs, int(rank), int(world),
                                               int(bucket_offset), int(bucket_count), int(inbox_offset), int(inbox_stride),
                                               bucket_state.data_ptr(), N.LAUNCH_OVERLAP_SETUP, N.stream_of(x)))
    return out


def check_connections(a, b, n_in, start=None, lst=None, plan=None):
    """Checks a layer's index tensors on the device (dl_check_connections) and raises ValueError with the first violation
    found.  Synchronises; meant for construction time and debugging, not for the hot path."""
    n_out = a.numel()
    _index(a, "a")
    _index(b, "b", n_out)
    if start is not None:
        _index(start, "start", n_in + 1)
    if lst is not None:
        _index(lst, "list", 2 * n_out)
    if plan is not None:
        _need(plan.is_cuda and plan.dtype == torch.int32 and plan.is_contiguous() and tuple(plan.shape) == (2 * n_out, 2),
              "plan must be a contiguous int32 [2*n_out, 2] tensor")
    report = torch.zeros(4, dtype=torch.int64, device=a.device)
    with torch.cuda.device(a.device):
        N.check(N.lib().dl_check_connections(a.data_ptr(), b.data_ptr(), N.ptr(start), N.ptr(lst), N.ptr(plan), int(n_in), n_out,
                                             report.data_ptr(), N.stream_of(a)))
    code, where, value, limit = report.tolist()
    if code != 0:
        raise ValueError("difflogic_b200: %s (position %d, value %d, limit %d)" % (_VIOLATIONS.get(code, "violation %d" % code),
                                                                                 where, value, limit))


def logic_backward_x(x, coef, grad_y, start, plan, grad_scale=1.0, overlap=False, rows_per_class=1):
    """Gradient w.r.t. the layer's input.  rows_per_class > 1: grad_y holds one row per class (see logic_backward_w)."""
    _f32_matrix(x, "x")
    _f32_matrix(grad_y, "grad_y")
    _f32_matrix(coef, "coef")
    n_in, batch = x.shape
    rows_per_class = int(rows_per_class)
    _need(rows_per_class >= 1, "rows_per_class must be positive")
    n_out = grad_y.shape[0] * rows_per_class
    _need(grad_y.shape[1] == batch, "grad_y and x disagree on the batch size")
    _need(tuple(coef.shape) == (n_out, 4), "coef must be [n_out, 4]")
    _index(start, "start", n_in + 1)
    N.require_cuda(plan)
    _need(plan.dtype == torch.int32 and plan.is_contiguous() and tuple(plan.shape) == (2 * n_out, 2),
          "plan must be a contiguous int32 [2*n_out, 2] tensor")
    gx = torch.empty_like(x)
    with torch.cuda.device(x.device):
        if rows_per_class == 1:
            N.check(N.lib().dl_backward_x_f32(x.data_ptr(), coef.data_ptr(), grad_y.data_ptr(), start.data_ptr(),
                                              plan.data_ptr(), float(grad_scale), gx.data_ptr(), n_in, n_out, batch,
                                              int(overlap), N.stream_of(x)))
        else:
            N.check(N.lib().dl_backward_x_classes_f32(x.data_ptr(), coef.data_ptr(), grad_y.data_ptr(), start.data_ptr(),
                                                      plan.data_ptr(), float(grad_scale), gx.data_ptr(), n_in, n_out, batch,
                                                      rows_per_class, int(overlap), N.stream_of(x)))
    return gx


# ------------------------------------------------------------------------------------------------
# packed-bit inference
# ------------------------------------------------------------------------------------------------

def bits_of(t):
    _need(t.dtype in _DTYPE_TO_BITS, "packed tensor must be int8/int16/int32/int64, got %s" % t.dtype)
    return _DTYPE_TO_BITS[t.dtype]


def argmax_gates(w):
    _f32_matrix(w, "w")
    _need(w.shape[1] == 16, "w must be [n_out, 16]")
    g = torch.empty((w.shape[0],), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        N.check(N.lib().dl_argmax_gate_u8(w.data_ptr(), g.data_ptr(), w.shape[0], N.stream_of(w)))
    return g


def eval_packed(x, a, b, gate, out=None):
    N.require_cuda(x, gate)
    _need(x.dim() == 2 and x.is_contiguous(), "x must be a contiguous 2-D tensor")
    bits = bits_of(x)
    n_in, words = x.shape
    n_out = gate.numel()
    _need(gate.dtype == torch.uint8 and gate.is_contiguous(), "gate must be a contiguous uint8 vector")
    _index(a, "a", n_out)
    _index(b, "b", n_out)
    if out is None:
        out = torch.empty((n_out, words), dtype=x.dtype, device=x.device)
    else:
        _need(out.dtype == x.dtype and tuple(out.shape) == (n_out, words) and out.is_contiguous() and out.is_cuda,
              "out must be a contiguous [n_out, words] tensor of x's dtype")
        _need(out.data_ptr() != x.data_ptr(), "eval_packed cannot run in place")
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_eval_packed(x.data_ptr(), a.data_ptr(), b.data_ptr(), gate.data_ptr(), out.data_ptr(),
                                       n_in, n_out, words, bits, N.stream_of(x)))
    return out


def _as_bool_bytes(t):
    N.require_cuda(t)
    _need(t.dim() == 2 and t.is_contiguous(), "t must be a contiguous 2-D tensor")
    _need(t.dtype in (torch.bool, torch.uint8), "t must be a bool tensor, got %s" % t.dtype)
    return t


def _check_bit_count(bit_count):
    if bit_count not in _BITS_TO_DTYPE:
        raise ValueError("`bit_count` has to be in { 8, 16, 32, 64 }")


def packbits(t, bit_count):
    """bool [n, batch] (feature-major) -> (words [n, ceil(batch/bit_count)], pad_len)."""
    _check_bit_count(bit_count)
    t = _as_bool_bytes(t)
    n, batch = t.shape
    words = -(-batch // bit_count)
    out = torch.empty((n, words), dtype=_BITS_TO_DTYPE[bit_count], device=t.device)
    with torch.cuda.device(t.device):
        N.check(N.lib().dl_packbits(t.data_ptr(), out.data_ptr(), n, batch, bit_count, N.stream_of(t)))
    return out, (bit_count - batch % bit_count) % bit_count


def packbits_batch_major(t, bit_count):
    """bool [batch, n] (as the user holds it) -> (words [n, ceil(batch/bit_count)], pad_len)."""
    _check_bit_count(bit_count)
    t = _as_bool_bytes(t)
    batch, n = t.shape
    words = -(-batch // bit_count)
    out = torch.empty((n, words), dtype=_BITS_TO_DTYPE[bit_count], device=t.device)
    with torch.cuda.device(t.device):
        N.check(N.lib().dl_packbits_batch_major(t.data_ptr(), out.data_ptr(), n, batch, bit_count, N.stream_of(t)))
    return out, (bit_count - batch % bit_count) % bit_count


def threshold_packbits_batch_major(t, thresholds, bit_count):
    """uint8 [batch, n] -> (words [len(thresholds)*n, ceil(batch/bit_count)], pad_len); bit s of row i*n+f is
    t[s, f] > thresholds[i] (thermometer encoding and packing in one kernel)."""
    import ctypes
    _check_bit_count(bit_count)
    N.require_cuda(t)
    _need(t.dim() == 2 and t.is_contiguous() and t.dtype == torch.uint8, "t must be a contiguous 2-D uint8 tensor")
    thresholds = [int(v) for v in thresholds]
    _need(1 <= len(thresholds) <= 16 and all(0 <= v <= 255 for v in thresholds), "1..16 thresholds in 0..255")
    batch, n = t.shape
    words = -(-batch // bit_count)
    out = torch.empty((len(thresholds) * n, words), dtype=_BITS_TO_DTYPE[bit_count], device=t.device)
    arr = (ctypes.c_ubyte * len(thresholds))(*thresholds)
    with torch.cuda.device(t.device):
        N.check(N.lib().dl_threshold_packbits_batch_major(t.data_ptr(), ctypes.addressof(arr), len(thresholds), out.data_ptr(),
                                                          n, batch, bit_count, N.stream_of(t)))
    return out, (bit_count - batch % bit_count) % bit_count


def groupbitsum(x, pad_len, k):
    """words [n, W] -> int32 [W*bits - pad_len, k] class counts."""
    N.require_cuda(x)
    _need(x.dim() == 2 and x.is_contiguous(), "x must be a contiguous 2-D tensor")
    bits = bits_of(x)
    n, words = x.shape
    k = int(k)
    if k <= 0 or n % k != 0:
        raise ValueError("in_dim (%d) has to be divisible by k (%d) but it is not" % (n, k))
    batch = words * bits - int(pad_len)
    _need(batch >= 0, "pad_len exceeds the packed batch")
    out = torch.empty((batch, k), dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_groupbitsum(x.data_ptr(), out.data_ptr(), n, words, int(pad_len), k, bits, N.stream_of(x)))
    return out


def eval_groupbitsum_applicable(x, n_out, k):
    """True when the fused last-layer + group bit-sum kernel takes a layer of n_out gates on packed words x."""
    if not (x.is_cuda and x.dim() == 2 and x.is_contiguous()):
        return False
    n_in, words = x.shape
    return N.lib().dl_eval_groupbitsum_applicable(x.data_ptr(), n_in, int(n_out), words, bits_of(x), int(k)) == 1


def eval_groupbitsum(x, a, b, gate, pad_len, k):
    """groupbitsum(eval_packed(x, a, b, gate), pad_len, k) in one kernel; the layer's output is never stored."""
    N.require_cuda(x, a, b, gate)
    _need(x.dim() == 2 and x.is_contiguous(), "x must be a contiguous 2-D tensor")
    _need(a.dtype == torch.int64 and b.dtype == torch.int64 and gate.dtype == torch.uint8, "a, b int64 and gate uint8")
    _need(a.numel() == b.numel() == gate.numel(), "a, b and gate must have one entry per gate")
    bits = bits_of(x)
    n_in, words = x.shape
    n_out, k = a.numel(), int(k)
    if k <= 0 or n_out % k != 0:
        raise ValueError("in_dim (%d) has to be divisible by k (%d) but it is not" % (n_out, k))
    batch = words * bits - int(pad_len)
    _need(batch >= 0, "pad_len exceeds the packed batch")
    out = torch.empty((batch, k), dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_eval_groupbitsum(x.data_ptr(), a.data_ptr(), b.data_ptr(), gate.data_ptr(), out.data_ptr(), n_in, n_out,
                                            words, int(pad_len), k, bits, N.stream_of(x)))
    return out


# ------------------------------------------------------------------------------------------------
# float GroupSum
# ------------------------------------------------------------------------------------------------

_workspaces = {}


def _groupsum_workspace(device, stream, nbytes):
    """Zero-initialised scratch for dl_groupsum_f32, grown on demand.  The kernel leaves the counters at
    zero, so a buffer is cleared only when it is created.  Eager calls use one buffer per (device, stream).
    Calls made while a CUDA graph is being captured share one buffer per device that is created by the first
    eager call on that device (warm-up steps), so that a captured step contains no allocation and no memset;
    graphs replayed concurrently on different streams must therefore not both contain a GroupSum."""
    want = max(nbytes, 1 << 20)
    graph_key = (device, "graph")
    capturing = torch.cuda.is_current_stream_capturing()
    if not capturing:
        gws = _workspaces.get(graph_key)
        if gws is None or gws.numel() < want:
            _workspaces[graph_key] = torch.zeros(want, dtype=torch.uint8, device=device)
    key = graph_key if capturing else (device, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(want, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def groupsum(x, k, tau):
    """feature-major x [n, batch] -> [batch, k] = per-class row sums / tau."""
    _f32_matrix(x, "x")
    n, batch = x.shape
    k = int(k)
    _need(k > 0 and n % k == 0, "n (%d) must be divisible by k (%d)" % (n, k))
    out = torch.empty((batch, k), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        stream = N.stream_of(x)
        ws = _groupsum_workspace(x.device, stream, N.lib().dl_groupsum_workspace_bytes(n, batch, k))
        N.check(N.lib().dl_groupsum_f32(x.data_ptr(), out.data_ptr(), ws.data_ptr(), n, batch, k, float(tau), stream))
    return out


_HEAD_COUNTERS = {}


def groupsum_cross_entropy_applicable(n, batch, k):
    return N.lib().dl_groupsum_cross_entropy_applicable(int(n), int(batch), int(k)) == 1


def groupsum_cross_entropy(x, target, k, tau):
    """Head of a training step in one kernel.  feature-major x [n, batch], int64 target [batch] ->
    (loss scalar, scores [batch, k], grad_classes [k, batch]); grad_classes is the gradient of the mean cross-entropy
    loss w.r.t. every output row of a class, for logic_backward_w / logic_backward_x with rows_per_class = n / k."""
    _f32_matrix(x, "x")
    n, batch = x.shape
    k = int(k)
    _need(k > 0 and n % k == 0, "n (%d) must be divisible by k (%d)" % (n, k))
    _need(target.is_cuda and target.dtype == torch.int64 and target.dim() == 1 and target.is_contiguous()
          and target.shape[0] == batch and target.device == x.device, "target must be a contiguous int64 [batch] CUDA tensor")
    _need(groupsum_cross_entropy_applicable(n, batch, k), "classes of %d rows are outside the fused kernel's range" % (n // k))
    scores = torch.empty((batch, k), dtype=torch.float32, device=x.device)
    loss = torch.empty((), dtype=torch.float32, device=x.device)
    grad_classes = torch.empty((k, batch), dtype=torch.float32, device=x.device)
    counter = _HEAD_COUNTERS.get(x.device)
    if counter is None:
        counter = _HEAD_COUNTERS[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        N.check(N.lib().dl_groupsum_cross_entropy_f32(x.data_ptr(), target.data_ptr(), scores.data_ptr(), loss.data_ptr(),
                                                      grad_classes.data_ptr(), counter.data_ptr(), n, batch, k, float(tau),
                                                      N.stream_of(x)))
    return loss, scores, grad_classes


def forward_head_applicable(n_out, batch, k):
    """True when logic_forward_head takes these sizes: classes at least as long as a forward CTA's run of rows."""
    return N.lib().dl_forward_class_sums_rows(int(n_out), int(batch), int(k)) > 0


def logic_forward_head(x, a, b, w, target, k, tau, w_mode=W_LOGITS):
    """Last layer + GroupSum(k, tau) + mean cross-entropy in two kernels that never store the layer's output:
    (loss scalar, scores [batch, k], grad_classes [k, batch], coef [n_out, 4]).  The forward kernel's CTAs add up
    their rows per class; a small second kernel adds those pieces in a fixed order and does the loss.  grad_classes
    is for logic_backward_w / logic_backward_x with rows_per_class = n_out / k."""
    _f32_matrix(x, "x")
    _f32_matrix(w, "w")
    n_in, batch = x.shape
    n_out, k = w.shape[0], int(k)
    _need(w.shape[1] == 16, "w must be [n_out, 16]")
    _index(a, "a", n_out)
    _index(b, "b", n_out)
    _need(k > 0 and n_out % k == 0, "n_out (%d) must be divisible by k (%d)" % (n_out, k))
    _need(target.is_cuda and target.dtype == torch.int64 and target.dim() == 1 and target.is_contiguous()
          and target.shape[0] == batch and target.device == x.device, "target must be a contiguous int64 [batch] CUDA tensor")
    lib = N.lib()
    rows = lib.dl_forward_class_sums_rows(n_out, batch, k)
    _need(rows > 0, "classes of %d rows are shorter than a forward CTA's run of rows" % (n_out // k))
    sums = torch.empty((rows, batch), dtype=torch.float32, device=x.device)
    coef = torch.empty((n_out, 4), dtype=torch.float32, device=x.device)
    scores = torch.empty((batch, k), dtype=torch.float32, device=x.device)
    loss = torch.empty((), dtype=torch.float32, device=x.device)
    grad_classes = torch.empty((k, batch), dtype=torch.float32, device=x.device)
    counter = _HEAD_COUNTERS.get(x.device)
    if counter is None:
        counter = _HEAD_COUNTERS[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        st = N.stream_of(x)
        N.check(lib.dl_forward_class_sums_f32(x.data_ptr(), a.data_ptr(), b.data_ptr(), w.data_ptr(), w_mode, sums.data_ptr(),
                                              coef.data_ptr(), n_in, n_out, batch, k, N.LAUNCH_OVERLAP_SETUP, st))
        N.check(lib.dl_class_sums_cross_entropy_f32(sums.data_ptr(), target.data_ptr(), scores.data_ptr(), loss.data_ptr(),
                                                    grad_classes.data_ptr(), counter.data_ptr(), n_out, batch, k,
                                                    lib.dl_forward_class_sums_run(batch), float(tau), st))
    return loss, scores, grad_classes, coef


def groupsum_backward(grad_out, n, tau):
    """[batch, k] -> feature-major [n, batch] with grad_x[i,:] = grad_out[:, i // (n/k)] / tau."""
    _f32_matrix(grad_out, "grad_out")
    batch, k = grad_out.shape
    gx = torch.empty((n, batch), dtype=torch.float32, device=grad_out.device)
    with torch.cuda.device(grad_out.device):
        N.check(N.lib().dl_groupsum_backward_f32(grad_out.data_ptr(), gx.data_ptr(), n, batch, k, float(tau),
                                                 N.stream_of(grad_out)))
    return gx
