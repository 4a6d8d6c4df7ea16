"""CPU oracle for the logic-layer hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the algorithm of the reference
(Felix-Petersen/difflogic) for the training forward/backward, the packed-bit
eval, bit packing and the group bit-sum.  It is the checker the CUDA path is
compared with; nothing in the shipped package imports it.  Only the tests, the
smoke check and the CPU-baseline leg of the benchmark may call it.

Pinning: the reference ships no tests and no golden vectors.  The oracle is
pinned against outputs of the reference itself, produced by importing the
reference's pure-python path and its CompiledLogicNet C build on a CPU and
committed as small fixtures (tests/golden/*.npz, made by
tests/golden/make_golden.py).  The bit layout of the packed words produced by
`pack_bits` is pinned only indirectly (packed pipeline == CompiledLogicNet
counts); the word layout itself follows a reading of the reference kernel.

Each function cites the reference file:line it follows (paths are relative to
the reference project root).
"""
from __future__ import annotations

import math

import numpy as np
import torch

# ---------------------------------------------------------------------------------------------
# Gate table.  Gate id i has truth-table bits  i = 8*f(0,0) + 4*f(0,1) + 2*f(1,0) + f(1,1)
# (difflogic/functional.py:7-24, difflogic/cuda/difflogic_kernel.cu:418-435).
# ---------------------------------------------------------------------------------------------

NUM_GATES = 16


def truth_table() -> np.ndarray:
    """[16,4] array of f(0,0), f(0,1), f(1,0), f(1,1) per gate id."""
    t = np.zeros((16, 4), dtype=np.int64)
    for i in range(16):
        t[i] = [(i >> 3) & 1, (i >> 2) & 1, (i >> 1) & 1, i & 1]
    return t


def gate_real(a: torch.Tensor, b: torch.Tensor, i: int) -> torch.Tensor:
    """Real-valued relaxation of gate i (difflogic/functional.py:26-62).

    The products are written out term by term, as the reference does, so that autograd
    accumulates in the same order and the fixtures are reproduced to the last bit."""
    forms = (
        lambda: torch.zeros_like(a),
        lambda: a * b,
        lambda: a - a * b,
        lambda: a,
        lambda: b - a * b,
        lambda: b,
        lambda: a + b - 2 * a * b,
        lambda: a + b - a * b,
        lambda: 1 - (a + b - a * b),
        lambda: 1 - (a + b - 2 * a * b),
        lambda: 1 - b,
        lambda: 1 - b + a * b,
        lambda: 1 - a,
        lambda: 1 - a + a * b,
        lambda: 1 - a * b,
        lambda: torch.ones_like(a),
    )
    return forms[i]()


def mix_gates(a: torch.Tensor, b: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Sum over the 16 gates of w[..., i] * gate_i(a, b), accumulated in gate order
    (difflogic/functional.py:65-70)."""
    r = torch.zeros_like(a)
    for i in range(16):
        r = r + w[..., i] * gate_real(a, b, i)
    return r


def layer_forward(x, idx_a, idx_b, weights, training: bool):
    """One logic layer on batch-major x [B, n_in] (difflogic/difflogic.py:94-108).

    training: softmax mixing of all gates; eval: the arg-max gate only (first max on ties)."""
    a, b = x[..., idx_a], x[..., idx_b]
    if training:
        w = torch.nn.functional.softmax(weights, dim=-1)
    else:
        w = torch.nn.functional.one_hot(weights.argmax(-1), 16).to(x.dtype)
    return mix_gates(a, b, w)


class _GradScale(torch.autograd.Function):
    """Identity whose gradient is scaled by f (difflogic/functional.py:130-138)."""

    @staticmethod
    def forward(ctx, x, f):
        ctx.f = f
        return x

    @staticmethod
    def backward(ctx, g):
        return g * ctx.f, None


def group_sum(x, k: int, tau: float):
    """Float GroupSum on batch-major x [..., n] (difflogic/difflogic.py:195-196)."""
    assert x.shape[-1] % k == 0
    return x.reshape(*x.shape[:-1], k, x.shape[-1] // k).sum(-1) / tau


def random_connections(in_dim: int, out_dim: int):
    """'random' connectivity, same CPU-RNG draw order as difflogic/difflogic.py:158-165."""
    c = torch.randperm(2 * out_dim) % in_dim
    c = torch.randperm(in_dim)[c]
    c = c.reshape(2, out_dim)
    return c[0].to(torch.int64), c[1].to(torch.int64)


class OracleNet:
    """Flatten -> L logic layers -> GroupSum, CPU, fp32 or fp64.

    build() draws from the global CPU generator in the same order as constructing the
    reference's Sequential of LogicLayer(device='cpu') objects does: for each layer first
    randn(out,16) (difflogic/difflogic.py:33) and then the two randperm calls of the 'random'
    connections (difflogic/difflogic.py:159-160)."""

    def __init__(self, weights, idx_a, idx_b, k, tau, grad_factor_=1.0):
        self.weights = [w.clone().requires_grad_(True) for w in weights]
        self.idx_a = idx_a
        self.idx_b = idx_b
        self.k = k
        self.tau = tau
        self.grad_factor = grad_factor_

    @staticmethod
    def build(dims, k, tau, grad_factor_=1.0):
        ws, aa, bb = [], [], []
        for n_in, n_out in zip(dims[:-1], dims[1:]):
            ws.append(torch.randn(n_out, 16))
            a, b = random_connections(n_in, n_out)
            aa.append(a)
            bb.append(b)
        return OracleNet(ws, aa, bb, k, tau, grad_factor_)

    def double(self):
        return OracleNet([w.detach().double() for w in self.weights], self.idx_a, self.idx_b,
                         self.k, self.tau, self.grad_factor)

    def activations(self, x, training: bool):
        """List of per-layer outputs (batch-major)."""
        outs = []
        h = x.reshape(x.shape[0], -1)
        for w, a, b in zip(self.weights, self.idx_a, self.idx_b):
            if self.grad_factor != 1.0:
                h = _GradScale.apply(h, self.grad_factor)
            h = layer_forward(h, a, b, w, training)
            outs.append(h)
        return outs

    def forward(self, x, training: bool):
        return group_sum(self.activations(x, training)[-1], self.k, self.tau)

    def train_step(self, x, y, lr=0.01):
        """forward + CrossEntropyLoss + backward + one Adam step (experiments/main.py:174-181).
        Returns (loss, logits, [grad per layer]); the weights are updated in place."""
        opt = torch.optim.Adam(self.weights, lr=lr)
        logits = self.forward(x, training=True)
        loss = torch.nn.functional.cross_entropy(logits, y)
        opt.zero_grad()
        loss.backward()
        grads = [w.grad.detach().clone() for w in self.weights]
        opt.step()
        return loss.detach(), logits.detach(), grads

    def gate_ids(self):
        """Arg-max gate per neuron (difflogic/difflogic.py:146, compiled_model.py:77)."""
        return [w.detach().argmax(-1).to(torch.uint8) for w in self.weights]


# ---------------------------------------------------------------------------------------------
# Closed-form backward (float64-capable), used to check backward_w / backward_x kernels one
# layer at a time.  Feature-major layout like the kernels: x [n_in, B], grad_y [n_out, B].
# ---------------------------------------------------------------------------------------------

def layer_backward_closed_form(x_fm, idx_a, idx_b, w_mix, grad_y_fm):
    """Gradients of y[j,:] = sum_i w_mix[j,i] gate_i(x[a_j,:], x[b_j,:]).

    Returns (grad_w_mix [n_out,16], grad_x [n_in,B]).  grad_w follows the four batch sums of
    difflogic_kernel.cu:157-176 and the 16 combinations of :343-360; grad_x is the true
    derivative (d/da + d/db, also when a_j == b_j), which is what autograd of the python path
    gives (difflogic.py:102-104)."""
    a = x_fm[idx_a]
    b = x_fm[idx_b]
    g = grad_y_fm
    tt = torch.tensor(truth_table(), dtype=x_fm.dtype)
    # per-gate multilinear coefficients [16,4]: const, a, b, ab
    coef = torch.stack([tt[:, 0], tt[:, 2] - tt[:, 0], tt[:, 1] - tt[:, 0],
                        tt[:, 0] - tt[:, 1] - tt[:, 2] + tt[:, 3]], dim=1)
    s = torch.stack([g.sum(1), (a * g).sum(1), (b * g).sum(1), (a * b * g).sum(1)], dim=1)
    grad_w = s @ coef.T
    c = w_mix @ coef  # [n_out,4]
    da = (c[:, 1:2] + c[:, 3:4] * b) * g
    db = (c[:, 2:3] + c[:, 3:4] * a) * g
    grad_x = torch.zeros_like(x_fm)
    grad_x.index_add_(0, idx_a, da)
    grad_x.index_add_(0, idx_b, db)
    return grad_w, grad_x


def softmax_backward(w_raw, grad_p):
    p = torch.softmax(w_raw, dim=-1)
    return p * (grad_p - (p * grad_p).sum(-1, keepdim=True))


# ---------------------------------------------------------------------------------------------
# Packed-bit path (integer, bit-exact).  numpy.
# ---------------------------------------------------------------------------------------------

BITS_TO_NP = {8: np.int8, 16: np.int16, 32: np.int32, 64: np.int64}
BITS_TO_NPU = {8: np.uint8, 16: np.uint16, 32: np.uint32, 64: np.uint64}


def pack_bits(t_fm: np.ndarray, bits: int):
    """bool [n, B] (feature-major) -> (signed words [n, ceil(B/bits)], pad_len).

    Sample s lands in word s // bits at bit s % bits, least-significant bit first; pad bits are
    zero (difflogic_kernel.cu:547-625, pad_len at :592)."""
    n, B = t_fm.shape
    W = -(-B // bits)
    pad = (bits - B % bits) % bits
    padded = np.zeros((n, W * bits), dtype=np.uint64)
    padded[:, :B] = (t_fm != 0)
    padded = padded.reshape(n, W, bits)
    shifts = np.arange(bits, dtype=np.uint64)
    words = (padded << shifts).sum(-1, dtype=np.uint64) if bits < 64 else np.bitwise_or.reduce(padded << shifts, axis=-1)
    return words.astype(BITS_TO_NPU[bits]).view(BITS_TO_NP[bits]), pad


def gate_bitwise(a: np.ndarray, b: np.ndarray, op: np.ndarray) -> np.ndarray:
    """Bitwise form of the 16 gates on packed words (difflogic_kernel.cu:437-472);
    op broadcasts against a and b."""
    op = np.asarray(op)
    ones = ~np.zeros_like(a)
    zeros = np.zeros_like(a)
    table = [zeros, a & b, a & ~b, a, b & ~a, b, a ^ b, a | b, ~(a | b), ~(a ^ b), ~b, ~b | a, ~a, ~a | b,
             ~(a & b), ones]
    out = np.zeros_like(a)
    for i in range(16):
        out = np.where(op == i, table[i], out)
    return out


def eval_packed(x_words: np.ndarray, idx_a, idx_b, gate_ids) -> np.ndarray:
    """Packed eval of one layer: words [n_in, W] -> [n_out, W] (difflogic_kernel.cu:474-541)."""
    idx_a = np.asarray(idx_a)
    idx_b = np.asarray(idx_b)
    op = np.asarray(gate_ids).astype(np.int64)[:, None]
    return gate_bitwise(x_words[idx_a], x_words[idx_b], op)


def group_bit_sum(words: np.ndarray, pad_len: int, k: int) -> np.ndarray:
    """words [n, W] -> int32 [B, k] with B = W*bits - pad_len: per class the number of set bits
    of each sample over the class's n/k rows (difflogic_kernel.cu:631-700; divisibility check at
    difflogic/cuda/difflogic.cpp:77-80)."""
    n, W = words.shape
    if n % k != 0:
        raise ValueError("in_dim (%d) has to be divisible by k (%d) but it is not" % (n, k))
    bits = words.dtype.itemsize * 8
    u = words.view(BITS_TO_NPU[bits])
    B = W * bits - pad_len
    # unpack LSB-first: byte view is little-endian, so bit order within the row is sample order
    by = u.view(np.uint8).reshape(n, W * bits // 8)
    bit = np.unpackbits(by, axis=1, bitorder="little")[:, :B]  # [n, B]
    return bit.reshape(k, n // k, B).sum(1, dtype=np.int64).T.astype(np.int32).copy()


def packed_net_counts(x_bool_bm: np.ndarray, idx_a, idx_b, gate_ids, k: int, bits: int = 64) -> np.ndarray:
    """bool [B, n_in] -> class counts [B, k]: pack, eval every layer, group bit-sum
    (the chain of experiments/main.py:198-210; same result as compiled_model.py:159-239)."""
    words, pad = pack_bits(np.ascontiguousarray(x_bool_bm.T), bits)
    for a, b, g in zip(idx_a, idx_b, gate_ids):
        words = eval_packed(words, np.asarray(a), np.asarray(b), np.asarray(g))
    return group_bit_sum(words, pad, k)


def csr_of_connections(idx_a, idx_b, n_in: int):
    """Inverse connection index of difflogic/difflogic.py:56-69: for each input the list of
    consumer neurons in increasing order (a neuron with a==b appears twice), and the offsets."""
    idx_a = np.asarray(idx_a)
    idx_b = np.asarray(idx_b)
    lists = [[] for _ in range(n_in)]
    for y in range(len(idx_a)):
        lists[idx_a[y]].append(y)
        lists[idx_b[y]].append(y)
    start = np.array([0] + [len(l) for l in lists]).cumsum().astype(np.int64)
    flat = np.array([v for l in lists for v in l], dtype=np.int64)
    return start, flat


# ---------------------------------------------------------------------------------------------
# C restatement of the whole packed net (oracle/bitnet_oracle.c), used for larger batches and as
# the timed CPU baseline.
# ---------------------------------------------------------------------------------------------

_c_lib = None


def c_oracle():
    """Loads oracle/_ref/libbitnet_oracle.so, building it with gcc when it is missing."""
    global _c_lib
    if _c_lib is None:
        import ctypes
        from oracle import build_oracle
        lib = ctypes.CDLL(build_oracle.build())
        p, i64 = ctypes.c_void_p, ctypes.c_int64
        lib.oracle_apply_net.restype = None
        lib.oracle_apply_net.argtypes = [p, p, i64, i64, ctypes.c_int, p, p, p, p, i64, ctypes.c_int]
        lib.oracle_eval_layer.restype = None
        lib.oracle_eval_layer.argtypes = [p, p, p, p, p, i64, i64]
        _c_lib = lib
    return _c_lib


def c_packed_net_counts(x_bool_bm: np.ndarray, idx_a, idx_b, gate_ids, k: int, threads: int = 1) -> np.ndarray:
    """bool [B, n_in] -> int32 [B, k], 64 samples per block like CompiledLogicNet(num_bits=64)
    (compiled_model.py:342-370 for the padding, :159-239 for the per-block work)."""
    B, n_in = x_bool_bm.shape
    blocks = -(-B // 64)
    padded = np.zeros((blocks * 64, n_in), dtype=np.uint8)
    padded[:B] = x_bool_bm != 0
    widths = np.array([len(a) for a in idx_a], dtype=np.int64)
    a = np.ascontiguousarray(np.concatenate([np.asarray(v, dtype=np.int64) for v in idx_a]))
    b = np.ascontiguousarray(np.concatenate([np.asarray(v, dtype=np.int64) for v in idx_b]))
    op = np.ascontiguousarray(np.concatenate([np.asarray(v, dtype=np.uint8) for v in gate_ids]))
    out = np.zeros((blocks * 64, k), dtype=np.int32)
    c_oracle().oracle_apply_net(padded.ctypes.data, out.ctypes.data, blocks, n_in, len(widths), widths.ctypes.data,
                                a.ctypes.data, b.ctypes.data, op.ctypes.data, k, threads)
    return out[:B]
