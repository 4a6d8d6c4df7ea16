"""Gate algebra and connection helpers of the Python API (pure torch, device-agnostic).

Drop-in for the reference module difflogic/functional.py: `bin_op`, `bin_op_s`,
`get_unique_connections`, `GradFactor`, `BITS_TO_NP_DTYPE`.  The CUDA kernels do not call into
this file; it is the `implementation='python'` path and the definition the kernels are tested
against.

Gate id i has the truth table  i = 8 f(0,0) + 4 f(0,1) + 2 f(1,0) + f(1,1):
0 false, 1 and, 2 a&~b, 3 a, 4 ~a&b, 5 b, 6 xor, 7 or, 8 nor, 9 xnor, 10 ~b, 11 a|~b, 12 ~a,
13 ~a|b, 14 nand, 15 true.
"""
import numpy as np
import torch

BITS_TO_NP_DTYPE = {8: np.int8, 16: np.int16, 32: np.int32, 64: np.int64}

# Real-valued relaxations (probabilistic interpretation: A, B independent), one per gate id.
# The arithmetic forms are those of the reference (functional.py:31-62) so that the python
# path gives the same floating-point results.
_RELAXED_GATES = (
    lambda a, b: torch.zeros_like(a),
    lambda a, b: a * b,
    lambda a, b: a - a * b,
    lambda a, b: a,
    lambda a, b: b - a * b,
    lambda a, b: b,
    lambda a, b: a + b - 2 * a * b,
    lambda a, b: a + b - a * b,
    lambda a, b: 1 - (a + b - a * b),
    lambda a, b: 1 - (a + b - 2 * a * b),
    lambda a, b: 1 - b,
    lambda a, b: 1 - b + a * b,
    lambda a, b: 1 - a,
    lambda a, b: 1 - a + a * b,
    lambda a, b: 1 - a * b,
    lambda a, b: torch.ones_like(a),
)


def bin_op(a, b, i):
    """Relaxed gate number `i` applied element-wise to a and b (same shapes)."""
    assert a[0].shape == b[0].shape, (a[0].shape, b[0].shape)
    if a.shape[0] > 1:
        assert a[1].shape == b[1].shape, (a[1].shape, b[1].shape)
    if not 0 <= i < 16:
        return None
    return _RELAXED_GATES[i](a, b)


def bin_op_s(a, b, i_s):
    """Mix of all 16 gates: sum_i i_s[..., i] * bin_op(a, b, i), accumulated in gate order."""
    total = torch.zeros_like(a)
    for gate in range(16):
        total = total + i_s[..., gate] * bin_op(a, b, gate)
    return total


def get_unique_connections(in_dim, out_dim, device='cuda'):
    """Connections in which no (a, b) pair repeats.

    Pairs are enumerated as (0,1),(2,3),...; then (1,2),(3,4),...; then (i, i+d) for d = 2, 3, ...
    until out_dim pairs exist; the first out_dim are kept and shuffled with one randperm(out_dim)
    drawn from the CPU generator.  Same enumeration and RNG use as the reference
    (functional.py:76-124), so equal seeds give equal connections."""
    assert out_dim * 2 >= in_dim, 'The number of neurons ({}) must not be smaller than half of the number of inputs ' \
                                  '({}) because otherwise not all inputs could be used or considered.'.format(
        out_dim, in_dim)

    def pairs_from(first, step, gap):
        lo = torch.arange(first, in_dim - gap, step, dtype=torch.int64)
        return lo, lo + gap

    a, b = pairs_from(0, 2, 1)
    if a.numel() < out_dim:
        a2, b2 = pairs_from(1, 2, 1)
        a, b = torch.cat([a, a2]), torch.cat([b, b2])
    gap = 2
    while out_dim > a.numel() > gap:
        a2, b2 = pairs_from(0, 1, gap)
        a, b = torch.cat([a, a2]), torch.cat([b, b2])
        gap += 1
    assert a.numel() >= out_dim, (a.numel(), gap, out_dim)
    a, b = a[:out_dim], b[:out_dim]

    perm = torch.randperm(out_dim)
    a, b = a[perm].to(device).contiguous(), b[perm].to(device).contiguous()
    return a, b


class GradFactor(torch.autograd.Function):
    """Identity in the forward pass; multiplies the incoming gradient by `f` in the backward pass."""

    @staticmethod
    def forward(ctx, x, f):
        ctx.f = f
        return x

    @staticmethod
    def backward(ctx, grad_y):
        return grad_y * ctx.f, None
