"""Stand-in for the reference's native module `difflogic_cuda` (difflogic/cuda/difflogic.cpp:45-84).

The six functions keep the reference's names, argument order, layouts and return values, but run
on the sm_100a kernels.  Registering this module as `difflogic_cuda` (see `install()`) lets the
reference's own Python files run unchanged on the new kernels:

    import difflogic_b200.difflogic_cuda as shim; shim.install()
    import difflogic            # the reference package, if it is on sys.path

Unlike the reference's functions these launch on torch's current stream and do not synchronise.
"""
import sys

import torch

from . import ops


def forward(x, a, b, w):
    """x [in, batch], w [out, 16] mixing weights (already soft-maxed) -> y [out, batch]."""
    return ops.logic_forward(x, a, b, w, ops.W_PROBS)[0]


def backward_w(x, a, b, grad_y):
    """Gradient w.r.t. the mixing weights, [out, 16]."""
    return ops.logic_backward_w(x, a, b, grad_y, None, ops.W_PROBS)


def backward_x(x, a, b, w, grad_y, given_x_indices_of_y_start, given_x_indices_of_y):
    """Gradient w.r.t. x.  A neuron whose two inputs are the same row contributes d/da + d/db, as the
    reference's python path does (its CUDA kernel adds 2 * d/da for such a neuron)."""
    plan = ops.build_backward_plan(a, b, given_x_indices_of_y_start, given_x_indices_of_y)
    return ops.logic_backward_x(x, ops.logic_coefs(w, ops.W_PROBS), grad_y, given_x_indices_of_y_start, plan, 1.0)


def eval(x, a, b, w):  # noqa: A001 - the reference's name
    """Packed words x [in, words], w uint8 gate ids [out] -> [out, words]."""
    return ops.eval_packed(x, a, b, w)


def tensor_packbits_cuda(t, bit_count):
    """bool [n, batch] -> (int{bit_count} [n, ceil(batch/bit_count)], pad_len)."""
    return ops.packbits(t, bit_count)


def groupbitsum(b, pad_len, k):
    """Packed [n, words] -> int32 [batch, k]; ValueError when n is not divisible by k."""
    return ops.groupbitsum(b, pad_len, k)


def install(name="difflogic_cuda"):
    """Makes `import difflogic_cuda` resolve to this module."""
    sys.modules[name] = sys.modules[__name__]
    return sys.modules[name]
