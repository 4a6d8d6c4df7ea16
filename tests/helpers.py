"""Shared helpers of the parity tests: model construction from oracle weights, tolerances."""
import numpy as np
import torch

import difflogic_b200 as D
from oracle import logic_oracle as O

# Tolerances named by the build target: forward activations 1e-5 relative, gradients 1e-4 relative
# (per tensor, relative to the largest reference entry: element-wise relative error is meaningless
# for the near-zero entries that softmax-backward cancellation produces).
FWD_RTOL = 1e-5
GRAD_RTOL = 1e-4


def assert_forward_close(got, ref, what=""):
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    # element-wise relative with an absolute floor of FWD_RTOL * max|ref| * 1e-1 for entries near zero
    scale = ref.abs().max().item() if ref.numel() else 1.0
    err = (got - ref).abs()
    bound = FWD_RTOL * ref.abs() + FWD_RTOL * 0.1 * scale
    assert bool((err <= bound).all()), "%s: max err %.3e (scale %.3e)" % (what, err.max().item(), scale)


def assert_grad_close(got, ref, what="", rtol=GRAD_RTOL):
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    scale = ref.abs().max().item() if ref.numel() else 1.0
    err = (got - ref).abs().max().item() if ref.numel() else 0.0
    assert err <= rtol * scale + 1e-30, "%s: max|diff| %.3e > %.1e * max|ref| %.3e" % (what, err, rtol, scale)


def build_model(dims, k, tau, weights, idx_a, idx_b, device="cuda", grad_factor=1.0, implementation=None):
    layers = [torch.nn.Flatten()]
    for i, (n_in, n_out) in enumerate(zip(dims[:-1], dims[1:])):
        layer = D.LogicLayer(n_in, n_out, device=device, grad_factor=grad_factor, implementation=implementation)
        with torch.no_grad():
            layer.weights.copy_(weights[i].detach().to(torch.float32))
        layer.set_connections(idx_a[i], idx_b[i])
        layers.append(layer)
    layers.append(D.GroupSum(k, tau, device=device))
    return torch.nn.Sequential(*layers)


def logic_layers(model):
    return [m for m in model if isinstance(m, D.LogicLayer)]


def random_layer(n_in, n_out, seed, force_same_input=False):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(0, n_in, (n_out,), generator=g)
    b = torch.randint(0, n_in, (n_out,), generator=g)
    if force_same_input and n_out >= 3:
        b[1] = a[1]           # a neuron wired twice to the same input
        b[n_out - 1] = a[n_out - 1]
    w = torch.randn(n_out, 16, generator=g)
    return a, b, w
