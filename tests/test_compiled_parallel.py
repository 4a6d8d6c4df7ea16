"""CompiledLogicNet built from several translation units in parallel gives the same library behaviour."""
import os

import numpy as np
import torch

import difflogic_b200 as D
from difflogic_b200 import compiled_model


def test_parallel_translation_units_match_single_unit(golden_dir, monkeypatch):
    g = np.load(os.path.join(golden_dir, "small_net_gf2.npz"))
    dims = [int(v) for v in g["dims"]]
    layers = [torch.nn.Flatten()]
    for i, (n_in, n_out) in enumerate(zip(dims[:-1], dims[1:])):
        layer = D.LogicLayer(n_in, n_out, device='cpu')
        with torch.no_grad():
            layer.weights.copy_(torch.tensor(g["w0_%d" % i]))
        layer.set_connections(torch.tensor(g["a_%d" % i]), torch.tensor(g["b_%d" % i]))
        layers.append(layer)
    model = torch.nn.Sequential(*layers, D.GroupSum(int(g["k"]), float(g["tau"]), device='cpu'))
    monkeypatch.setattr(compiled_model, "_STATEMENTS_PER_FUNCTION", 16)  # many small functions -> several units
    net = D.CompiledLogicNet(model, num_bits=64)
    assert len(net._c_sources(4)) == 4 and len(net._c_sources(1)) == 1
    net.compile(opt_level=0, jobs=4)
    x = g["x"].astype(bool)
    assert np.array_equal(net.forward(x).numpy(), g["compiled_counts_64"])
    single = D.CompiledLogicNet(model, num_bits=64)
    single.compile(opt_level=0, jobs=1)
    assert np.array_equal(single.forward(x).numpy(), g["compiled_counts_64"])
