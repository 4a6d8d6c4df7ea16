"""Pins the CPU oracle against fixtures produced by the reference implementation itself
(tests/golden/make_golden.py).  No GPU needed."""
import os

import numpy as np
import pytest
import torch

from oracle import logic_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_gate_table_matches_reference(golden_dir):
    g = _load(golden_dir, "gates.npz")
    a, b, w = (torch.tensor(g[k]) for k in ("a", "b", "w"))
    for i in range(16):
        assert torch.equal(O.gate_real(a, b, i), torch.tensor(g["gates"][i])), i
    assert torch.equal(O.mix_gates(a, b, w), torch.tensor(g["mix"]))
    # truth table agrees with the relaxations at the corners
    tt = O.truth_table()
    for i in range(16):
        for q, (av, bv) in enumerate(((0., 0.), (0., 1.), (1., 0.), (1., 1.))):
            assert O.gate_real(torch.tensor([av]), torch.tensor([bv]), i).item() == tt[i, q]


def _net_from_fixture(g):
    dims = [int(v) for v in g["dims"]]
    L = len(dims) - 1
    ws = [torch.tensor(g["w0_%d" % i]) for i in range(L)]
    aa = [torch.tensor(g["a_%d" % i]) for i in range(L)]
    bb = [torch.tensor(g["b_%d" % i]) for i in range(L)]
    return O.OracleNet(ws, aa, bb, int(g["k"]), float(g["tau"]), float(g["grad_factor"])), L


@pytest.mark.parametrize("name", ["small_net.npz", "small_net_gf2.npz"])
def test_small_net_train_step_matches_reference(golden_dir, name):
    g = _load(golden_dir, name)
    net, L = _net_from_fixture(g)
    x = torch.tensor(g["x"])
    y = torch.tensor(g["y"])
    # regenerating from the seed gives the very same weights and connections
    torch.manual_seed(int(g["seed"]))
    regen = O.OracleNet.build([int(v) for v in g["dims"]], int(g["k"]), float(g["tau"]))
    for i in range(L):
        assert torch.equal(regen.weights[i].detach(), net.weights[i].detach())
        assert torch.equal(regen.idx_a[i], net.idx_a[i]) and torch.equal(regen.idx_b[i], net.idx_b[i])

    eval_logits = net.forward(x, training=False).detach()
    assert torch.equal(eval_logits, torch.tensor(g["eval_logits"]))

    xr = x.clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(net.forward(xr, True), y).backward()
    assert torch.equal(xr.grad, torch.tensor(g["grad_x"]))
    for w in net.weights:
        w.grad = None

    loss, logits, grads = net.train_step(x, y)
    assert torch.equal(logits, torch.tensor(g["train_logits"]))
    assert loss.item() == pytest.approx(float(g["loss"]), rel=0, abs=0)
    for i in range(L):
        assert torch.equal(grads[i], torch.tensor(g["grad_%d" % i])), i
        assert torch.equal(net.weights[i].detach(), torch.tensor(g["w1_%d" % i])), i
    assert torch.equal(net.forward(x, False).detach(), torch.tensor(g["eval_logits_after_step"]))


@pytest.mark.parametrize("name", ["small_net.npz", "small_net_gf2.npz"])
@pytest.mark.parametrize("bits", [8, 16, 32, 64])
def test_packed_pipeline_matches_compiled_logic_net(golden_dir, name, bits):
    g = _load(golden_dir, name)
    net, L = _net_from_fixture(g)
    counts = O.packed_net_counts(g["x"].astype(bool), net.idx_a, net.idx_b, net.gate_ids(), int(g["k"]), bits)
    assert counts.dtype == np.int32
    assert np.array_equal(counts, g["compiled_counts_%d" % bits])
    # and with the float eval path times tau (GroupSum on packed input does not divide by tau)
    assert np.array_equal(counts, np.rint(g["eval_logits"] * float(g["tau"])).astype(np.int32))


def test_closed_form_backward_matches_autograd(golden_dir):
    g = _load(golden_dir, "small_net.npz")
    net, L = _net_from_fixture(g)
    net = net.double()
    torch.manual_seed(5)
    x = torch.rand(37, 20, dtype=torch.float64, requires_grad=True)
    w = net.weights[0]
    y = O.layer_forward(x, net.idx_a[0], net.idx_b[0], w, True)
    gy = torch.randn_like(y)
    y.backward(gy)
    p = torch.softmax(w.detach(), -1)
    gw_mix, gx = O.layer_backward_closed_form(x.detach().T.contiguous(), net.idx_a[0], net.idx_b[0], p,
                                              gy.T.contiguous())
    assert torch.allclose(gx.T, x.grad, rtol=1e-12, atol=1e-14)
    assert torch.allclose(O.softmax_backward(w.detach(), gw_mix), w.grad, rtol=1e-11, atol=1e-13)


def test_config1_matches_reference(golden_dir):
    """Config 1 (784 -> 4 x 8000 -> GroupSum(10, tau=10), batch 100), regenerated from seed 0."""
    g = _load(golden_dir, "config1.npz")
    torch.manual_seed(0)
    net = O.OracleNet.build([784, 8000, 8000, 8000, 8000], 10, 10.0)
    x = (torch.rand(100, 784) < 0.19).float()
    y = torch.randint(0, 10, (100,))
    assert np.array_equal(y.numpy(), g["y"]) and np.array_equal(x.sum(1).numpy(), g["x_rowsum"])
    for i in range(4):
        ar = torch.arange(8000)
        assert [(net.idx_a[i] * ar).sum().item(), (net.idx_b[i] * ar).sum().item()] == list(g["idx_check_%d" % i])
    eval_logits = net.forward(x, False).detach().numpy()
    assert np.array_equal(eval_logits, g["eval_logits"])
    counts = O.packed_net_counts(x.bool().numpy(), net.idx_a, net.idx_b, net.gate_ids(), 10, 64)
    assert np.array_equal(counts, g["compiled_counts_64"])
    assert np.array_equal(counts, np.rint(g["eval_logits"] * 10.0).astype(np.int32))
    loss, logits, grads = net.train_step(x, y)
    assert np.array_equal(logits.numpy(), g["train_logits"])
    assert loss.item() == float(g["loss"])
    for i in range(4):
        pos = torch.tensor(g["pos_%d" % i])
        assert np.array_equal(grads[i].reshape(-1)[pos].numpy(), g["grad_sample_%d" % i])
        assert grads[i].abs().max().item() == float(g["grad_absmax_%d" % i])
        assert np.array_equal(net.weights[i].detach().reshape(-1)[pos].numpy(), g["w1_sample_%d" % i])


def test_csr_of_connections_lists_each_neuron_twice():
    a = np.array([0, 2, 2, 1])
    b = np.array([1, 2, 0, 1])
    start, flat = O.csr_of_connections(a, b, 3)
    assert list(start) == [0, 2, 5, 8]
    assert list(flat) == [0, 2, 0, 3, 3, 1, 1, 2]


@pytest.mark.parametrize("name", ["small_net.npz", "small_net_gf2.npz"])
def test_c_oracle_matches_compiled_logic_net(golden_dir, name):
    g = _load(golden_dir, name)
    net, L = _net_from_fixture(g)
    for threads in (1, 3):
        counts = O.c_packed_net_counts(g["x"].astype(bool), net.idx_a, net.idx_b, net.gate_ids(), int(g["k"]), threads)
        assert np.array_equal(counts, g["compiled_counts_64"])


def test_c_oracle_matches_numpy_oracle_on_ragged_batch():
    torch.manual_seed(8)
    net = O.OracleNet.build([30, 64, 50], 5, 1.0)
    x = torch.rand(200, 30) < 0.5
    ref = O.packed_net_counts(x.numpy(), net.idx_a, net.idx_b, net.gate_ids(), 5, 64)
    assert np.array_equal(O.c_packed_net_counts(x.numpy(), net.idx_a, net.idx_b, net.gate_ids(), 5, 2), ref)
