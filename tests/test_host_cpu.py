"""Host-side checks that need no GPU: the C ABI library loads and exports every declared symbol,
argument errors are reported before any launch, and the pure-python / compiled CPU paths of the
API reproduce the reference fixtures."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import difflogic_b200 as D
from difflogic_b200 import _native, build as dl_build
from tests.helpers import build_model, logic_layers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    dl_build.build()
    return _native.lib()


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "difflogic_b200.h")).read()
    declared = set(re.findall(r"DL_API[^;(]*?\b(dl_\w+)\s*\(", header))
    assert len(declared) >= 15
    assert declared == set(_native.SIGNATURES), declared ^ set(_native.SIGNATURES)
    raw = ctypes.CDLL(_native.library_path())
    for name in declared:
        assert hasattr(raw, name), name
    assert lib.dl_version() >= 100


def test_argument_errors_are_reported_before_any_launch(lib):
    null = None
    assert lib.dl_eval_packed(null, null, null, null, null, 4, 4, 4, 12, null) == _native.DL_ERR_BAD_BIT_COUNT
    assert b"bit_count" in lib.dl_last_error_string()
    with pytest.raises(ValueError):
        _native.check(lib.dl_packbits(null, null, 4, 4, 7, null))
    assert lib.dl_groupbitsum(null, null, 10, 4, 0, 3, 64, null) == _native.DL_ERR_NOT_DIVISIBLE
    with pytest.raises(ValueError, match="divisible"):
        _native.check(lib.dl_groupbitsum(null, null, 10, 4, 0, 3, 64, null))
    assert lib.dl_forward_f32(null, null, null, null, 0, null, null, 4, 4, 4, 0, null) == _native.DL_ERR_INVALID_ARG
    assert lib.dl_forward_f32(null, null, null, null, 9, null, null, 4, 4, 4, 0, null) == _native.DL_ERR_INVALID_ARG
    assert lib.dl_forward_f32(null, null, null, null, 0, null, null, -1, 4, 4, 0, null) == _native.DL_ERR_INVALID_ARG
    with pytest.raises(RuntimeError):
        _native.check(lib.dl_backward_x_f32(null, null, null, null, null, 1.0, null, 4, 4, 4, 0, null))
    assert lib.dl_backward_x_f32(null, null, null, null, null, 1.0, null, 4, 1 << 31, 4, 0, null) == _native.DL_ERR_TOO_LARGE
    assert lib.dl_groupsum_f32(null, null, null, 10, 4, 3, 1.0, null) == _native.DL_ERR_NOT_DIVISIBLE
    # empty problems are fine and launch nothing
    assert lib.dl_forward_f32(null, null, null, null, 0, null, null, 4, 0, 4, 0, null) == _native.DL_OK
    assert lib.dl_eval_packed(null, null, null, null, null, 4, 4, 0, 64, null) == _native.DL_OK
    assert lib.dl_groupsum_workspace_bytes(16000, 128, 10) > 4096


def test_cuda_path_has_no_cpu_stand_in():
    layer = D.LogicLayer(8, 8, device='cpu', implementation='cuda')
    with pytest.raises((RuntimeError, AssertionError)):
        layer(torch.rand(3, 8))
    from difflogic_b200 import ops
    with pytest.raises(RuntimeError):
        ops.logic_forward(torch.rand(8, 3), torch.zeros(4, dtype=torch.int64), torch.zeros(4, dtype=torch.int64),
                          torch.rand(4, 16))


def _fixture_model(golden_dir, name):
    g = np.load(os.path.join(golden_dir, name))
    dims = [int(v) for v in g["dims"]]
    L = len(dims) - 1
    model = build_model(dims, int(g["k"]), float(g["tau"]), [torch.tensor(g["w0_%d" % i]) for i in range(L)],
                        [torch.tensor(g["a_%d" % i]) for i in range(L)], [torch.tensor(g["b_%d" % i]) for i in range(L)],
                        device='cpu', grad_factor=float(g["grad_factor"]))
    return g, model


@pytest.mark.parametrize("name", ["small_net.npz", "small_net_gf2.npz"])
def test_python_implementation_reproduces_reference(golden_dir, name):
    g, model = _fixture_model(golden_dir, name)
    assert all(l.implementation == 'python' for l in logic_layers(model))
    x, y = torch.tensor(g["x"]), torch.tensor(g["y"])
    model.train()
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    logits = model(x)
    loss = torch.nn.functional.cross_entropy(logits, y)
    opt.zero_grad()
    loss.backward()
    assert torch.equal(logits.detach(), torch.tensor(g["train_logits"]))
    for i, l in enumerate(logic_layers(model)):
        assert torch.equal(l.weights.grad, torch.tensor(g["grad_%d" % i]))
    opt.step()
    for i, l in enumerate(logic_layers(model)):
        assert torch.equal(l.weights.detach(), torch.tensor(g["w1_%d" % i]))


@pytest.mark.parametrize("bits", [8, 16, 32, 64])
def test_compiled_logic_net_reproduces_reference(golden_dir, bits, tmp_path):
    g, model = _fixture_model(golden_dir, "small_net.npz")
    net = D.CompiledLogicNet(model, num_bits=bits)
    assert "apply_logic_gate_net" in net.get_c_code()
    path = str(tmp_path / "net.so")
    net.compile(opt_level=0, save_lib_path=path)
    x = g["x"].astype(bool)
    out = net.forward(x)
    assert out.dtype == torch.int32 and np.array_equal(out.numpy(), g["compiled_counts_%d" % bits])
    assert np.array_equal(net(torch.tensor(x)).numpy(), g["compiled_counts_%d" % bits])
    # a batch smaller than one word is padded correctly
    assert np.array_equal(net.forward(x[:3]).numpy(), g["compiled_counts_%d" % bits][:3])
    loaded = D.CompiledLogicNet.load(path, int(g["k"]), bits)
    assert np.array_equal(loaded.forward(x).numpy(), g["compiled_counts_%d" % bits])


def test_unique_connections_reproduce_reference(golden_dir):
    u = np.load(os.path.join(golden_dir, "unique_connections.npz"))
    j = 0
    while "a_%d" % j in u:
        torch.manual_seed(100 + j)
        a, b = D.functional.get_unique_connections(int(u["dims_%d" % j][0]), int(u["dims_%d" % j][1]), 'cpu')
        assert np.array_equal(a.numpy(), u["a_%d" % j]) and np.array_equal(b.numpy(), u["b_%d" % j])
        j += 1
    assert j == 6


def test_random_connections_use_the_reference_rng_order(golden_dir):
    g = np.load(os.path.join(golden_dir, "small_net.npz"))
    torch.manual_seed(int(g["seed"]))
    dims = [int(v) for v in g["dims"]]
    for i, (n_in, n_out) in enumerate(zip(dims[:-1], dims[1:])):
        layer = D.LogicLayer(n_in, n_out, device='cpu')
        assert torch.equal(layer.weights.detach(), torch.tensor(g["w0_%d" % i]))
        assert np.array_equal(layer.indices[0].numpy(), g["a_%d" % i])
        assert np.array_equal(layer.indices[1].numpy(), g["b_%d" % i])


def test_gates_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "gates.npz"))
    a, b, w = (torch.tensor(g[k]) for k in ("a", "b", "w"))
    for i in range(16):
        assert torch.equal(D.functional.bin_op(a, b, i), torch.tensor(g["gates"][i]))
    assert torch.equal(D.functional.bin_op_s(a, b, w), torch.tensor(g["mix"]))


def test_packet_inbox_plan_gives_every_bucket_its_own_slots():
    """plan_inboxes: a bucket's slots hold the largest slice any rank owns, regions of different buckets do not overlap,
    and every float4 of a bucket maps to exactly one (owner, slot) -- the addressing of exchange_packets_kernel."""
    from difflogic_b200.optim import plan_inboxes
    for world in (1, 2, 3, 4, 8):
        counts = [16000 * 16, 4 * 1237, 4, 64, 4 * 999]
        offsets, stride = plan_inboxes(counts, world)
        assert offsets[0] == 0 and len(offsets) == len(counts)
        end = 0
        for count, off in zip(counts, offsets):
            n4 = count // 4
            per = -(-n4 // world)
            assert off >= end                      # behind the bucket before it
            end = off + per
            seen = set()
            for i in range(0, n4, max(1, n4 // 97)):           # a sample of the bucket's float4
                owner, k = i // per, i % per
                assert owner < world and off + k < end
                seen.add((owner, k))
            assert len(seen) == len(range(0, n4, max(1, n4 // 97)))
        assert stride >= end
    assert plan_inboxes([], 4) == ([], 1)
