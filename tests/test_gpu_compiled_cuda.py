"""CompiledLogicNet(device='cuda'): the frozen network on the packed-bit kernels against the C build of the same
network and against the oracle.  Needs a B200; every test is marked gpu."""
import numpy as np
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import build_model

pytestmark = pytest.mark.gpu

pytest.importorskip("difflogic_b200.ops")
import difflogic_b200 as D  # noqa: E402


@pytest.mark.parametrize("num_bits", [8, 64])
@pytest.mark.parametrize("case", [([30, 64, 40], 4, 37), ([100, 640, 640, 800], 10, 5100)])
def test_compiled_cuda_equals_compiled_c_and_oracle(case, num_bits):
    dims, k, batch = case
    torch.manual_seed(sum(dims))
    net = O.OracleNet.build(dims, k, 1.0)
    model = build_model(dims, k, 1.0, net.weights, net.idx_a, net.idx_b)
    model.eval()
    x = torch.rand(batch, dims[0]) < 0.4
    ref = O.packed_net_counts(x.numpy(), net.idx_a, net.idx_b, net.gate_ids(), k, 64)

    on_gpu = D.CompiledLogicNet(model, device='cuda', num_bits=num_bits)
    on_gpu.compile()
    got = on_gpu(x)                       # CPU in -> CPU out
    assert not got.is_cuda and got.dtype == torch.int32 and np.array_equal(got.numpy(), ref)
    got_dev = on_gpu(x.cuda())            # GPU in -> GPU out
    assert got_dev.is_cuda and torch.equal(got_dev.cpu(), got)
    assert np.array_equal(on_gpu(x.numpy()).numpy(), ref)   # numpy in

    on_cpu = D.CompiledLogicNet(model, device='cpu', num_bits=num_bits)
    on_cpu.compile(opt_level=0)
    assert torch.equal(on_cpu(x), got)


def test_compiled_cuda_is_a_snapshot_of_the_weights():
    torch.manual_seed(3)
    model = torch.nn.Sequential(D.LogicLayer(16, 64, device='cuda'), D.LogicLayer(64, 64, device='cuda'), D.GroupSum(2))
    model.eval()
    x = torch.rand(100, 16) < 0.5
    frozen = D.CompiledLogicNet(model, device='cuda')
    frozen.compile()
    before = frozen(x)
    with torch.no_grad():
        for layer in model:
            if isinstance(layer, D.LogicLayer):
                layer.weights.copy_(torch.randn_like(layer.weights))
    assert torch.equal(frozen(x), before)            # compile() froze the gates
    with torch.no_grad():
        live = model(D.PackBitsTensor(x.cuda()))
    assert live.shape == before.shape
