"""GroupSum + cross-entropy as one autograd node against the two modules one after the other.
Needs a B200; every test is marked gpu."""
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import build_model, logic_layers

pytestmark = pytest.mark.gpu

pytest.importorskip("difflogic_b200.ops")
import difflogic_b200 as D  # noqa: E402
from difflogic_b200 import _native as N  # noqa: E402
from difflogic_b200.losses import CrossEntropyLoss, group_sum_cross_entropy  # noqa: E402
from difflogic_b200.optim import FlatAdam  # noqa: E402
from difflogic_b200.training import TrainStep  # noqa: E402


@pytest.mark.parametrize("shape", [(128, 16000, 10, 30.0), (37, 640, 10, 1.0), (5, 96, 3, 2.5), (260, 4096, 1, 10.0), (64, 200, 100, 1.0)])
def test_head_is_bit_identical_to_groupsum_then_cross_entropy(shape):
    batch, n, k, tau = shape
    g = torch.Generator().manual_seed(batch + n)
    x = torch.rand(batch, n, generator=g).cuda()
    y = torch.randint(0, k, (batch,), generator=g).cuda()
    up = torch.rand((), generator=g).cuda() + 0.5          # a gradient that is not 1

    xa = x.clone().requires_grad_(True)
    scores = D.GroupSum(k, tau)(xa)
    loss_a = CrossEntropyLoss()(scores, y)
    loss_a.backward(gradient=up)

    xb = x.clone().requires_grad_(True)
    loss_b, scores_b = group_sum_cross_entropy(xb, y, k, tau)
    assert not scores_b.requires_grad
    loss_b.backward(gradient=up)

    assert torch.equal(loss_a, loss_b) and torch.equal(scores.detach(), scores_b)
    assert torch.equal(xa.grad, xb.grad)
    # and close to torch's own loss
    xt = x.clone().requires_grad_(True)
    lt = torch.nn.functional.cross_entropy(xt.reshape(batch, k, n // k).sum(-1) / tau, y)
    lt.backward(gradient=up)
    torch.testing.assert_close(loss_b, lt, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(xb.grad, xt.grad, rtol=1e-4, atol=1e-9)


def test_head_rejects_what_it_cannot_do():
    x = torch.rand(8, 30, device='cuda')
    y = torch.zeros(8, dtype=torch.int64, device='cuda')
    with pytest.raises(ValueError):
        group_sum_cross_entropy(x, y, 4, 1.0)                      # 30 % 4 != 0
    with pytest.raises(ValueError):
        group_sum_cross_entropy(x.double(), y, 3, 1.0)
    with pytest.raises(ValueError):
        group_sum_cross_entropy(x, y.int(), 3, 1.0)


@pytest.mark.parametrize("loss_cls", [CrossEntropyLoss, torch.nn.CrossEntropyLoss])
def test_train_step_with_fused_head_equals_unfused(loss_cls):
    torch.manual_seed(5)
    dims = [40, 96, 96, 60]
    net = O.OracleNet.build(dims, 6, 4.0)
    x = (torch.rand(48, 40) < 0.4).float().cuda()
    y = torch.randint(0, 6, (48,)).cuda()
    results = []
    for fuse in (False, True):
        model = build_model(dims, 6, 4.0, net.weights, net.idx_a, net.idx_b)
        step = TrainStep(model, FlatAdam(model.parameters(), lr=0.01), loss_cls(), fuse_head=fuse)
        assert (step._head is not None) == fuse
        before = N.launch_count()
        losses = [step(x, y).clone() for _ in range(4)]
        launches = N.launch_count() - before
        results.append((losses, [l.weights.detach().clone() for l in logic_layers(model)], launches))
    (la, wa, na), (lb, wb, nb) = results
    if loss_cls is CrossEntropyLoss:
        # same kernels' arithmetic in the same order: identical to the bit
        assert all(torch.equal(p, q) for p, q in zip(la, lb))
        assert all(torch.equal(p, q) for p, q in zip(wa, wb))
        assert nb == na - 4          # one library launch less per step (loss backward and GroupSum backward are one)
    else:
        # unfused, torch computes the loss itself: equal up to its rounding
        for p, q in zip(la, lb):
            torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)
        for p, q in zip(wa, wb):
            torch.testing.assert_close(p, q, rtol=1e-3, atol=1e-4)


def test_label_smoothing_is_not_fused():
    model = torch.nn.Sequential(D.LogicLayer(8, 16, device='cuda'), D.GroupSum(2))
    step = TrainStep(model, torch.optim.Adam(model.parameters()), torch.nn.CrossEntropyLoss(label_smoothing=0.1))
    assert step._head is None
    step = TrainStep(model, torch.optim.Adam(model.parameters()), torch.nn.MSELoss())
    assert step._head is None
