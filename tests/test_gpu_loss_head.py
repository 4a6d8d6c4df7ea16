"""GroupSum + cross-entropy as one autograd node against the two modules one after the other.
Needs a B200; every test is marked gpu."""
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import assert_grad_close, build_model, logic_layers

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


# ---- last layer + GroupSum + loss as one autograd node (class-row gradients) -------------------------------------

from difflogic_b200 import ops  # noqa: E402
from difflogic_b200.difflogic import logic_layer_head  # noqa: E402
from tests.helpers import random_layer  # noqa: E402


@pytest.mark.parametrize("shape", [(16000, 128, 10, 30.0), (640, 37, 10, 1.0), (4096, 260, 1, 10.0), (6400, 64, 100, 1.0),
                                   (1280, 1000, 5, 2.0)])
def test_head_kernel_matches_the_separate_kernels(shape):
    n, batch, k, tau = shape
    g = torch.Generator().manual_seed(n + batch)
    x = torch.rand(n, batch, generator=g).cuda()                     # feature-major
    y = torch.randint(0, k, (batch,), generator=g).cuda()
    assert ops.groupsum_cross_entropy_applicable(n, batch, k)
    for _ in range(2):                                               # the ticket counter is left at zero
        loss, scores, grad_classes = ops.groupsum_cross_entropy(x, y, k, tau)
    ref_scores = ops.groupsum(x, k, tau)
    assert torch.equal(scores, ref_scores)
    ref_loss = torch.nn.functional.cross_entropy(ref_scores, y)
    torch.testing.assert_close(loss, ref_loss, rtol=1e-5, atol=1e-6)
    # gradient rows: the separate kernels' [n, batch] gradient has equal rows within a class
    sc = ref_scores.clone().requires_grad_(True)
    CrossEntropyLoss()(sc, y).backward()
    expanded = ops.groupsum_backward(sc.grad.contiguous(), n, tau)
    m = n // k
    assert torch.equal(expanded, grad_classes.repeat_interleave(m, dim=0))


def test_head_kernel_range():
    assert not ops.groupsum_cross_entropy_applicable(630, 16, 10)     # 63 rows per class
    assert not ops.groupsum_cross_entropy_applicable(50000, 16, 10)   # 5000 rows per class
    assert not ops.groupsum_cross_entropy_applicable(641, 16, 10)
    x = torch.rand(630, 16, device='cuda')
    y = torch.zeros(16, dtype=torch.int64, device='cuda')
    with pytest.raises(RuntimeError, match="outside"):
        ops.groupsum_cross_entropy(x, y, 10, 1.0)


@pytest.mark.parametrize("shape", [(300, 1000, 128, 100), (33, 60, 100, 20), (50, 64, 7, 64), (12, 24, 516, 3)])
def test_backward_kernels_with_one_gradient_row_per_class(shape):
    n_in, n_out, batch, m = shape
    a, b, w = random_layer(n_in, n_out, seed=sum(shape), force_same_input=True)
    g = torch.Generator().manual_seed(7)
    x = torch.rand(n_in, batch, generator=g).cuda()
    gc = torch.randn(n_out // m, batch, generator=g).cuda()
    gy = gc.repeat_interleave(m, dim=0).contiguous()
    a, b, w = a.cuda(), b.cuda(), w.cuda()
    start, lst = ops.inverse_index(a, b, n_in)
    plan = ops.build_backward_plan(a, b, start, lst)
    _, coef = ops.logic_forward(x, a, b, w, ops.W_LOGITS, True)
    assert torch.equal(ops.logic_backward_w(x, a, b, gc, w, ops.W_LOGITS, rows_per_class=m),
                       ops.logic_backward_w(x, a, b, gy, w, ops.W_LOGITS))
    assert torch.equal(ops.logic_backward_x(x, coef, gc, start, plan, 1.5, rows_per_class=m),
                       ops.logic_backward_x(x, coef, gy, start, plan, 1.5))
    with pytest.raises(RuntimeError):
        ops.logic_backward_w(x[:, :4].contiguous(), a, b, gc, w, ops.W_LOGITS, rows_per_class=m)  # batch mismatch is caught


@pytest.mark.parametrize("unit", [True, False])
def test_last_layer_head_node_equals_the_three_modules(unit):
    torch.manual_seed(3)
    layer_a = D.LogicLayer(50, 640, device='cuda', grad_factor=1.3)
    layer_b = D.LogicLayer(50, 640, device='cuda', grad_factor=1.3)
    layer_b.set_connections(*layer_a.indices)
    with torch.no_grad():
        layer_b.weights.copy_(layer_a.weights)
    x = torch.rand(48, 50, device='cuda')
    y = torch.randint(0, 10, (48,), device='cuda')
    up = torch.ones((), device='cuda') if unit else torch.full((), 0.37, device='cuda')
    if unit:
        up._dl_is_one = True

    xa = x.clone().requires_grad_(True)
    loss_a = CrossEntropyLoss()(D.GroupSum(10, 3.0)(layer_a(xa)), y)
    loss_a.backward(gradient=up)

    xb = x.clone().requires_grad_(True)
    before = N.launch_count()
    loss_b, scores = logic_layer_head(layer_b, xb, y, 10, 3.0)
    loss_b.backward(gradient=up)
    assert N.launch_count() - before == 4            # forward, head, backward_w, backward_x
    torch.testing.assert_close(loss_a, loss_b, rtol=1e-6, atol=1e-7)
    # the head adds a class's rows in another order than GroupSum does: equal up to that rounding
    assert_grad_close(xb.grad, xa.grad, "grad_x", rtol=1e-5)
    assert_grad_close(layer_b.weights.grad, layer_a.weights.grad, "grad_w", rtol=1e-5)
    assert scores.shape == (48, 10) and not scores.requires_grad


@pytest.mark.parametrize("captured", [False, True])
def test_train_step_with_last_layer_head(captured):
    torch.manual_seed(5)
    dims = [40, 96, 128, 640]
    net = O.OracleNet.build(dims, 10, 4.0)
    g = torch.Generator().manual_seed(2)
    xs = [(torch.rand(48, 40, generator=g) < 0.4).float().cuda() for _ in range(5)]
    ys = [torch.randint(0, 10, (48,), generator=g).cuda() for _ in range(5)]
    results = []
    for fuse in (False, True):
        model = build_model(dims, 10, 4.0, net.weights, net.idx_a, net.idx_b)
        step = TrainStep(model, FlatAdam(model.parameters(), lr=0.01), CrossEntropyLoss(), fuse_head=fuse)
        assert (step._last is not None) == fuse
        if captured:
            step.capture(xs[0], ys[0], warmup=2)
        before = N.launch_count()
        losses = [step(x, y).clone() for x, y in zip(xs, ys)]
        launches = N.launch_count() - before
        torch.cuda.synchronize()
        results.append((losses, [l.weights.detach().clone() for l in logic_layers(model)], launches))
        step.close()
    (la, wa, na), (lb, wb, nb) = results
    for p, q in zip(la, lb):
        torch.testing.assert_close(p, q, rtol=1e-6, atol=1e-7)
    # The head adds a class's rows in another order than GroupSum does, so the gradients differ in the last bits;
    # after five Adam steps that shows only where a gradient is so close to zero that its sign is rounding noise.
    for p, q in zip(wa, wb):
        diff = (p - q).abs()
        assert float(diff.max()) <= 5 * 0.01 * 1.01 and float((diff > 1e-5).float().mean()) < 2e-3
    if not captured:
        assert nb == na - 5 * 3      # per step: GroupSum + loss -> 1 kernel, loss backward + GroupSum backward -> 0


# ---- the Adam step inside backward_w -------------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(300, 1000, 128, 1), (33, 60, 100, 20), (16, 40, 7, 1), (12, 24, 516, 3)])
def test_backward_w_with_adam_epilogue_equals_backward_w_then_adam(shape):
    n_in, n_out, batch, m = shape
    a, b, w = random_layer(n_in, n_out, seed=sum(shape), force_same_input=True)
    g = torch.Generator().manual_seed(11)
    x = torch.rand(n_in, batch, generator=g).cuda()
    gy = torch.randn(n_out // m, batch, generator=g).cuda()
    a, b = a.cuda(), b.cuda()
    hp = dict(lr=0.01, beta1=0.9, beta2=0.999, eps=1e-8)
    # reference: backward_w, then the flat Adam kernel
    w1 = torch.nn.Parameter(w.clone().cuda())
    opt = FlatAdam([w1], lr=hp["lr"])
    # fused: same start
    w2 = w.clone().cuda()
    m2 = torch.zeros(n_out * 16, device='cuda')
    v2 = torch.zeros(n_out * 16, device='cuda')
    state = torch.zeros(2, dtype=torch.int32, device='cuda')
    for _ in range(3):
        w1.grad = ops.logic_backward_w(x, a, b, gy, w1.data, ops.W_LOGITS, rows_per_class=m)
        opt.step()
        got = ops.logic_backward_w_adam(x, a, b, gy, w2, m2, v2, state, grad_scale=1.0, grad_out=torch.empty_like(w2),
                                        rows_per_class=m, **hp)
    assert state.tolist() == [3, 0] and int(opt.state_t[0].item()) == 3
    assert torch.equal(w1.data, w2)
    assert torch.equal(opt.exp_avg[:n_out * 16], m2) and torch.equal(opt.exp_avg_sq[:n_out * 16], v2)
    assert got.shape == (n_out, 16)
    # without grad_out nothing but the update happens
    assert ops.logic_backward_w_adam(x, a, b, gy, w2, m2, v2, state, rows_per_class=m, **hp) is None


@pytest.mark.parametrize("captured", [False, True])
def test_train_step_with_adam_inside_backward(captured):
    torch.manual_seed(5)
    dims = [40, 96, 128, 640]
    net = O.OracleNet.build(dims, 10, 4.0)
    g = torch.Generator().manual_seed(2)
    xs = [(torch.rand(48, 40, generator=g) < 0.4).float().cuda() for _ in range(5)]
    ys = [torch.randint(0, 10, (48,), generator=g).cuda() for _ in range(5)]
    results = []
    for inside in (False, True):
        model = build_model(dims, 10, 4.0, net.weights, net.idx_a, net.idx_b)
        opt = FlatAdam(model.parameters(), lr=0.01)
        step = TrainStep(model, opt, CrossEntropyLoss(), step_in_backward=inside)
        assert step._in_backward == inside
        if captured:
            step.capture(xs[0], ys[0], warmup=2)
        losses = [step(x, y).clone() for x, y in zip(xs, ys)]
        torch.cuda.synchronize()
        weights_after = [l.weights.detach().clone() for l in logic_layers(model)]
        moments = (opt.exp_avg.clone(), opt.exp_avg_sq.clone())
        # outside a step the model behaves as usual: backward fills .grad and does not touch the weights
        before = [l.weights.detach().clone() for l in logic_layers(model)]
        model.train()
        torch.nn.functional.cross_entropy(model(xs[0]), ys[0]).backward()
        assert all(l.weights.grad is not None for l in logic_layers(model))
        assert all(torch.equal(p, l.weights.detach()) for p, l in zip(before, logic_layers(model)))
        step.close()                                   # hands the step count back to optimizer.step()
        results.append((losses, weights_after, int(opt.state_t[0].item()), moments[0], moments[1]))
    (la, wa, ca, ma, va), (lb, wb, cb, mb, vb) = results
    assert ca == cb == (7 if captured else 5)
    assert all(torch.equal(p, q) for p, q in zip(la, lb))
    assert all(torch.equal(p, q) for p, q in zip(wa, wb))
    assert torch.equal(ma, mb) and torch.equal(va, vb)


def test_resident_batches_replay_without_copies():
    """capture_resident: one graph per batch that reads the batch where it lies; the same steps as eager ones."""
    torch.manual_seed(8)
    dims = [40, 96, 128, 640]
    net = O.OracleNet.build(dims, 10, 4.0)
    g = torch.Generator().manual_seed(4)
    xs = [(torch.rand(48, 40, generator=g) < 0.4).float().cuda() for _ in range(3)]
    ys = [torch.randint(0, 10, (48,), generator=g).cuda() for _ in range(3)]
    results = []
    for resident in (False, True):
        model = build_model(dims, 10, 4.0, net.weights, net.idx_a, net.idx_b)
        step = TrainStep(model, FlatAdam(model.parameters(), lr=0.01), CrossEntropyLoss())
        if resident:
            step.capture(xs[0], ys[0], warmup=0)
            assert step.capture_resident(xs, ys) == 3
            losses = [step.replay_resident(i).clone() for i in (0, 1, 2, 1)]
        else:
            losses = [step(xs[i], ys[i]).clone() for i in (0, 1, 2, 1)]
        torch.cuda.synchronize()
        results.append((losses, [l.weights.detach().clone() for l in logic_layers(model)]))
        step.close()
    (la, wa), (lb, wb) = results
    assert all(torch.equal(p, q) for p, q in zip(la, lb))
    assert all(torch.equal(p, q) for p, q in zip(wa, wb))

