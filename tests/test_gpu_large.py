"""Full-size shapes of the benchmark configurations, checked through size-independent properties: a sample's
output depends only on that sample's input column, so any slice of a large batch must equal a small run on the
same columns.  Exercises 64-bit offsets (tensors beyond 2^31 elements / 2^32 bytes) and the wide layers of the
image- and tabular-shaped configurations.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import logic_oracle as O
from tests.helpers import assert_forward_close, assert_grad_close

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("difflogic_b200.ops")


def _random_connections(n_in, n_out, seed):
    g = torch.Generator().manual_seed(seed)
    c = torch.randperm(2 * n_out, generator=g) % n_in
    c = torch.randperm(n_in, generator=g)[c].reshape(2, n_out)
    return c[0].contiguous(), c[1].contiguous()


def test_wide_image_shaped_layer_against_oracle():
    """9216 -> 128000 (first layer of the 32x32x3 thermometer configuration), batch 48."""
    n_in, n_out, batch = 9216, 128000, 48
    a, b = _random_connections(n_in, n_out, 1)
    g = torch.Generator().manual_seed(2)
    w = torch.randn(n_out, 16, generator=g)
    x = (torch.rand(batch, n_in, generator=g) < 0.5).float()
    gy = torch.randn(batch, n_out, generator=g)
    wr = w.clone().requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    ref = O.layer_forward(xr, a, b, wr, training=True)
    ref.backward(gy)
    ad, bd, wd, xd, gyd = a.cuda(), b.cuda(), w.cuda(), x.T.contiguous().cuda(), gy.T.contiguous().cuda()
    y, coef = ops.logic_forward(xd, ad, bd, wd, ops.W_LOGITS, want_coef=True)
    assert_forward_close(y.T, ref, "wide forward")
    assert_grad_close(ops.logic_backward_w(xd, ad, bd, gyd, wd, ops.W_LOGITS), wr.grad, "wide backward_w")
    start, lst = ops.inverse_index(ad, bd, n_in)
    plan = ops.build_backward_plan(ad, bd, start, lst)
    assert int((start[1:] - start[:-1]).max()) <= 28  # 'random' connections are balanced: fan-out 27 or 28
    assert_grad_close(ops.logic_backward_x(xd, coef, gyd, start, plan, 1.0).T, xr.grad, "wide backward_x")


def test_training_kernels_beyond_2_to_31_elements():
    """64000 x 36000 fp32 activations (2.3e9 elements, 9.2 GB each): slices equal a small run."""
    n, batch, small = 64000, 36000, 96
    a, b = _random_connections(n, n, 3)
    ad, bd = a.cuda(), b.cuda()
    w = torch.randn(n, 16, device="cuda")
    x = torch.rand(n, batch, device="cuda")
    y, coef = ops.logic_forward(x, ad, bd, w, ops.W_LOGITS, want_coef=True)
    cols = torch.cat([torch.arange(0, small // 2), torch.arange(batch - small // 2, batch)]).cuda()
    xs = x[:, cols].contiguous()
    ys, _ = ops.logic_forward(xs, ad, bd, w, ops.W_LOGITS)
    assert torch.equal(y[:, cols], ys)
    gy = torch.randn(n, batch, device="cuda")
    start, lst = ops.inverse_index(ad, bd, n)
    plan = ops.build_backward_plan(ad, bd, start, lst)
    gx = ops.logic_backward_x(x, coef, gy, start, plan, 2.0)
    gxs = ops.logic_backward_x(xs, coef, gy[:, cols].contiguous(), start, plan, 2.0)
    assert torch.equal(gx[:, cols], gxs)
    del gx, y
    # backward_w sums over the batch: compare with the sum of two halves (different summation order -> tolerance)
    gw = ops.logic_backward_w(x, ad, bd, gy, w, ops.W_PROBS)
    half = batch // 2
    gw2 = ops.logic_backward_w(x[:, :half].contiguous(), ad, bd, gy[:, :half].contiguous(), None, ops.W_PROBS) + \
        ops.logic_backward_w(x[:, half:].contiguous(), ad, bd, gy[:, half:].contiguous(), None, ops.W_PROBS)
    assert_grad_close(gw, gw2, "backward_w halves")


def test_packed_eval_beyond_2_to_32_bytes():
    """64000 rows x 2^18 samples... scaled: 64000 rows x 40960 int64 words = 21 GB per activation."""
    n, words = 64000, 40960
    a, b = _random_connections(n, n, 5)
    ad, bd = a.cuda(), b.cuda()
    gate = torch.randint(0, 16, (n,), dtype=torch.uint8, device="cuda")
    x = torch.randint(-2 ** 62, 2 ** 62, (n, words), dtype=torch.int64, device="cuda")
    y = ops.eval_packed(x, ad, bd, gate)
    cols = torch.cat([torch.arange(0, 8), torch.arange(20000, 20008), torch.arange(words - 16, words)]).cuda()
    ys = O.eval_packed(x[:, cols].cpu().numpy(), a.numpy(), b.numpy(), gate.cpu().numpy())
    assert np.array_equal(y[:, cols].cpu().numpy(), ys)
    counts = ops.groupbitsum(y, 0, 2)
    # checksum of checksums: every sample's two class counts add up to the popcount over all rows of that sample
    sub = y[:, cols].cpu().numpy()
    ref_counts = O.group_bit_sum(sub, 0, 2)
    got = counts.view(words, 64, 2)[cols.cpu()].reshape(-1, 2).cpu().numpy()
    assert np.array_equal(got, ref_counts)
    from difflogic_b200 import _native as N
    assert N.lib().dl_async_error() == 0


def test_deep_tabular_net_trains_and_packs():
    """256 -> 12 x 64000 with grad_factor 2 (the deep tabular-shaped configuration) at a reduced batch: the step
    runs, gradients are finite everywhere, and packed eval agrees with float eval."""
    import difflogic_b200 as D
    torch.manual_seed(7)
    layers = [torch.nn.Flatten(), D.LogicLayer(256, 64000, grad_factor=2.0)]
    layers += [D.LogicLayer(64000, 64000, grad_factor=2.0) for _ in range(11)]
    model = torch.nn.Sequential(*layers, D.GroupSum(2, 20.0))
    x = (torch.rand(256, 256, device="cuda") < 0.5)
    y = torch.randint(0, 2, (256,), device="cuda")
    model.train()
    loss = torch.nn.functional.cross_entropy(model(x.float()), y)
    loss.backward()
    for l in layers[1:]:
        assert torch.isfinite(l.weights.grad).all() and float(l.weights.grad.abs().max()) > 0
    model.eval()
    with torch.no_grad():
        fl = model(x.float())
        counts = model(D.PackBitsTensor(x, bit_count=64))
    assert torch.equal(torch.round(fl * 20.0).to(torch.int32), counts)


def test_packed_inference_at_the_benchmark_size_is_bit_exact():
    """784 -> 4 x 8000 -> GroupSum(10) on 2^20 samples in int64 words (the packed benchmark, staged kernels, last layer
    fused with the class count): every one of the 2^20 x 10 counts equals the C oracle's."""
    import difflogic_b200 as D
    from tests.helpers import build_model
    torch.manual_seed(0)
    dims, k = [784] + [8000] * 4, 10
    net = O.OracleNet.build(dims, k, 10.0)
    model = build_model(dims, k, 10.0, net.weights, net.idx_a, net.idx_b)
    model.eval()
    samples = 1 << 20
    g = torch.Generator().manual_seed(11)
    x = torch.empty(samples, dims[0], dtype=torch.bool)
    for s in range(0, samples, 1 << 16):
        x[s:s + (1 << 16)] = torch.rand(1 << 16, dims[0], generator=g) < 0.19
    with torch.no_grad():
        counts = model(D.PackBitsTensor(x.cuda(), bit_count=64))
    ref = O.c_packed_net_counts(x.numpy(), net.idx_a, net.idx_b, net.gate_ids(), k, threads=torch.get_num_threads())
    assert counts.shape == (samples, k)
    assert np.array_equal(counts.cpu().numpy(), np.asarray(ref))
    from difflogic_b200 import _native as N
    assert N.lib().dl_async_error() == 0


def test_captured_training_step_at_the_benchmark_size_against_oracle():
    """784 -> 5 x 16000 -> GroupSum(10, tau=30), batch 128, through a CUDA-graph-captured TrainStep (fused head, Adam
    inside backward_w): loss, weight gradients (read back from Adam's first moments of the first step) and updated
    weights against the oracle's step."""
    from difflogic_b200.optim import FlatAdam
    from difflogic_b200.training import TrainStep
    from tests.helpers import build_model, logic_layers
    torch.manual_seed(0)
    dims, k, tau, batch, lr = [784] + [16000] * 5, 10, 30.0, 128, 0.01
    net = O.OracleNet.build(dims, k, tau)
    model = build_model(dims, k, tau, net.weights, net.idx_a, net.idx_b)
    model.train()
    g = torch.Generator().manual_seed(21)
    x = (torch.rand(batch, dims[0], generator=g) < 0.19).float()
    y = torch.randint(0, k, (batch,), generator=g)
    opt = FlatAdam(model.parameters(), lr=lr)
    step = TrainStep(model, opt, torch.nn.CrossEntropyLoss())
    step.capture(x.cuda(), y.cuda(), warmup=0)          # nothing runs before the first replay
    loss = step(x.cuda(), y.cuda())
    torch.cuda.synchronize()
    start = [w.detach().clone() for w in net.weights]
    ref_loss, _, ref_grads = net.train_step(x, y, lr=lr)
    assert abs(float(loss) - float(ref_loss)) <= 1e-5 * abs(float(ref_loss))
    for p, ref in zip(opt._params, ref_grads):
        off, cnt = opt._slices[p]
        assert_grad_close((opt.exp_avg[off:off + cnt] / 0.1).view_as(p), ref, "weight gradient via the first moment")
    for layer, w0, gr in zip(logic_layers(model), start, ref_grads):
        want = w0 - lr * gr / (gr.abs() + 1e-8)          # first Adam step from zero moments
        sure = gr.abs() > 1e-3 * gr.abs().max()          # where the sign of the gradient is beyond doubt
        assert float((layer.weights.detach().cpu() - want)[sure].abs().max()) <= 2e-3 * lr
    step.close()
